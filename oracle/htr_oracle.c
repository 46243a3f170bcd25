/*
 * CPU oracle for the HTR-W1 packed-linear decode path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the algorithm of the reference's CPU decoder
 * (htr/wire.py) followed by the dense contraction the reference performs on the
 * decoded matrix (htr/ops.py:93, F.linear).  Only the test-suite, the smoke check
 * and the CPU-baseline leg of the benchmark may call it; the product library never
 * links or loads it.
 *
 * Parity pin: every function below is checked against outputs of the reference's
 * own htr/wire.py (imported and executed when the golden fixtures were generated,
 * see tests/golden/make_golden.py) and against the vectors of the reference's
 * tests/test_release.py (bit layout :28-38, sign byte 170 :40-43, Hadamard :45-47,
 * encoder round trip :53-73).
 *
 * Conventions (docs/FORMAT.md:16-32):
 *   tile   = 16 output rows x 16 input cols, 8K uint32 words, MSB-first circular stream
 *   step t = 16*r + c inside a tile; state s_t = the 16 stream bits ending at bit (t+1)K-1
 *   v(s)   = bytesum((s*0xDF6ADF + 0x34983) mod 2^32) - 510
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define HTRO_STATES 65536u
#define HTRO_MUL 0xDF6ADFu
#define HTRO_ADD 0x34983u

/* ---- codebook: htr/wire.py:10-13 (gen_values) ------------------------------------ */
int htro_gen_value(uint32_t s) {
  uint32_t x = s * HTRO_MUL + HTRO_ADD; /* uint32 wrap == "& 0xFFFFFFFF" */
  return (int)((x & 255u) + ((x >> 8) & 255u) + ((x >> 16) & 255u) + (x >> 24)) - 510;
}

void htro_gen_values(const uint32_t *states, int16_t *out, size_t count) {
  for (size_t i = 0; i < count; ++i) out[i] = (int16_t)htro_gen_value(states[i] & 0xFFFFu);
}

/* 1/sqrt(mean v^2) over all 65536 states in float64: htr/wire.py:27-30 (cbscale) */
double htro_cbscale(void) {
  double acc = 0.0;
  for (uint32_t s = 0; s < HTRO_STATES; ++s) {
    double v = (double)htro_gen_value(s);
    acc += v * v;
  }
  return 1.0 / sqrt(acc / (double)HTRO_STATES);
}

/* cb[s] = float32(v / rms64): htr/wire.py:19-24 (codebook_f32) */
void htro_codebook_f32(float *cb) {
  double acc = 0.0;
  for (uint32_t s = 0; s < HTRO_STATES; ++s) {
    double v = (double)htro_gen_value(s);
    acc += v * v;
  }
  double rms = sqrt(acc / (double)HTRO_STATES);
  for (uint32_t s = 0; s < HTRO_STATES; ++s) cb[s] = (float)((double)htro_gen_value(s) / rms);
}

/* ---- bit stream: htr/wire.py:46-63 (stream_bits, unpack_states) ------------------- */
static inline unsigned stream_bit(const uint32_t *words, unsigned p) {
  return (words[p >> 5] >> (31u - (p & 31u))) & 1u;
}

/* words [ntiles, 8K] -> states [ntiles, 256]; deliberately bit-by-bit (no funnel shifts) */
int htro_unpack_states(const uint32_t *words, int K, size_t ntiles, uint16_t *states) {
  if (K < 2 || K > 8) return -1;
  const unsigned nbits = 256u * (unsigned)K;
  for (size_t b = 0; b < ntiles; ++b) {
    const uint32_t *w = words + b * (size_t)(8 * K);
    for (unsigned t = 0; t < 256u; ++t) {
      unsigned first = ((t + 1u) * (unsigned)K + nbits - 16u) % nbits;
      unsigned s = 0;
      for (unsigned j = 0; j < 16u; ++j) s = (s << 1) | stream_bit(w, (first + j) % nbits);
      states[b * 256 + t] = (uint16_t)s;
    }
  }
  return 0;
}

/* states [ntiles,256] -> words [ntiles,8K]: htr/wire.py:33-43 (pack_states): the low K bits
 * of each state are the step's new bits, MSB first */
int htro_pack_states(const uint16_t *states, int K, size_t ntiles, uint32_t *words) {
  if (K < 2 || K > 8) return -1;
  for (size_t b = 0; b < ntiles; ++b) {
    uint32_t *w = words + b * (size_t)(8 * K);
    memset(w, 0, sizeof(uint32_t) * (size_t)(8 * K));
    for (unsigned t = 0; t < 256u; ++t) {
      unsigned nb = states[b * 256 + t] & ((1u << K) - 1u);
      for (int j = 0; j < K; ++j) {
        unsigned bit = (nb >> (K - 1 - j)) & 1u;
        unsigned p = t * (unsigned)K + (unsigned)j;
        w[p >> 5] |= bit << (31u - (p & 31u));
      }
    }
  }
  return 0;
}

/* int16 v(s_t) per tile in stream order; the "bitwise oracle hook" contract of
 * htr/csrc/htr_kernels.cu:153-172 (k_decode_raw) expressed through wire.py */
int htro_decode_raw(const uint32_t *words, int K, size_t ntiles, int16_t *out) {
  uint16_t st[256];
  for (size_t b = 0; b < ntiles; ++b) {
    if (htro_unpack_states(words + b * (size_t)(8 * K), K, 1, st)) return -1;
    for (int t = 0; t < 256; ++t) out[b * 256 + t] = (int16_t)htro_gen_value(st[t]);
  }
  return 0;
}

/* ---- signs: htr/wire.py:66-74 (LSB-first, bit set = -1) --------------------------- */
void htro_unpack_signs(const uint8_t *packed, size_t n, float *out) {
  for (size_t j = 0; j < n; ++j) out[j] = ((packed[j >> 3] >> (j & 7u)) & 1u) ? -1.0f : 1.0f;
}

void htro_pack_signs(const float *signs, size_t n, uint8_t *packed) {
  memset(packed, 0, n / 8);
  for (size_t j = 0; j < n; ++j)
    if (signs[j] < 0.0f) packed[j >> 3] |= (uint8_t)(1u << (j & 7u));
}

/* ---- Hadamard: htr/wire.py:80-87 (Sylvester H128 / sqrt(128), float64 then float32) - */
void htro_hadamard128(float *h) {
  const double r = 1.0 / sqrt(128.0);
  for (unsigned a = 0; a < 128u; ++a)
    for (unsigned b = 0; b < 128u; ++b) h[a * 128 + b] = (float)((__builtin_popcount(a & b) & 1) ? -r : r);
}

/* IEEE binary16 -> float (scales are stored as float16, docs/FORMAT.md:27) */
float htro_half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 31u, m = h & 1023u, bits;
  if (e == 0) {
    if (m == 0) bits = sign;
    else {
      int sh = 0;
      while (!(m & 1024u)) { m <<= 1; ++sh; }
      bits = sign | ((uint32_t)(113 - sh) << 23) | ((m & 1023u) << 13);
    }
  } else if (e == 31u) bits = sign | 0x7F800000u | (m << 13);
  else bits = sign | ((e + 112u) << 23) | (m << 13);
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* ---- rotated-domain Q rows: htr/wire.py:95-102 (dequant_Q) ------------------------ */
/* Q[16ti+r, 16tj+c] = cb[s_{16r+c}] * float32(scales[16ti+r]) for strips ti in [ti0, ti1) */
static void dequant_q_rows(const uint32_t *qw, const uint16_t *scales, int nt, int K, const float *cb, int ti0, int ti1,
                           float *Q /* [(ti1-ti0)*16, nt*16] */) {
  const int n = nt * 16;
  uint16_t st[256];
  for (int ti = ti0; ti < ti1; ++ti)
    for (int tj = 0; tj < nt; ++tj) {
      htro_unpack_states(qw + ((size_t)ti * nt + tj) * (size_t)(8 * K), K, 1, st);
      for (int r = 0; r < 16; ++r) {
        float sc = htro_half_to_float(scales[ti * 16 + r]);
        float *dst = Q + (size_t)((ti - ti0) * 16 + r) * n + tj * 16;
        for (int c = 0; c < 16; ++c) dst[c] = cb[st[r * 16 + c]] * sc;
      }
    }
}

int htro_dequant_q(const uint32_t *qw, const uint16_t *scales, int mt, int nt, int K, float *Q) {
  if (K < 2 || K > 8) return -1;
  float *cb = (float *)malloc(sizeof(float) * HTRO_STATES);
  htro_codebook_f32(cb);
  dequant_q_rows(qw, scales, nt, K, cb, 0, mt, Q);
  free(cb);
  return 0;
}

/* One 128-row block of W = Sv Ho Q Hi Su, same op order as htr/wire.py:105-113 (dequant):
 * Hadamard over the 128 rows first, then over each 128-column block, then the signs. */
static void dequant_block(const uint32_t *qw, const uint16_t *scales, const uint8_t *su8, const uint8_t *sv8, int nt, int K,
                          const float *cb, const float *H, int rb, float *Qb /* scratch [128,n] */, float *Wb /* [128,n] */) {
  const int n = nt * 16;
  dequant_q_rows(qw, scales, nt, K, cb, rb * 8, rb * 8 + 8, Qb);
  /* rows: T[a, j] = sum_b Q[b, j] * H[b, a] */
  for (int a = 0; a < 128; ++a) {
    float *dst = Wb + (size_t)a * n;
    memset(dst, 0, sizeof(float) * (size_t)n);
    for (int b = 0; b < 128; ++b) {
      const float h = H[b * 128 + a];
      const float *src = Qb + (size_t)b * n;
      for (int j = 0; j < n; ++j) dst[j] += src[j] * h;
    }
  }
  /* cols, then signs: W[i, 128c + a] = sv_i * su_j * sum_b T[i, 128c + b] * H[b, a] */
  float tmp[128];
  for (int i = 0; i < 128; ++i) {
    const int gi = rb * 128 + i;
    const float svi = ((sv8[gi >> 3] >> (gi & 7)) & 1) ? -1.0f : 1.0f;
    float *row = Wb + (size_t)i * n;
    for (int c = 0; c < n / 128; ++c) {
      float acc[128];
      memcpy(tmp, row + c * 128, sizeof(tmp));
      memset(acc, 0, sizeof(acc));
      for (int b = 0; b < 128; ++b) {
        const float t = tmp[b];
        const float *hrow = H + b * 128;
        for (int a = 0; a < 128; ++a) acc[a] += t * hrow[a];
      }
      for (int a = 0; a < 128; ++a) {
        const int gj = c * 128 + a;
        const float suj = ((su8[gj >> 3] >> (gj & 7)) & 1) ? -1.0f : 1.0f;
        row[gj] = acc[a] * svi * suj;
      }
    }
  }
}

/* full original-basis W [m, n] float32: htr/wire.py:105-113 (dequant) */
int htro_dequant(const uint32_t *qw, const uint16_t *scales, const uint8_t *su8, const uint8_t *sv8, int mt, int nt, int K,
                 float *W) {
  if (K < 2 || K > 8 || mt % 8 || nt % 8) return -1;
  const int n = nt * 16;
  float *cb = (float *)malloc(sizeof(float) * HTRO_STATES);
  float *H = (float *)malloc(sizeof(float) * 128 * 128);
  htro_codebook_f32(cb);
  htro_hadamard128(H);
#pragma omp parallel
  {
    float *Qb = (float *)malloc(sizeof(float) * 128 * (size_t)n);
#pragma omp for schedule(dynamic)
    for (int rb = 0; rb < mt / 8; ++rb) dequant_block(qw, scales, su8, sv8, nt, K, cb, H, rb, Qb, W + (size_t)rb * 128 * n);
    free(Qb);
  }
  free(cb);
  free(H);
  return 0;
}

/* The reference CPU path for one packed linear: decode W (wire.dequant) and contract
 * y[r, i] = sum_j x[r, j] * W[i, j] (+ bias), htr/ops.py:93.  W is produced one 128-row
 * block at a time and consumed immediately, so arbitrarily tall matrices fit in memory.
 * x is float32 (callers widen bf16/fp16 activations exactly); accumulation in float64. */
int htro_linear(const float *x, int M, const uint32_t *qw, const uint16_t *scales, const uint8_t *su8, const uint8_t *sv8,
                const float *bias, int mt, int nt, int K, float *y) {
  if (K < 2 || K > 8 || mt % 8 || nt % 8) return -1;
  const int n = nt * 16, m = mt * 16;
  float *cb = (float *)malloc(sizeof(float) * HTRO_STATES);
  float *H = (float *)malloc(sizeof(float) * 128 * 128);
  htro_codebook_f32(cb);
  htro_hadamard128(H);
#pragma omp parallel
  {
    float *Qb = (float *)malloc(sizeof(float) * 128 * (size_t)n);
    float *Wb = (float *)malloc(sizeof(float) * 128 * (size_t)n);
#pragma omp for schedule(dynamic)
    for (int rb = 0; rb < mt / 8; ++rb) {
      dequant_block(qw, scales, su8, sv8, nt, K, cb, H, rb, Qb, Wb);
      for (int r = 0; r < M; ++r)
        for (int i = 0; i < 128; ++i) {
          const float *wrow = Wb + (size_t)i * n, *xr = x + (size_t)r * n;
          double acc = 0.0;
          for (int j = 0; j < n; ++j) acc += (double)xr[j] * (double)wrow[j];
          if (bias) acc += (double)bias[rb * 128 + i];
          y[(size_t)r * m + rb * 128 + i] = (float)acc;
        }
    }
    free(Qb);
    free(Wb);
  }
  free(cb);
  free(H);
  return 0;
}

/* block-diagonal H128/sqrt(128) applied to rows of x after the input sign flip:
 * xt = blk_had(su * x), the activation transform of docs/FORMAT.md:8 (htr/wire.py:90-92) */
int htro_rht(const float *x, int M, int n, const uint8_t *su8, float *xt) {
  if (n % 128) return -1;
  float *H = (float *)malloc(sizeof(float) * 128 * 128);
  htro_hadamard128(H);
  for (int r = 0; r < M; ++r)
    for (int c = 0; c < n / 128; ++c)
      for (int a = 0; a < 128; ++a) {
        double acc = 0.0;
        for (int b = 0; b < 128; ++b) {
          const int gj = c * 128 + b;
          const float s = ((su8[gj >> 3] >> (gj & 7)) & 1) ? -1.0f : 1.0f;
          acc += (double)(x[(size_t)r * n + gj] * s) * (double)H[b * 128 + a];
        }
        xt[(size_t)r * n + c * 128 + a] = (float)acc;
      }
  free(H);
  return 0;
}

/* ---- encoder search: htr/reference.py:7-50 (viterbi) ---------------------------------------
 * Tail-biting Viterbi over the bit-shift trellis of one tile per batch row: minimises
 * sum_t w[t] * (x[t] - cb[s_t])^2 subject to s_t = ((s_{t-1} << K) & 0xFFFF) | new bits.  Same float32 operation order as
 * the reference (subtract, square, times w, plus the running minimum), first minimum wins on ties (torch.min / argmin return
 * the first minimal index), two passes for tail-biting: the low 16-K bits of the unconstrained winner become the required
 * high bits of the first state and low bits of the last.  states: [B][T] int32, total: [B] cost of the returned path's
 * final state (pass-2 value).  Returns 0, or -1 on bad arguments / allocation failure. */
int htro_viterbi(const float *x, const float *w, size_t B, int T, int K, int tailbite, int32_t *states, float *total) {
  if (K < 1 || K > 8 || T < 1) return -1;
  const uint32_t nb = 1u << K, Sj = HTRO_STATES >> K;
  float *cb = (float *)malloc(HTRO_STATES * sizeof(float));
  if (!cb) return -1;
  htro_codebook_f32(cb);
  int failed = 0;
#pragma omp parallel for schedule(dynamic, 1)
  for (long long b = 0; b < (long long)B; ++b) {
    float *cost = (float *)malloc(HTRO_STATES * sizeof(float));
    float *mins = (float *)malloc(Sj * sizeof(float));
    uint8_t *bps = (uint8_t *)malloc((size_t)(T > 1 ? T - 1 : 1) * Sj);
    if (!cost || !mins || !bps) {
      failed = 1;
      free(cost); free(mins); free(bps);
      continue;
    }
    const float *xb = x + (size_t)b * T, *wb = w + (size_t)b * T;
    long long j0 = -1;
    for (int pass = 0; pass < (tailbite ? 2 : 1); ++pass) {
      for (uint32_t s = 0; s < HTRO_STATES; ++s) {           /* reference.py:22-27 */
        const float d = xb[0] - cb[s];
        const float dd = d * d;
        const float c = wb[0] * dd;
        cost[s] = (j0 >= 0 && (long long)(s >> K) != j0) ? INFINITY : c;
      }
      for (int t = 1; t < T; ++t) {                          /* reference.py:29-33 */
        for (uint32_t j = 0; j < Sj; ++j) {
          float m = cost[j];
          uint32_t arg = 0;
          for (uint32_t top = 1; top < nb; ++top) {
            const float v = cost[top * Sj + j];
            if (v < m) { m = v; arg = top; }
          }
          mins[j] = m;
          bps[(size_t)(t - 1) * Sj + j] = (uint8_t)arg;
        }
        for (uint32_t j = 0; j < Sj; ++j)
          for (uint32_t a = 0; a < nb; ++a) {
            const float d = xb[t] - cb[j * nb + a];
            const float dd = d * d;
            const float wd = wb[t] * dd;
            cost[j * nb + a] = mins[j] + wd;
          }
      }
      if (tailbite && pass == 0) {                           /* reference.py:36-38 */
        uint32_t best = 0;
        for (uint32_t s = 1; s < HTRO_STATES; ++s)
          if (cost[s] < cost[best]) best = s;
        j0 = best & (Sj - 1);
      }
    }
    uint32_t s = 0;                                          /* reference.py:39-42 */
    int have = 0;
    for (uint32_t c = 0; c < HTRO_STATES; ++c) {
      if (tailbite && (long long)(c & (Sj - 1)) != j0) continue;
      if (!have || cost[c] < cost[s]) { s = c; have = 1; }
    }
    if (total) total[b] = cost[s];
    states[(size_t)b * T + T - 1] = (int32_t)s;
    for (int t = T - 1; t >= 1; --t) {                       /* reference.py:45-49 */
      const uint32_t low = s >> K;
      s = (uint32_t)bps[(size_t)(t - 1) * Sj + low] * Sj + low;
      states[(size_t)b * T + t - 1] = (int32_t)s;
    }
    free(cost); free(mins); free(bps);
  }
  free(cb);
  return failed ? -1 : 0;
}

/* cost of a given path under the same arithmetic, summed in double (independent check of a search result) */
double htro_path_cost(const float *x, const float *w, int T, const int32_t *states) {
  float *cb = (float *)malloc(HTRO_STATES * sizeof(float));
  if (!cb) return -1.0;
  htro_codebook_f32(cb);
  double acc = 0.0;
  for (int t = 0; t < T; ++t) {
    const double d = (double)x[t] - (double)cb[states[t] & 0xFFFF];
    acc += (double)w[t] * d * d;
  }
  free(cb);
  return acc;
}

int htro_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void htro_set_num_threads(int t) {
#ifdef _OPENMP
  if (t > 0) omp_set_num_threads(t);
#else
  (void)t;
#endif
}
