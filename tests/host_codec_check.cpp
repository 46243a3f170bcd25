// Host-side check of the index arithmetic in htr_b200/csrc/htr_codec.cuh: the header compiles as plain
// C++, so the per-thread window extraction can be compared with a bit-by-bit reading of the circular
// stream without a GPU.  Built and run by tests/test_host_logic.py; prints "ok" and exits 0 on success.
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "../htr_b200/csrc/htr_codec.cuh"

static unsigned stream_bit(const std::vector<uint32_t>& w, unsigned p) { return (w[p >> 5] >> (31u - (p & 31u))) & 1u; }

template <int K>
static int check_width(std::mt19937& rng) {
  int bad = 0;
  for (int rep = 0; rep < 64; ++rep) {
    std::vector<uint32_t> tile(8 * K);
    for (auto& x : tile) x = rng();
    if (rep == 0) for (auto& x : tile) x = 0xFFFFFFFFu;
    if (rep == 1) for (auto& x : tile) x = 0u;
    const unsigned nbits = 256u * K;
    for (int q = 0; q < 8; ++q) {
      uint32_t V[K + 1];
      V[0] = tile[htr::history_word<K>(q)];
      for (int k = 0; k < K; ++k) V[k + 1] = tile[q * K + k];
      uint32_t s[32];
      htr::unit_states<K>(V, s);
      for (int u = 0; u < 32; ++u) {
        const unsigned t = 32u * q + u, first = ((t + 1u) * K + nbits - 16u) % nbits;
        unsigned ref = 0;
        for (unsigned j = 0; j < 16; ++j) ref = (ref << 1) | stream_bit(tile, (first + j) % nbits);
        if (ref != s[u]) { ++bad; if (bad < 5) std::printf("K%d q%d u%d: got %u want %u\n", K, q, u, s[u], ref); }
        const uint32_t x = ref * 0xDF6ADFu + 0x34983u;
        const int v = (int)((x & 255) + ((x >> 8) & 255) + ((x >> 16) & 255) + (x >> 24)) - 510;
        if (htr::code_value(ref) != v) ++bad;
        float f;
        const uint32_t mb = htr::code_magic_bits(ref);
        __builtin_memcpy(&f, &mb, 4);
        if (f - htr::kMagic != (float)v) ++bad;
      }
    }
  }
  // staging permutation: a bijection of 0..15 whose window partners are neighbours at an even position
  bool seen[16] = {false};
  constexpr int P = htr::PairStride<K>::value;
  for (int c = 0; c < 16; ++c) {
    const int pos = htr::staged_col<K>(c);
    if (pos < 0 || pos > 15 || seen[pos]) ++bad;
    else seen[pos] = true;
    if (P > 1 && (c % (2 * P)) < P && (htr::staged_col<K>(c + P) != pos + 1 || (pos & 1))) ++bad;
  }
  return bad;
}

int main() {
  std::mt19937 rng(20260101u);
  int bad = 0;
  bad += check_width<2>(rng);
  bad += check_width<3>(rng);
  bad += check_width<4>(rng);
  bad += check_width<5>(rng);
  bad += check_width<6>(rng);
  bad += check_width<7>(rng);
  bad += check_width<8>(rng);
  if (bad) { std::printf("FAILED: %d mismatches\n", bad); return 1; }
  std::printf("ok\n");
  return 0;
}
