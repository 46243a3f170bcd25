// HTR-W1 stream decoding primitives shared by every kernel of the library.
//
// Wire facts restated from the format text (docs/FORMAT.md:11-21) and the reference decoder
// (htr/wire.py:10-13 codebook, :46-63 circular stream):
//   * a tile is 8K uint32 words; stream bit p lives in word p>>5 at bit 31-(p&31);
//   * step t = 16*row + col; its state is the 16 stream bits that end at bit (t+1)K-1;
//   * v(s) = bytesum((s*0xDF6ADF + 0x34983) mod 2^32) - 510.
//
// Work unit of one thread ("lane unit"): two consecutive tile rows = 32 steps.  Their bits are
// the K words [qK, qK+K) of the tile (q = row pair) plus the word before them, circularly
// inside the tile, for the 16-K history bits.  With that word in V[0] and the own words in
// V[1..K], step u (0..31) of the unit is the 16-bit window of V that starts at bit 16+(u+1)K.
//
// Everything here also compiles as host code so that the index arithmetic can be unit-tested
// without a GPU (tests/host_codec_check.cpp).
#pragma once
#include <cstdint>
#include <utility>

#if defined(__CUDACC__)
#define HTR_HD __host__ __device__ __forceinline__
#else
#define HTR_HD inline
#endif

namespace htr {

constexpr uint32_t kGenMul = 0xDF6ADFu;
constexpr uint32_t kGenAdd = 0x34983u;
// float32 bit pattern of 1.5*2^23: adding an integer in (-2^22, 2^22) to these bits yields the float 12582912 + integer.
constexpr uint32_t kMagicBits = 0x4B400000u;
constexpr float kMagic = 12582912.0f;

HTR_HD uint32_t funnel_left(uint32_t hi, uint32_t lo, int sh) {  // upper word of (hi:lo) << sh, 0 < sh < 32
#if defined(__CUDA_ARCH__)
  return __funnelshift_l(lo, hi, sh);
#else
  return (hi << sh) | (lo >> (32 - sh));
#endif
}

HTR_HD uint32_t bytesum_add(uint32_t x, uint32_t acc) {  // acc + sum of the four bytes of x
#if defined(__CUDA_ARCH__)
  return __dp4a(x, 0x01010101u, acc);
#else
  return acc + (x & 255u) + ((x >> 8) & 255u) + ((x >> 16) & 255u) + (x >> 24);
#endif
}

HTR_HD uint32_t middle_bytes(uint32_t x) {  // bits 8..23 of x, zero-extended
#if defined(__CUDA_ARCH__)
  return __byte_perm(x, 0u, 0x4421);
#else
  return (x >> 8) & 0xFFFFu;
#endif
}

HTR_HD uint32_t bytesum_add_alu(uint32_t x, uint32_t acc) {  // same value through the byte-wise |a-b| sum (a different pipe)
#if defined(__CUDA_ARCH__)
  uint32_t d;
  asm("vabsdiff4.u32.u32.u32.add %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(0u), "r"(acc));
  return d;
#else
  return acc + (x & 255u) + ((x >> 8) & 255u) + ((x >> 16) & 255u) + (x >> 24);
#endif
}

// codebook integer of a 16-bit state
HTR_HD int code_value(uint32_t s) { return (int)bytesum_add(s * kGenMul + kGenAdd, 0u) - 510; }
// float32 bits of 12582912 + v(s): one multiply-add and one byte dot product, no conversion instruction
HTR_HD uint32_t code_magic_bits(uint32_t s) { return bytesum_add(s * kGenMul + kGenAdd, kMagicBits - 510u); }
HTR_HD uint32_t code_magic_bits_alu(uint32_t s) { return bytesum_add_alu(s * kGenMul + kGenAdd, kMagicBits - 510u); }

// step distance of two states that sit side by side in one 32-bit window of the stream (K | 16), else 1
template <int K>
struct PairStride {
  static constexpr int value = (16 % K == 0) ? 16 / K : 1;
};

// Position (0..15) at which column c of a tile is stored in the activation staging buffer, chosen so
// that the two columns decoded from one 32-bit window are neighbours (one 8-byte shared-memory word).
template <int K>
HTR_HD int staged_col(int c) {
  constexpr int P = PairStride<K>::value;
  if constexpr (P == 1) return c;
  else return 2 * ((c / (2 * P)) * P + (c % P)) + ((c % (2 * P)) >= P ? 1 : 0);
}

// 32-bit window of V starting at bit BIT (BIT + 32 <= 32*(K+1))
template <int K, int BIT>
HTR_HD uint32_t window32(const uint32_t (&V)[K + 1]) {
  constexpr int w = BIT >> 5, off = BIT & 31;
  if constexpr (off == 0) return V[w];
  else return funnel_left(V[w], V[w + 1], off);
}

// 16-bit window of V starting at bit BIT, zero-extended
template <int K, int BIT>
HTR_HD uint32_t window16(const uint32_t (&V)[K + 1]) {
  constexpr int w = BIT >> 5, off = BIT & 31;
  if constexpr (off == 0) return V[w] >> 16;
  else if constexpr (off == 16) return V[w] & 0xFFFFu;
  else if constexpr (off == 8) return middle_bytes(V[w]);
  else if constexpr (off < 16) return (V[w] >> (16 - off)) & 0xFFFFu;
  else return funnel_left(V[w], V[w + 1], off) >> 16;
}

namespace detail {
template <int K, int CHAIN, int J>
HTR_HD void pair_window(const uint32_t (&V)[K + 1], uint32_t (&s)[32]) {
  constexpr int P = PairStride<K>::value;
  const uint32_t win = window32<K, 16 + (CHAIN + 1) * K + 32 * J>(V);
  s[CHAIN + (2 * J) * P] = win >> 16;
  s[CHAIN + (2 * J + 1) * P] = win & 0xFFFFu;
}
template <int K, int CHAIN, int... J>
HTR_HD void pair_chain(const uint32_t (&V)[K + 1], uint32_t (&s)[32], std::integer_sequence<int, J...>) {
  (pair_window<K, CHAIN, J>(V, s), ...);
}
template <int K, int... CHAIN>
HTR_HD void pair_all(const uint32_t (&V)[K + 1], uint32_t (&s)[32], std::integer_sequence<int, CHAIN...>) {
  constexpr int P = PairStride<K>::value;
  (pair_chain<K, CHAIN>(V, s, std::make_integer_sequence<int, 16 / P>{}), ...);
}
template <int K, int... U>
HTR_HD void single_all(const uint32_t (&V)[K + 1], uint32_t (&s)[32], std::integer_sequence<int, U...>) {
  ((s[U] = window16<K, 16 + (U + 1) * K>(V)), ...);
}
}  // namespace detail

// The 32 states of a lane unit, indexed by step u.  For K dividing 16 the states u and u+16/K are the
// two halves of one 32-bit window: one funnel shift then serves two states.
template <int K>
HTR_HD void unit_states(const uint32_t (&V)[K + 1], uint32_t (&s)[32]) {
  if constexpr (PairStride<K>::value > 1) detail::pair_all<K>(V, s, std::make_integer_sequence<int, PairStride<K>::value>{});
  else detail::single_all<K>(V, s, std::make_integer_sequence<int, 32>{});
}

// index (inside the tile's 8K words) of the history word of row pair q
template <int K>
HTR_HD int history_word(int q) { return (q * K + 8 * K - 1) % (8 * K); }

}  // namespace htr
