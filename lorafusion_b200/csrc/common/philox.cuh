// Counter-based dropout mask shared by every kernel that needs it (and by the CPU oracle
// in lorafusion_b200/ops/philox.py, which must produce identical bits).
//
// One Philox4x32-7 call is keyed by (seed_lo, seed_hi) and indexed by the counter
// (row, col / 8, stream, 0).  Its 128 output bits are read as eight 16-bit lanes; element
// (row, col) uses lane (col % 8): lane j = (out[j >> 1] >> (16 * (j & 1))) & 0xffff and is
// KEPT iff lane >= thresh16, where thresh16 = round(p * 65536).  Because the mask is a
// pure function of (seed, stream, row, col) it is never stored: forward, recompute and
// the backward kernels regenerate it.
#pragma once
#include <stdint.h>

namespace lf {

struct Philox4 {
  uint32_t x, y, z, w;
};

__host__ __device__ __forceinline__ uint32_t mulhi32(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
  return __umulhi(a, b);
#else
  return static_cast<uint32_t>((static_cast<uint64_t>(a) * b) >> 32);
#endif
}

template <int ROUNDS = 7>
__host__ __device__ __forceinline__ Philox4 philox4x32(uint32_t c0, uint32_t c1, uint32_t c2,
                                                        uint32_t c3, uint32_t k0, uint32_t k1) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  constexpr uint32_t W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
    const uint32_t hi0 = mulhi32(M0, c0), lo0 = M0 * c0;
    const uint32_t hi1 = mulhi32(M1, c2), lo1 = M1 * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0;
    const uint32_t n2 = hi0 ^ c3 ^ k1;
    c0 = n0;
    c1 = lo1;
    c2 = n2;
    c3 = lo0;
    k0 += W0;
    k1 += W1;
  }
  return Philox4{c0, c1, c2, c3};
}

// Bit j of the result is 1 iff element (row, 8 * col8 + j) is kept.
__host__ __device__ __forceinline__ uint32_t dropout_keep8(uint32_t row, uint32_t col8,
                                                           uint32_t stream, uint32_t seed_lo,
                                                           uint32_t seed_hi, uint32_t thresh16) {
  const Philox4 o = philox4x32<7>(row, col8, stream, 0u, seed_lo, seed_hi);
  const uint32_t w[4] = {o.x, o.y, o.z, o.w};
  uint32_t bits = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t lane = (w[j >> 1] >> (16 * (j & 1))) & 0xffffu;
    bits |= (lane >= thresh16 ? 1u : 0u) << j;
  }
  return bits;
}

}  // namespace lf
