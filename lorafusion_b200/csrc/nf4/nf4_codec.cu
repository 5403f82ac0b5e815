// NF4 (4-bit NormalFloat) block quantisation of frozen base weights and the standalone
// dequantiser.
//
// Format (compatible with the bitsandbytes layout the reference dequantises in
// lorafusion/ops/triton_ops/dequantize_nf4.py:16-161): the weight [N, K] is flattened
// row-major and cut into blocks of 64 elements (K % 64 == 0, so a block never crosses a
// row); each block stores absmax and 64 4-bit codes, two per byte with the EVEN element in
// the high nibble.  The absmax vector is itself quantised ("double quantisation"): after
// subtracting its mean (`offset`), groups of 256 absmax values share one fp32 scale and
// each value is an 8-bit index into a 256-entry code table.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lf {

__constant__ float kNf4Code[16] = {
    -1.0f,
    -0.6961928009986877f,
    -0.5250730514526367f,
    -0.39491748809814453f,
    -0.28444138169288635f,
    -0.18477343022823334f,
    -0.09105003625154495f,
    0.0f,
    0.07958029955625534f,
    0.16093020141124725f,
    0.24611230194568634f,
    0.33791524171829224f,
    0.44070982933044434f,
    0.5626170039176941f,
    0.7229568362236023f,
    1.0f,
};

// Nearest code by comparing with the midpoints between consecutive code values.
__device__ __forceinline__ uint32_t nf4_encode(float x) {
  uint32_t q = 0;
#pragma unroll
  for (int i = 0; i < 15; ++i) {
    const float mid = 0.5f * (kNf4Code[i] + kNf4Code[i + 1]);
    q += (x > mid) ? 1u : 0u;
  }
  return q;
}

// Each thread quantises 8 consecutive elements; 8 threads cover one 64-element block.
__global__ void nf4_quantize_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ packed,
                                    float* __restrict__ absmax, long long n_elems) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long e0 = t * 8;
  float f[8];
  if (e0 < n_elems) {
    uint4 raw = *reinterpret_cast<const uint4*>(w + e0);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 v = __bfloat1622float2(h[j]);
      f[2 * j] = v.x;
      f[2 * j + 1] = v.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = 0.f;
  }
  float am = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(f[j]));
  am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
  am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
  am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 4));
  if (e0 >= n_elems) return;
  const float inv = am > 0.f ? 1.f / am : 0.f;
  uint32_t out = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t hi = nf4_encode(f[2 * j] * inv);
    const uint32_t lo = nf4_encode(f[2 * j + 1] * inv);
    out |= ((hi << 4) | lo) << (8 * j);
  }
  *reinterpret_cast<uint32_t*>(packed + e0 / 2) = out;
  if ((t & 7) == 0) absmax[e0 / 64] = am;
}

// Each thread expands four 4-byte words (8 codes each) that lie one block-width apart, so that
// every load instruction of a warp reads 128 contiguous bytes and every store instruction writes
// 512 contiguous bytes (one thread expanding 16 adjacent bytes made each store hit 32 separate
// 64-byte pieces).
//   absmax_q == nullptr : `absmax` holds fp32 block scales
//   absmax_q != nullptr : scale = code256[absmax_q[b]] * nested[b / 256] + offset
constexpr int kDequantWordsPerThread = 4;

__global__ void nf4_dequantize_kernel(const uint8_t* __restrict__ packed,
                                      const float* __restrict__ absmax,
                                      const uint8_t* __restrict__ absmax_q,
                                      const float* __restrict__ code256,
                                      const float* __restrict__ nested, float offset,
                                      __nv_bfloat16* __restrict__ out, long long n_elems) {
  __shared__ float lut[16];
  if (threadIdx.x < 16) lut[threadIdx.x] = kNf4Code[threadIdx.x];
  __syncthreads();
  const long long n_words = n_elems / 8;
  const long long w0 = (long long)blockIdx.x * blockDim.x * kDequantWordsPerThread + threadIdx.x;
  uint32_t word[kDequantWordsPerThread];
  float scale[kDequantWordsPerThread];
#pragma unroll
  for (int k = 0; k < kDequantWordsPerThread; ++k) {   // all loads first
    const long long wi = w0 + (long long)k * blockDim.x;
    if (wi < n_words) {
      word[k] = reinterpret_cast<const uint32_t*>(packed)[wi];
      const long long blk = wi / 8;   // 64 codes per scale block
      scale[k] = (absmax_q != nullptr) ? code256[absmax_q[blk]] * nested[blk / 256] + offset : absmax[blk];
    }
  }
#pragma unroll
  for (int k = 0; k < kDequantWordsPerThread; ++k) {
    const long long wi = w0 + (long long)k * blockDim.x;
    if (wi >= n_words) continue;
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t byte = (word[k] >> (8 * j)) & 0xffu;
      // even element in the high nibble
      __nv_bfloat162 v = __floats2bfloat162_rn(lut[byte >> 4] * scale[k], lut[byte & 15u] * scale[k]);
      o[j] = *reinterpret_cast<uint32_t*>(&v);
    }
    reinterpret_cast<uint4*>(out)[wi] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace lf

using namespace lf;

extern "C" {

int lf_nf4_quantize(const void* w, void* packed, float* absmax, long long n_elems, void* stream) {
  if (n_elems % 64 != 0) return -1;
  if (n_elems == 0) return 0;
  const long long threads = n_elems / 8;
  const int block = 256;
  const long long grid = (threads + block - 1) / block;
  nf4_quantize_kernel<<<(unsigned)grid, block, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)w, (uint8_t*)packed, absmax, n_elems);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int lf_nf4_dequantize(const void* packed, const float* absmax, const void* absmax_q,
                      const float* code256, const float* nested, float offset, void* out,
                      long long n_elems, void* stream) {
  if (n_elems % 64 != 0) return -1;
  if (n_elems == 0) return 0;
  const int block = 256;
  const long long per_block = (long long)block * kDequantWordsPerThread * 8;   // codes per block
  const long long grid = (n_elems + per_block - 1) / per_block;
  nf4_dequantize_kernel<<<(unsigned)grid, block, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)packed, absmax, (const uint8_t*)absmax_q, code256, nested, offset,
      (__nv_bfloat16*)out, n_elems);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
