// Memory-bound token-wise kernels of the decoder block: RMSNorm (+ fused residual add),
// rotary embedding applied in place to the packed QKV projection, SwiGLU on the merged
// gate|up projection, and the embedding gather.  The base model is frozen, so none of the
// backward kernels produces weight gradients.  They stand in for the Liger Triton kernels
// the reference patches into HF models (lorafusion/utils/module.py:40-69).
//
// All kernels use 16-byte vector accesses; feature sizes must be multiples of 8.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lf {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < THREADS / 32) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

struct alignas(16) BF8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  BF8 b = *reinterpret_cast<const BF8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(b.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  BF8 b;
#pragma unroll
  for (int i = 0; i < 4; ++i) b.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<BF8*>(p) = b;
}

// ---------------------------------------------------------------------------------
// RMSNorm forward:  h = x (+ res);  y = h * rsqrt(mean(h^2) + eps) * w
// One CTA per token row; the row stays in registers between the reduction and the write.
// ---------------------------------------------------------------------------------
constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_VEC = 8;  // supports H up to 256 * 8 * 8 = 16384

// NV = 16-byte vectors per thread (ceil(H / 8 / 256)); a template so that the row fits in
// as few registers as the hidden size needs (occupancy is what hides the DRAM latency here).
template <int NV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int H,
                   float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * H;
  const int nvec = H / 8;
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      load8(xr + c * 8, v[i]);
      if (res != nullptr) {
        float r[8];
        load8(res + row * H + c * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += r[j];
        // the residual stream is stored in bf16: normalise exactly what is stored
        BF8 b;
#pragma unroll
        for (int j = 0; j < 4; ++j) b.v[j] = __floats2bfloat162_rn(v[i][2 * j], v[i][2 * j + 1]);
        if (h_out != nullptr) *reinterpret_cast<BF8*>(h_out + row * H + c * 8) = b;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 t = __bfloat1622float2(b.v[j]);
          v[i][2 * j] = t.x;
          v[i][2 * j + 1] = t.y;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  ss = block_sum<NORM_THREADS>(ss, red);
  const float rstd = rsqrtf(ss / float(H) + eps);
  if (threadIdx.x == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      float wv[8], o[8];
      load8(w + c * 8, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * wv[j];
      store8(y + row * H + c * 8, o);
    }
  }
}

// RMSNorm backward (no weight grad):
//   g = dy * w;  dx = rstd * (g - xhat * mean(g * xhat))  (+ dres),  xhat = h * rstd
template <int NV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx, int H) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int nvec = H / 8;
  const float rstd = rstd_in[row];
  // Two passes over the row: the first forms the dot product, the second re-reads dy and h (they
  // were fetched microseconds ago and sit in L2, of which the rows in flight take a few percent)
  // and writes dx.  Keeping the row in registers instead cost 96-106 registers per thread and
  // with them the resident CTAs that hide the DRAM latency.
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      float g[8], xh[8], wv[8];
      load8(dy + row * H + c * 8, g);
      load8(h + row * H + c * 8, xh);
      load8(w + c * 8, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += (g[j] * wv[j]) * (xh[j] * rstd);
    }
  }
  dot = block_sum<NORM_THREADS>(dot, red) / float(H);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      float g[8], xh[8], wv[8], o[8];
      load8(dy + row * H + c * 8, g);
      load8(h + row * H + c * 8, xh);
      load8(w + c * 8, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rstd * (g[j] * wv[j] - (xh[j] * rstd) * dot);
      if (dres != nullptr) {
        float r[8];
        load8(dres + row * H + c * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      store8(dx + row * H + c * 8, o);
    }
  }
}

// ---------------------------------------------------------------------------------
// Rotary embedding, rotate-half convention, in place on the q and k parts of the packed
// QKV activation [M, (Hq + 2 Hkv) * D].  cos/sin come from a table [max_pos, D/2] gathered
// by position id.  `sign` = +1 forward, -1 backward (the transpose of a rotation).
// ---------------------------------------------------------------------------------
__global__ void rope_inplace_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos,
                                    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                    int M, int n_rot_heads, int D, int row_stride, float sign) {
  const int half = D / 2;
  const int vec_per_head = half / 8;
  const long long total = (long long)M * n_rot_heads * vec_per_head;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int vi = int(idx % vec_per_head);
    const long long t = idx / vec_per_head;
    const int head = int(t % n_rot_heads);
    const long long row = t / n_rot_heads;
    const int p = pos[row];
    __nv_bfloat16* base = qkv + row * row_stride + head * D + vi * 8;
    float lo[8], hi[8], c[8], s[8];
    load8(base, lo);
    load8(base + half, hi);
    const float* cp = cos_t + (long long)p * half + vi * 8;
    const float* sp = sin_t + (long long)p * half + vi * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      c[j] = cp[j];
      s[j] = sign * sp[j];
    }
    float olo[8], ohi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      olo[j] = lo[j] * c[j] - hi[j] * s[j];
      ohi[j] = hi[j] * c[j] + lo[j] * s[j];
    }
    store8(base, olo);
    store8(base + half, ohi);
  }
}

// ---------------------------------------------------------------------------------
// SwiGLU on the merged projection gu[M, 2I] = [gate | up]:  out = silu(gate) * up
// ---------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ out, long long M, int I) {
  const int vec = I / 8;
  const long long total = M * vec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long row = idx / vec;
    const int c = int(idx % vec) * 8;
    float g[8], u[8], o[8];
    load8(gu + row * 2 * I + c, g);
    load8(gu + row * 2 * I + I + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    store8(out + row * I + c, o);
  }
}

// dgu[M, 2I] from dout[M, I] and the saved gu.
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout,
                                  const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, long long M, int I) {
  const int vec = I / 8;
  const long long total = M * vec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long row = idx / vec;
    const int c = int(idx % vec) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + row * 2 * I + c, g);
    load8(gu + row * 2 * I + I + c, u);
    load8(dout + row * I + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sig = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sig;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (sig + silu * (1.f - sig));
    }
    store8(dgu + row * 2 * I + c, dg);
    store8(dgu + row * 2 * I + I + c, du);
  }
}

// ---------------------------------------------------------------------------------
// Embedding gather: out[m, :] = table[ids[m], :]
// ---------------------------------------------------------------------------------
__global__ void embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, long long M, int H, int vocab) {
  const int vec = H / 8;
  const long long total = M * vec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long row = idx / vec;
    const int c = int(idx % vec) * 8;
    int id = ids[row];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    *reinterpret_cast<BF8*>(out + row * H + c) =
        *reinterpret_cast<const BF8*>(table + (long long)id * H + c);
  }
}

// out = a + b (bf16), used for residual adds that are not fused into a norm.
__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ out, long long n8) {
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n8;
       idx += (long long)gridDim.x * blockDim.x) {
    float x[8], y[8];
    load8(a + idx * 8, x);
    load8(b + idx * 8, y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += y[j];
    store8(out + idx * 8, x);
  }
}

static inline int grid_for(long long total, int threads) {
  long long b = (total + threads - 1) / threads;
  const long long cap = 148LL * 16;
  return int(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace lf

using namespace lf;

extern "C" {

int lf_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out,
                   float* rstd, long long M, int H, float eps, void* stream) {
  if (H % 8 != 0 || H > NORM_THREADS * NORM_MAX_VEC * 8) return -1;
  if (M == 0) return 0;
  const int nv = (H / 8 + NORM_THREADS - 1) / NORM_THREADS;
#define LF_NORM_FWD(NVV)                                                                        \
  rmsnorm_fwd_kernel<NVV><<<(unsigned)M, NORM_THREADS, 0, (cudaStream_t)stream>>>(               \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w,              \
      (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, rstd, H, eps)
  if (nv <= 1) LF_NORM_FWD(1);
  else if (nv == 2) LF_NORM_FWD(2);
  else if (nv == 3) LF_NORM_FWD(3);
  else if (nv == 4) LF_NORM_FWD(4);
  else LF_NORM_FWD(8);
#undef LF_NORM_FWD
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int lf_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd,
                   const void* dres, void* dx, long long M, int H, void* stream) {
  if (H % 8 != 0 || H > NORM_THREADS * NORM_MAX_VEC * 8) return -1;
  if (M == 0) return 0;
  const int nv = (H / 8 + NORM_THREADS - 1) / NORM_THREADS;
#define LF_NORM_BWD(NVV)                                                                        \
  rmsnorm_bwd_kernel<NVV><<<(unsigned)M, NORM_THREADS, 0, (cudaStream_t)stream>>>(               \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w, rstd,         \
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, H)
  if (nv <= 1) LF_NORM_BWD(1);
  else if (nv == 2) LF_NORM_BWD(2);
  else if (nv == 3) LF_NORM_BWD(3);
  else if (nv == 4) LF_NORM_BWD(4);
  else LF_NORM_BWD(8);
#undef LF_NORM_BWD
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int lf_rope_inplace(void* qkv, const int* pos, const float* cos_t, const float* sin_t, int M,
                    int n_rot_heads, int D, int row_stride, int backward, void* stream) {
  if (D % 16 != 0 || row_stride % 8 != 0) return -1;
  if (M == 0) return 0;
  const long long total = (long long)M * n_rot_heads * (D / 16);
  rope_inplace_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)qkv, pos, cos_t, sin_t, M, n_rot_heads, D, row_stride,
      backward ? -1.f : 1.f);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int lf_swiglu_fwd(const void* gu, void* out, long long M, int I, void* stream) {
  if (I % 8 != 0) return -1;
  if (M == 0) return 0;
  swiglu_fwd_kernel<<<grid_for(M * (I / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, M, I);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int lf_swiglu_bwd(const void* dout, const void* gu, void* dgu, long long M, int I, void* stream) {
  if (I % 8 != 0) return -1;
  if (M == 0) return 0;
  swiglu_bwd_kernel<<<grid_for(M * (I / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dout, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, M, I);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int lf_embedding(const int* ids, const void* table, void* out, long long M, int H, int vocab,
                 void* stream) {
  if (H % 8 != 0) return -1;
  if (M == 0) return 0;
  embedding_kernel<<<grid_for(M * (H / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, M, H, vocab);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int lf_add(const void* a, const void* b, void* out, long long n, void* stream) {
  if (n % 8 != 0) return -1;
  if (n == 0) return 0;
  add_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, n / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
