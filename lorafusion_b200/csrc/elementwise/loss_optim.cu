// Cross-entropy over a chunk of logits (loss + in-place gradient) and the multi-tensor
// Adam step for LoRA adapters.
//
// Cross-entropy: the lm_head GEMM is run chunk by chunk over tokens so that the
// [tokens, vocab] logits never exist in full; this kernel turns one bf16 logits chunk into
// per-token losses and overwrites it with d(loss)/d(logits), which the next GEMM multiplies
// by the lm_head weight.  (The reference goes through HF's lm_head + torch cross-entropy,
// lorafusion/pipeline_parallel/pipe_module.py:218-221.)
//
// Adam: one launch updates every LoRA tensor of one adapter.  Tensors are described by a
// chunk table (offset, length) into parallel arenas: fp32 gradient, fp32 master weight,
// fp32 m, fp32 v and the bf16 working copy the GEMM kernels read.  The gradient arena is
// zeroed as it is consumed.  (The reference uses torch.optim.AdamW(fused=True) per adapter,
// benchmarks_paper/bench_multi_gpu.py:225-230.)
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lf {

constexpr int CE_THREADS = 512;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum2(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One CTA per token.  Pass 1: online max / sum-exp.  Pass 2: write the gradient in place.
// labels < 0 are ignored (loss 0, gradient 0).  grad_scale multiplies the gradient
// (1 / number of valid tokens for a mean loss).
__global__ void __launch_bounds__(CE_THREADS)
cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const int* __restrict__ labels,
                     float* __restrict__ loss_out, int V, long long ld, float grad_scale) {
  __shared__ float red_m[CE_THREADS / 32];
  __shared__ float red_s[CE_THREADS / 32];
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const int label = labels[row];
  const int nvec = V / 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (label < 0) {
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int c = threadIdx.x; c < nvec; c += CE_THREADS) reinterpret_cast<uint4*>(lr)[c] = z;
    for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) lr[c] = __float2bfloat16(0.f);
    if (threadIdx.x == 0) loss_out[row] = 0.f;
    return;
  }

  float m = -INFINITY, s = 0.f;
  for (int c = threadIdx.x; c < nvec; c += CE_THREADS) {
    uint4 raw = reinterpret_cast<const uint4*>(lr)[c];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(h[j]);
      f[2 * j] = t.x;
      f[2 * j + 1] = t.y;
    }
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    if (lm > m) {
      s *= __expf(m - lm);
      m = lm;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) {
    const float f = __bfloat162float(lr[c]);
    if (f > m) {
      s *= __expf(m - f);
      m = f;
    }
    s += __expf(f - m);
  }
  // block reduce (max, then rescaled sums)
  float wm = warp_max(m);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - wm);  // threads that saw no element
  s = warp_sum2(s);
  if (lane == 0) {
    red_m[warp] = wm;
    red_s[warp] = s;
  }
  __syncthreads();
  float bm = red_m[0];
  for (int i = 1; i < CE_THREADS / 32; ++i) bm = fmaxf(bm, red_m[i]);
  float bs = 0.f;
  for (int i = 0; i < CE_THREADS / 32; ++i)
    bs += (red_m[i] == -INFINITY) ? 0.f : red_s[i] * __expf(red_m[i] - bm);
  const float lse = bm + __logf(bs);
  const float inv_sum = 1.f / bs;
  const float label_logit = __bfloat162float(lr[label]);
  __syncthreads();  // everyone has read lr[label] before it is overwritten
  if (threadIdx.x == 0) loss_out[row] = lse - label_logit;

  for (int c = threadIdx.x; c < nvec; c += CE_THREADS) {
    uint4 raw = reinterpret_cast<const uint4*>(lr)[c];
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(h[j]);
      const int col = c * 8 + 2 * j;
      float g0 = __expf(t.x - bm) * inv_sum - (col == label ? 1.f : 0.f);
      float g1 = __expf(t.y - bm) * inv_sum - (col + 1 == label ? 1.f : 0.f);
      h[j] = __floats2bfloat162_rn(g0 * grad_scale, g1 * grad_scale);
    }
    reinterpret_cast<uint4*>(lr)[c] = raw;
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) {
    const float f = __bfloat162float(lr[c]);
    const float g = __expf(f - bm) * inv_sum - (c == label ? 1.f : 0.f);
    lr[c] = __float2bfloat16(g * grad_scale);
  }
}

// ---------------------------------------------------------------------------------
// Adam / AdamW over a chunk table.
// ---------------------------------------------------------------------------------
// A chunk is a 2-D region of `rows` x `ld` elements starting at `offset` in every arena.
// Its gradient is always cleared; only columns [col0, col0 + cols) of each row are
// trainable (block-diagonal B matrices of merged projections keep their off-diagonal
// blocks at zero this way).  A flat tensor is rows = 1, ld = cols = length, col0 = 0.
// `grad` and `work` use the padded layout (`offset`); master / m / v hold the trainable
// elements only, densely: element (row, col) lives at state + row * cols + (col - col0).
struct AdamChunk {
  long long offset;
  long long rows;
  long long ld;
  long long col0;
  long long cols;
  long long state;
};

struct AdamHyper {
  float lr, beta1, beta2, eps, weight_decay;
  float bias_c1, bias_c2;  // 1 - beta1^t, 1 - beta2^t
  float grad_scale;        // multiplies the accumulated gradient before the update
};

__device__ __forceinline__ void adam_one(float g, float& w, float& mi, float& vi, const AdamHyper& h,
                                         float inv_c1, float inv_sqrt_c2) {
  mi = h.beta1 * mi + (1.f - h.beta1) * g;
  vi = h.beta2 * vi + (1.f - h.beta2) * g * g;
  w -= h.lr * h.weight_decay * w;
  w -= h.lr * (mi * inv_c1) / (sqrtf(vi) * inv_sqrt_c2 + h.eps);
}

// One CTA per work item {chunk, first element, element count}: regions differ in size by two
// orders of magnitude (a 16 x 8192 A block next to a 57344 x 64 B block), so the host cuts
// them into equal pieces instead of giving every region the same number of CTAs.  Regions
// whose offsets and sizes are all multiples of four elements (every region the adapter arenas
// produce) go through 16-byte accesses with 32-bit index arithmetic; anything else takes the
// scalar path.
struct AdamWorkItem {
  int chunk;
  unsigned first, count;  // elements; multiples of 4 inside vectorisable regions
};

__global__ void __launch_bounds__(256)
adam_chunks_kernel(const AdamChunk* __restrict__ chunks, const AdamWorkItem* __restrict__ items,
                   float* __restrict__ grad, float* __restrict__ master, float* __restrict__ m,
                   float* __restrict__ v, __nv_bfloat16* __restrict__ work, AdamHyper h) {
  const AdamWorkItem item = items[blockIdx.x];
  const AdamChunk c = chunks[item.chunk];
  const float inv_c1 = 1.f / h.bias_c1;
  const float inv_sqrt_c2 = rsqrtf(h.bias_c2);
  const long long total = c.rows * c.ld;
  const bool vec = (((c.offset | c.ld | c.col0 | c.cols | c.state) & 3) == 0) && total < (1ll << 31) &&
                   ((item.first | item.count) & 3u) == 0;
  if (vec) {
    float4* g4p = reinterpret_cast<float4*>(grad + c.offset);
    const unsigned ld = unsigned(c.ld), col0 = unsigned(c.col0), cols = unsigned(c.cols);
    const unsigned end4 = (item.first + item.count) >> 2;
    for (unsigned i4 = (item.first >> 2) + threadIdx.x; i4 < end4; i4 += 256u) {
      const float4 g = g4p[i4];
      g4p[i4] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (cols == 0) continue;  // padding: cleared only
      const unsigned e = i4 << 2;
      const unsigned row = e / ld;
      const unsigned col = e - row * ld;
      if (col < col0 || col >= col0 + cols) continue;
      const long long se = c.state + (long long)row * cols + (col - col0);
      float4 w4 = *reinterpret_cast<const float4*>(master + se);
      float4 m4 = *reinterpret_cast<const float4*>(m + se);
      float4 v4 = *reinterpret_cast<const float4*>(v + se);
      adam_one(g.x * h.grad_scale, w4.x, m4.x, v4.x, h, inv_c1, inv_sqrt_c2);
      adam_one(g.y * h.grad_scale, w4.y, m4.y, v4.y, h, inv_c1, inv_sqrt_c2);
      adam_one(g.z * h.grad_scale, w4.z, m4.z, v4.z, h, inv_c1, inv_sqrt_c2);
      adam_one(g.w * h.grad_scale, w4.w, m4.w, v4.w, h, inv_c1, inv_sqrt_c2);
      *reinterpret_cast<float4*>(master + se) = w4;
      *reinterpret_cast<float4*>(m + se) = m4;
      *reinterpret_cast<float4*>(v + se) = v4;
      __nv_bfloat162 lo = __floats2bfloat162_rn(w4.x, w4.y), hi = __floats2bfloat162_rn(w4.z, w4.w);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(work + c.offset + e) = packed;
    }
    return;
  }
  for (long long i = (long long)item.first + threadIdx.x; i < (long long)item.first + item.count; i += 256) {
    const long long e = c.offset + i;
    const float g = grad[e] * h.grad_scale;
    grad[e] = 0.f;
    const long long col = i % c.ld;
    if (col < c.col0 || col >= c.col0 + c.cols) continue;
    const long long se = c.state + (i / c.ld) * c.cols + (col - c.col0);
    float w = master[se], mi = m[se], vi = v[se];
    adam_one(g, w, mi, vi, h, inv_c1, inv_sqrt_c2);
    m[se] = mi;
    v[se] = vi;
    master[se] = w;
    work[e] = __float2bfloat16(w);
  }
}

}  // namespace lf

using namespace lf;

extern "C" {

int lf_cross_entropy(void* logits, const int* labels, float* loss, long long M, int V,
                     long long ld, float grad_scale, void* stream) {
  if (M == 0) return 0;
  if (ld % 8 != 0) return -1;
  cross_entropy_kernel<<<(unsigned)M, CE_THREADS, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)logits, labels, loss, V, ld, grad_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// chunks: device array of AdamChunk {int64 offset, rows, ld, col0, cols, state};
// items: device array of AdamWorkItem {int32 chunk, uint32 first, uint32 count} covering every
// element of every chunk exactly once (first and count multiples of 4 unless the chunk has odd
// offsets or sizes).
int lf_adam_chunks(const void* chunks, const void* items, int num_items, float* grad, float* master,
                   float* m, float* v, void* work, float lr, float beta1, float beta2, float eps,
                   float weight_decay, int step, float grad_scale, void* stream) {
  if (num_items <= 0) return 0;
  AdamHyper h;
  h.lr = lr;
  h.beta1 = beta1;
  h.beta2 = beta2;
  h.eps = eps;
  h.weight_decay = weight_decay;
  h.bias_c1 = 1.f - powf(beta1, (float)step);
  h.bias_c2 = 1.f - powf(beta2, (float)step);
  h.grad_scale = grad_scale;
  adam_chunks_kernel<<<num_items, 256, 0, (cudaStream_t)stream>>>(
      (const AdamChunk*)chunks, (const AdamWorkItem*)items, grad, master, m, v, (__nv_bfloat16*)work, h);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
