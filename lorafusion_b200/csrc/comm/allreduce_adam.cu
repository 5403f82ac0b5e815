// Data-parallel LoRA gradient reduction fused with the optimizer step, over NVLink peer
// memory: one kernel = reduce-scatter of the adapter's gradients + gradient scaling + AdamW on
// the rank's shard + all-gather of the updated bf16 weights.
//
// The reference reduces each adapter's gradients with Megatron DDP (bucketed NCCL all-reduce,
// no overlap) and then runs torch AdamW on every rank
// (lorafusion/ops/multi_lora.py:166-184, benchmarks_paper/bench_multi_gpu.py:135-149,225-230).
// Here the gradient and bf16 weight arenas live in symmetric memory (same offsets on every
// rank, peer pointers known to the kernel).  For every chunk of the adapter (see AdamChunk in
// loss_optim.cu) rank r owns the r-th contiguous slice of the chunk's elements and
//   1. loads that slice of the gradient from every rank (P2P loads, or one
//      multimem.ld_reduce through NVSwitch), sums in fp32 in a fixed rank order,
//   2. clears the slice in every rank's gradient arena,
//   3. applies AdamW to its local fp32 master / m / v (optimizer state is only ever touched
//      by the owner, i.e. it is sharded ZeRO-1 style even though the arenas are full-size),
//   4. stores the new bf16 weight into every rank's working copy (P2P stores or multimem.st).
// Cross-rank ordering uses epoch flags in a symmetric signal pad: "gradients ready" before
// step 1 and "weights written" after step 4.  All waits are bounded and report through the
// error word.  With sync_mode 0 the flags are skipped: that mode runs the ranks one after
// another on ONE GPU (for tests) or with a single rank.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../common/ptx.cuh"

namespace lf {

constexpr int kMaxRanks = 8;

struct ArAdamChunk {
  long long offset, rows, ld, col0, cols, state;
};

// {chunk, first element, element count} (multiples of 4): the part of a chunk one CTA handles.
// The host cuts THIS RANK's slice of every chunk into equal pieces, so that the CTAs are
// balanced although chunk sizes differ by two orders of magnitude.
struct ArAdamWorkItem {
  int chunk;
  unsigned first, count;
};

struct ArAdamParams {
  const ArAdamChunk* chunks;
  const ArAdamWorkItem* items;
  int num_chunks;
  int rank, world;
  float* grad[kMaxRanks];            // peer pointers to the fp32 gradient arenas
  __nv_bfloat16* work[kMaxRanks];    // peer pointers to the bf16 working copies
  float* grad_mc;                    // multicast address of the gradient arena (or null)
  __nv_bfloat16* work_mc;            // multicast address of the working copy (or null)
  float* master;
  float* m;
  float* v;
  int* flags[kMaxRanks];             // peer pointers to the signal pads: int[2 * kMaxRanks]
  int epoch;
  int sync_mode;                     // 0 = no cross-rank flags, 1 = flags
  int use_multimem;
  unsigned long long wait_ns;        // limit of every cross-rank flag wait
  unsigned int* done_counter;        // local, zero before launch, reset by the kernel
  float lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2, grad_scale;
  int* err;
  // optional [gridDim.x, 3] nanosecond stamps (globaltimer): block entry, every rank's gradients
  // seen complete, block exit -- what a trace needs to tell waiting for peers from working
  unsigned long long* trace;
};

__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc_ptr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_ptr)
               : "memory");
  return r;
}
__device__ __forceinline__ void multimem_st_f32x4(float* mc_ptr, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_ptr),
               "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ void multimem_st_b32x2(void* mc_ptr, uint32_t a, uint32_t b) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc_ptr),
               "f"(__uint_as_float(a)), "f"(__uint_as_float(b))
               : "memory");
}

__device__ __forceinline__ float adam_update(float g, float& w, float& mi, float& vi,
                                             const ArAdamParams& p, float inv_c1, float inv_sqrt_c2) {
  mi = p.beta1 * mi + (1.f - p.beta1) * g;
  vi = p.beta2 * vi + (1.f - p.beta2) * g * g;
  w -= p.lr * p.weight_decay * w;
  w -= p.lr * (mi * inv_c1) / (sqrtf(vi) * inv_sqrt_c2 + p.eps);
  return w;
}

__global__ void __launch_bounds__(256)
allreduce_adam_kernel(const ArAdamParams p) {
  __shared__ int abort_smem;
  if (threadIdx.x == 0) abort_smem = 0;
  __syncthreads();
  AbortCtx ctx{p.err, &abort_smem};
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[3 * blockIdx.x] = globaltimer_ns();

  // ---- phase 0: every rank's gradients are complete ---------------------------------
  if (p.sync_mode) {
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
      __threadfence_system();
      st_release_sys(p.flags[threadIdx.x] + p.rank, p.epoch);
    }
    if (threadIdx.x < p.world) {
      wait_flag_ge(p.flags[p.rank] + threadIdx.x, p.epoch, ctx, p.wait_ns);
    }
    __syncthreads();
  }

  if (p.trace != nullptr && threadIdx.x == 0) p.trace[3 * blockIdx.x + 1] = globaltimer_ns();
  if (!aborted(ctx)) {
    const ArAdamWorkItem item = p.items[blockIdx.x];
    const ArAdamChunk c = p.chunks[item.chunk];
    const float inv_c1 = 1.f / p.bias_c1;
    const float inv_sqrt_c2 = rsqrtf(p.bias_c2);
    // every chunk is cut in `world` slices of whole 4-element groups (ld and offsets are
    // multiples of 4); the work items of this launch cover slice `rank` of every chunk
    const bool aligned4 = ((c.cols | c.col0 | c.state) & 3) == 0;
    const long long lo4 = item.first >> 2, hi4 = (item.first + item.count) >> 2;
    for (long long i4 = lo4 + threadIdx.x; i4 < hi4; i4 += 256) {
      const long long e = c.offset + (i4 << 2);
      float4 g;
      if (p.use_multimem) {
        g = multimem_ld_reduce_f32x4(p.grad_mc + e);
        multimem_st_f32x4(p.grad_mc + e, make_float4(0.f, 0.f, 0.f, 0.f));
      } else {
        // all ranks' loads are issued before the first use: a peer load takes microseconds,
        // and one after the other they would bound the kernel by latency
        uint4 t[kMaxRanks];
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < p.world) t[r] = ld_global_v4(p.grad[r] + e);
        g = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {  // fixed rank order: bitwise identical on every rank
          if (r < p.world) {
            g.x += __uint_as_float(t[r].x);
            g.y += __uint_as_float(t[r].y);
            g.z += __uint_as_float(t[r].z);
            g.w += __uint_as_float(t[r].w);
            *reinterpret_cast<float4*>(p.grad[r] + e) = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
      }
      float gv[4] = {g.x * p.grad_scale, g.y * p.grad_scale, g.z * p.grad_scale, g.w * p.grad_scale};
      // 32-bit arithmetic: the arena builder rejects regions of 2^31 elements or more
      const unsigned e32 = unsigned(i4) << 2;
      const unsigned row32 = e32 / unsigned(c.ld);
      const long long col0 = e32 - row32 * unsigned(c.ld);
      const long long row = row32;
      if (col0 + 4 <= c.col0 || col0 >= c.col0 + c.cols) continue;  // padding: cleared only
      // optimizer state is dense over the trainable window: (row, col) -> state + row*cols + col-col0
      const long long s0 = c.state + row * c.cols + (col0 - c.col0);
      float wv[4], mv[4], vv[4];
      if (aligned4) {  // the whole group is inside the window and 16-byte aligned
        const float4 w4 = *reinterpret_cast<const float4*>(p.master + s0);
        const float4 m4 = *reinterpret_cast<const float4*>(p.m + s0);
        const float4 v4 = *reinterpret_cast<const float4*>(p.v + s0);
        wv[0] = w4.x, wv[1] = w4.y, wv[2] = w4.z, wv[3] = w4.w;
        mv[0] = m4.x, mv[1] = m4.y, mv[2] = m4.z, mv[3] = m4.w;
        vv[0] = v4.x, vv[1] = v4.y, vv[2] = v4.z, vv[3] = v4.w;
#pragma unroll
        for (int j = 0; j < 4; ++j) adam_update(gv[j], wv[j], mv[j], vv[j], p, inv_c1, inv_sqrt_c2);
        *reinterpret_cast<float4*>(p.master + s0) = make_float4(wv[0], wv[1], wv[2], wv[3]);
        *reinterpret_cast<float4*>(p.m + s0) = make_float4(mv[0], mv[1], mv[2], mv[3]);
        *reinterpret_cast<float4*>(p.v + s0) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      } else {
        const uint2 cur = *reinterpret_cast<const uint2*>(p.work[p.rank] + e);
        const float2 c01 = unpack_bf16x2(cur.x), c23 = unpack_bf16x2(cur.y);
        wv[0] = c01.x, wv[1] = c01.y, wv[2] = c23.x, wv[3] = c23.y;  // padding keeps its value
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const long long col = col0 + j;
          if (col < c.col0 || col >= c.col0 + c.cols) continue;
          float w = p.master[s0 + j], mi = p.m[s0 + j], vi = p.v[s0 + j];
          adam_update(gv[j], w, mi, vi, p, inv_c1, inv_sqrt_c2);
          p.master[s0 + j] = w, p.m[s0 + j] = mi, p.v[s0 + j] = vi;
          wv[j] = w;
        }
      }
      const uint32_t lo = pack_bf16x2(wv[0], wv[1]), hi = pack_bf16x2(wv[2], wv[3]);
      if (p.use_multimem) {
        multimem_st_b32x2(p.work_mc + e, lo, hi);
      } else {
        for (int r = 0; r < p.world; ++r)
          *reinterpret_cast<uint2*>(p.work[r] + e) = make_uint2(lo, hi);
      }
    }
  }

  // ---- phase 2: everyone's weights are written before this kernel ends ---------------
  if (p.sync_mode) {
    __threadfence_system();
    __syncthreads();
    __shared__ int is_last;
    if (threadIdx.x == 0) {
      const unsigned int prev = atomicAdd(p.done_counter, 1u);
      is_last = (prev == gridDim.x - 1);
    }
    __syncthreads();
    if (is_last) {
      if (threadIdx.x < p.world) {
        __threadfence_system();
        st_release_sys(p.flags[threadIdx.x] + kMaxRanks + p.rank, p.epoch);
        wait_flag_ge(p.flags[p.rank] + kMaxRanks + threadIdx.x, p.epoch, ctx, p.wait_ns);
      }
      if (threadIdx.x == 0) *p.done_counter = 0u;
    }
  }
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[3 * blockIdx.x + 2] = globaltimer_ns();
}

}  // namespace lf

using namespace lf;

typedef struct LfArAdamArgs {
  const void* chunks;
  const void* items;   // ArAdamWorkItem[num_items] on the device
  long long num_items;
  void* grad[8];
  void* work[8];
  void* grad_mc;
  void* work_mc;
  void* master;
  void* m;
  void* v;
  void* flags[8];
  void* done_counter;
  void* err;
  void* stream;
  int num_chunks, rank, world, epoch, sync_mode, use_multimem, step;
  int wait_ms;  // limit of the cross-rank flag waits in milliseconds; 0 = the 10 s default
  float lr, beta1, beta2, eps, weight_decay, grad_scale;
  void* trace;  // optional device uint64 [num_items, 3]: entry / peers ready / exit stamps in ns
} LfArAdamArgs;

extern "C" int lf_allreduce_adam(const LfArAdamArgs* a) {
  if (a == nullptr || a->num_chunks <= 0 || a->num_items <= 0) return 0;
  if (a->world < 1 || a->world > kMaxRanks || a->rank < 0 || a->rank >= a->world) return -1;
  ArAdamParams p;
  p.chunks = (const ArAdamChunk*)a->chunks;
  p.items = (const ArAdamWorkItem*)a->items;
  p.num_chunks = a->num_chunks;
  p.rank = a->rank;
  p.world = a->world;
  for (int r = 0; r < kMaxRanks; ++r) {
    p.grad[r] = (float*)a->grad[r];
    p.work[r] = (__nv_bfloat16*)a->work[r];
    p.flags[r] = (int*)a->flags[r];
  }
  p.grad_mc = (float*)a->grad_mc;
  p.work_mc = (__nv_bfloat16*)a->work_mc;
  p.master = (float*)a->master;
  p.m = (float*)a->m;
  p.v = (float*)a->v;
  p.epoch = a->epoch;
  p.sync_mode = a->sync_mode;
  p.use_multimem = (a->use_multimem && a->grad_mc != nullptr && a->work_mc != nullptr) ? 1 : 0;
  p.done_counter = (unsigned int*)a->done_counter;
  p.lr = a->lr;
  p.beta1 = a->beta1;
  p.beta2 = a->beta2;
  p.eps = a->eps;
  p.weight_decay = a->weight_decay;
  p.bias_c1 = 1.f - powf(a->beta1, (float)a->step);
  p.bias_c2 = 1.f - powf(a->beta2, (float)a->step);
  p.grad_scale = a->grad_scale;
  p.err = (int*)a->err;
  p.trace = (unsigned long long*)a->trace;
  p.wait_ns = a->wait_ms > 0 ? (unsigned long long)a->wait_ms * 1000000ull : kPeerWaitNs;
  if (p.sync_mode && p.done_counter == nullptr) return -2;
  // Blocks only ever wait on flags written by other GPUs, never on sibling blocks, so the
  // grid may exceed what is resident at once.
  allreduce_adam_kernel<<<(unsigned)a->num_items, 256, 0, (cudaStream_t)a->stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
