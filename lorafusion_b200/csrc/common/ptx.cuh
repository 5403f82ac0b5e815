// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05
// (TMEM alloc / MMA / commit / ld / st), shared-memory matrix descriptors, and the
// bounded-wait + error-word convention every kernel in this library follows.
//
// Bounded waits: no spin in this library is unbounded.  A wait that exceeds its time
// limit records a code in a global error word, raises a CTA-wide abort flag in shared
// memory, and returns false; every role loop then falls through to the common teardown
// (settle in-flight copies, free TMEM, return) so the context stays usable.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lf {

// ----------------------------------------------------------------------------------
// error codes written to the global error word (first writer wins)
// ----------------------------------------------------------------------------------
enum ErrCode : int {
  ERR_NONE = 0,
  ERR_WAIT_FULL = 1,        // consumer timed out waiting for a TMA stage
  ERR_WAIT_EMPTY = 2,       // producer timed out waiting for a free stage
  ERR_WAIT_TMEM_FULL = 3,   // epilogue timed out waiting for the accumulator
  ERR_WAIT_TMEM_EMPTY = 4,  // MMA issuer timed out waiting for a drained accumulator
  ERR_WAIT_READY = 5,       // MMA issuer timed out waiting for a transformed stage
  ERR_WAIT_PEER = 6,        // timed out on a flag another GPU (or another CTA) writes
  ERR_BAD_ARG = 7,
  ERR_WAIT_MISC = 8,
};

constexpr unsigned long long kLocalWaitNs = 2000000000ull;   // 2 s for intra-kernel barriers
constexpr unsigned long long kPeerWaitNs = 10000000000ull;   // 10 s for cross-GPU flags

struct AbortCtx {
  int* err_word;            // global, may be nullptr
  volatile int* abort_smem; // CTA-wide flag in shared memory
  // Limit of the intra-kernel waits.  A kernel whose TMA producer waits for another GPU (the
  // tensor-parallel fusions) sets it above the peer limit: its consumers must not give up on a
  // stage while the producer is still legitimately waiting for a late peer.
  unsigned long long local_wait_ns = kLocalWaitNs;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void raise_abort(const AbortCtx& ctx, int code) {
  if (ctx.err_word != nullptr) atomicCAS(ctx.err_word, 0, code);
  *ctx.abort_smem = 1;
  __threadfence_block();
}

__device__ __forceinline__ bool aborted(const AbortCtx& ctx) { return *ctx.abort_smem != 0; }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait on an mbarrier phase.  Returns false after an abort (own timeout or
// another role's); the caller must leave its loop and go to teardown.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const AbortCtx& ctx,
                                          int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 0xff) == 0) {
      if (aborted(ctx)) return false;
      if (globaltimer_ns() - t0 > ctx.local_wait_ns) {
        raise_abort(ctx, code);
        return false;
      }
    }
  }
}

// Named barrier over `NTHREADS` threads that also ANDs a predicate: every participant gets
// the same answer.  Used where a group of warps must agree on "go on" / "abort" before a later
// named barrier: a thread that saw the abort flag a few polls earlier than its neighbours
// would otherwise leave while they wait for its arrival.
template <int ID, int NTHREADS>
__device__ __forceinline__ bool named_bar_and(bool pred) {
  uint32_t out;
  asm volatile(
      "{\n"
      ".reg .pred pin, pout;\n"
      "setp.ne.u32 pin, %1, 0;\n"
      "bar.red.and.pred pout, %2, %3, pin;\n"
      "selp.u32 %0, 1, 0, pout;\n"
      "}\n"
      : "=r"(out)
      : "r"(uint32_t(pred)), "n"(ID), "n"(NTHREADS)
      : "memory");
  return out != 0;
}

// Same with the barrier id and the thread count in registers (e.g. one barrier per pair of warps).
__device__ __forceinline__ bool named_bar_and_id(int id, int nthreads, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n"
      ".reg .pred pin, pout;\n"
      "setp.ne.u32 pin, %1, 0;\n"
      "bar.red.and.pred pout, %2, %3, pin;\n"
      "selp.u32 %0, 1, 0, pout;\n"
      "}\n"
      : "=r"(out)
      : "r"(uint32_t(pred)), "r"(id), "r"(nthreads)
      : "memory");
  return out != 0;
}

// ----------------------------------------------------------------------------------
// cross-CTA / cross-GPU flag waits (system scope, acquire)
// ----------------------------------------------------------------------------------
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Wait until *flag >= target.  limit_ns bounds the spin.
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int target, const AbortCtx& ctx,
                                             unsigned long long limit_ns = kPeerWaitNs) {
  if (ld_acquire_sys(flag) >= target) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (ld_acquire_sys(flag) >= target) return true;
    if ((it & 0x3f) == 0) {
      if (aborted(ctx)) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        raise_abort(ctx, ERR_WAIT_PEER);
        return false;
      }
      __nanosleep(64);
    }
  }
}

// ----------------------------------------------------------------------------------
// proxy fences
// ----------------------------------------------------------------------------------
// Generic-proxy writes to shared memory -> visible to the async proxy (TMA / tcgen05).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// ----------------------------------------------------------------------------------
// TMA (tiled tensor maps).  The innermost coordinate times the element size must be a
// multiple of 16 bytes; every call site in this library passes x as a multiple of 8
// bf16 elements (or 16 bytes) by construction.
// ----------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int x,
                                             int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(m), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------------
// tcgen05 / TMEM
// ----------------------------------------------------------------------------------
// One full warp allocates `ncols` (power of two, 32..512) TMEM columns; the base
// address is written to *smem_dst.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once all tcgen05.mma issued so far by this thread complete.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::
                   "r"(smem_u32(bar))
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_bf16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor for kind::f16, bf16 x bf16 -> fp32, M x N, per-operand major
// (0 = K-major, 1 = MN-major).
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int a_mn, int b_mn) {
  return (1u << 4)                       // D format: fp32
         | (1u << 7)                     // A format: bf16
         | (1u << 10)                    // B format: bf16
         | (uint32_t(a_mn) << 15)        // A major
         | (uint32_t(b_mn) << 16)        // B major
         | (uint32_t(N >> 3) << 17)      // N / 8
         | (uint32_t(M >> 4) << 24);     // M / 16
}

// Shared-memory matrix descriptor, 128-byte swizzle, bf16.
//  K-major tile  : rows of 64 elements (128 B), 8-row groups 1024 B apart (SBO); LBO unused.
//  MN-major tile : blocks of [64 k-rows x 64 mn-elements] (8 KB); inside a block 8-row
//                  groups are 1024 B apart (SBO); consecutive 64-element MN chunks are
//                  `lbo_bytes` apart (LBO).
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3ffff) >> 4);
  d |= uint64_t((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= uint64_t(1) << 46;  // descriptor version for sm_100
  d |= uint64_t(2) << 61;  // SWIZZLE_128B
  return d;
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp receives columns
// [col, col+32) of TMEM lane (lane_base + i).  taddr = (lane << 16) | column.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
      "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
      "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
      "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------------
// small helpers
// ----------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t v) {
  __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&v);
  return __bfloat1622float2(b);
}
// Coherent 16-byte load (never the read-only path): for buffers other GPUs write into while
// this kernel runs; visibility comes from the acquire on the flag that guards them.
__device__ __forceinline__ uint4 ld_global_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p)
               : "memory");
  return r;
}
__device__ __forceinline__ void st_global_v4(void* p, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

}  // namespace lf

// ----------------------------------------------------------------------------------
// thread-block clusters and CTA pairs (tcgen05 cta_group::2)
// ----------------------------------------------------------------------------------
namespace lf {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `p` (an address in this CTA's shared memory) as seen in CTA
// `cta_rank` of the cluster: same offset, other CTA.
__device__ __forceinline__ uint32_t mapa_shared(const void* p, uint32_t cta_rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(p)), "r"(cta_rank));
  return out;
}
// Arrive on an mbarrier that may live in another CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// TMEM allocation shared by a CTA pair: the same warp index of BOTH CTAs executes it.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
// Pair MMA: D (256 x N over both CTAs' TMEM) (+)= A (128 rows from each CTA's smem) *
// B (N / 2 rows from each CTA's smem).  Issued by one thread of the leader CTA only.
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                  uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Completion of all pair MMAs issued so far -> one arrival on the mbarrier at the given
// shared::cluster address (own CTA or the peer).
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   cluster_addr)
               : "memory");
}
// TMA load issued by either CTA of a pair whose byte count is credited to an mbarrier
// given by its shared::cluster address (the leader CTA's "stage full" barrier).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m,
                                                 uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(m), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}

}  // namespace lf
