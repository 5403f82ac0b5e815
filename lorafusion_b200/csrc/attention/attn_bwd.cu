// Backward of the causal varlen GQA attention (head_dim 128) on sm_100a, as three kernels:
//   1. attn_delta_kernel : delta[h, m] = sum_d O[m, h, d] * dO[m, h, d]
//   2. attn_dq_kernel    : one CTA per (query tile, kv head) walks the group's query heads and
//                          for each loops over key tiles,
//                          recomputes P from the saved log-sum-exp and accumulates
//                          dQ += dS K in TMEM.
//   3. attn_dkdv_kernel  : one CTA per (key tile, kv head) loops over the query heads of
//                          its group and the query tiles at or below the diagonal and
//                          accumulates dV += P^T dO and dK += dS^T Q in TMEM.
// Splitting dQ from dK/dV costs two extra recomputation GEMMs per tile pair but keeps
// every output element owned by exactly one CTA: no atomics, bitwise-reproducible
// gradients.  Gradients are written into a buffer with the layout of the packed QKV
// projection so that the rotary backward and the QKV-linear backward consume it in place.
// (The reference calls FlashAttention-2's backward through autograd.)
#include <stdio.h>

#include "../common/launch.h"
#include "../common/tensormap.h"
#include "attn_common.cuh"

namespace lf {

struct AttnBwdParams {
  const int4* tiles;
  int num_tiles;
  int Hq, Hkv;
  int q_col0, k_col0, v_col0;
  __nv_bfloat16* dqkv;
  long long ld_qkv;
  const float* lse;
  const float* delta;
  long long M_total;
  float scale, scale_log2e;
  int* err;
};

constexpr int BWD_SMEM = ATT_TILE_BYTES * 7 + 256 + 1024;
// TMA warp, MMA warp and 8 element-wise warps: two threads per row of S / dP, 64 columns
// each (warps 2-5 columns 0-63, warps 6-9 columns 64-127; a warp reads the TMEM lane
// quarter warp % 4).  The backward needs no row reductions, so the halves never talk.
constexpr int BWD_THREADS = 64 + 256;

// ----------------------------------------------------------------------------------
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o,
                                  const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                                  long long M, int Hq, long long ld) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= M * Hq) return;
  const long long m = w / Hq;
  const int h = int(w % Hq);
  const uint2 a = *reinterpret_cast<const uint2*>(o + m * ld + h * ATT_D + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(d_o + m * ld + h * ATT_D + lane * 4);
  const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y);
  const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y);
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) delta[(long long)h * M + m] = s;
}

// ----------------------------------------------------------------------------------
// dQ
// ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_dq_kernel(const AttnBwdParams p, const __grid_constant__ CUtensorMap tmQKV,
               const __grid_constant__ CUtensorMap tmDO) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + ATT_TILE_BYTES;
  // Three K stages and one V stage: K of a tile is read twice (S early, dQ last), V once (dP), so
  // a V slot is free early and one suffices, while the K of tile J + 2 must already be on its way
  // during tile J (with two K stages its load could only start after dQ of tile J, and the load
  // latency sat between two tiles).
  uint8_t* sK3 = smem + 2 * ATT_TILE_BYTES;  // K stage s at s * 32 KB
  uint8_t* sV = smem + 5 * ATT_TILE_BYTES;
  uint8_t* sDS = smem + 6 * ATT_TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 7 * ATT_TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [3]
  uint64_t* v_full = bars + 4;
  uint64_t* v_empty = bars + 15;
  uint64_t* k_empty = bars + 16;  // [3]
  // S has two TMEM buffers and barriers of its own, dP one: S of tile J + 1 is issued while the
  // element-wise warps still work on tile J, and they turn it into P (the exponentials) while the
  // tensor pipe produces dP of the same tile.  With S and dP behind one barrier the tensor pipe and
  // the element-wise warps strictly took turns.
  uint64_t* s_full = bars + 5;     // [2]
  uint64_t* ds_full = bars + 7;
  uint64_t* dq_done = bars + 8;
  uint64_t* q_empty = bars + 9;    // every S / dP product of the current head has completed: sQ, sDO may be refilled
  uint64_t* dq_empty = bars + 10;  // the finished dQ has been read: the next head may overwrite the accumulator
  uint64_t* s_empty = bars + 11;   // [2]
  uint64_t* dp_full = bars + 13;
  uint64_t* dp_empty = bars + 14;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  AbortCtx ctx{p.err, abort_flag};
  const int4 tile = p.tiles[blockIdx.x];
  const int row0 = tile.x, rows = tile.y, seq_row0 = tile.z;
  // One CTA per (query tile, KV head): it walks the query heads of the group one after the
  // other, so TMEM, barriers and the K/V ring are set up once (see attn_fwd.cu).
  const int g = blockIdx.y;
  const int group = p.Hq / p.Hkv;
  const int h0 = g * group;
  const int n_kv = (row0 - seq_row0) / ATT_TILE + 1;
  const int total = group * n_kv;  // flat (head, key tile) sequence J = hi * n_kv + j

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 3; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    // one arrival per element-wise warp (lane 0 after __syncwarp): 256 arrivals on one word serialise
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 8);
    }
    mbar_init(dp_full, 1);
    mbar_init(dp_empty, 8);
    mbar_init(ds_full, 8);
    mbar_init(dq_done, 1);
    mbar_init(q_empty, 1);
    mbar_init(dq_empty, 8);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 128};
  const uint32_t tDP = tmem_base + 256, tDQ = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      for (int hi = 0; ok && hi < group; ++hi) {
        for (int j = 0; j < n_kv; ++j) {
          const int J = hi * n_kv + j;
          const int s = J % 3;
          if (!mbar_wait(&k_empty[s], ((J / 3) & 1) ^ 1, ctx, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&k_full[s], ATT_TILE_BYTES);
          att_load_tile(sK3 + s * ATT_TILE_BYTES, &tmQKV, &k_full[s], p.k_col0 + g * ATT_D, seq_row0 + j * ATT_TILE);
          if (j == 0) {
            if (hi > 0 && !mbar_wait(q_empty, (hi - 1) & 1, ctx, ERR_WAIT_EMPTY)) {
              ok = false;
              break;
            }
            mbar_expect_tx(q_full, 2 * ATT_TILE_BYTES);
            att_load_tile(sQ, &tmQKV, q_full, p.q_col0 + (h0 + hi) * ATT_D, row0);
            att_load_tile(sDO, &tmDO, q_full, (h0 + hi) * ATT_D, row0);
          }
          if (!mbar_wait(v_empty, (J & 1) ^ 1, ctx, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(v_full, ATT_TILE_BYTES);
          att_load_tile(sV, &tmQKV, v_full, p.v_col0 + g * ATT_D, seq_row0 + j * ATT_TILE);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // Issue order: S(0), dP(0), then per tile J: S(J + 1), dP(J + 1) (both as soon as their TMEM
      // buffers have been read), [dS(J) ready] dQ(J).
      auto issue_s = [&](int J1) -> bool {   // S of tile J1 into its buffer; K (and for a new head Q) must have landed
        const int hi1 = J1 / n_kv, j1 = J1 - hi1 * n_kv;
        const int b1 = J1 & 1;
        const uint32_t ph = (J1 >> 1) & 1;
        if ((j1 == 0 && !mbar_wait(q_full, hi1 & 1, ctx, ERR_WAIT_FULL)) ||
            !mbar_wait(&k_full[J1 % 3], (J1 / 3) & 1, ctx, ERR_WAIT_FULL) ||
            !mbar_wait(&s_empty[b1], ph ^ 1, ctx, ERR_WAIT_TMEM_EMPTY))
          return false;
        tc_fence_after_sync();
        att_mma_kk(tS[b1], smem_u32(sQ), smem_u32(sK3 + (J1 % 3) * ATT_TILE_BYTES), false);
        tc_commit(&s_full[b1]);
        return true;
      };
      auto issue_dp = [&](int J1) -> bool {  // dP of tile J1 (dO of its head was awaited by issue_s(J1))
        const int hi1 = J1 / n_kv, j1 = J1 - hi1 * n_kv;
        if (!mbar_wait(v_full, J1 & 1, ctx, ERR_WAIT_FULL) ||
            !mbar_wait(dp_empty, (J1 & 1) ^ 1, ctx, ERR_WAIT_TMEM_EMPTY))
          return false;
        tc_fence_after_sync();
        att_mma_kk(tDP, smem_u32(sDO), smem_u32(sV), false);
        tc_commit(dp_full);
        tc_commit(v_empty);
        if (j1 == n_kv - 1) tc_commit(q_empty);  // last use of this head's Q and dO
        return true;
      };
      bool ok = total > 0 && issue_s(0) && issue_dp(0);
      for (int J = 0; ok && J < total; ++J) {
        const int hi = J / n_kv, j = J - hi * n_kv;
        const int s = J % 3;
        const uint32_t sK = smem_u32(sK3 + s * ATT_TILE_BYTES);
        if (J + 1 < total && !(issue_s(J + 1) && issue_dp(J + 1))) {
          ok = false;
          break;
        }
        if (!mbar_wait(ds_full, J & 1, ctx, ERR_WAIT_READY) ||
            (j == 0 && hi > 0 && !mbar_wait(dq_empty, (hi - 1) & 1, ctx, ERR_WAIT_TMEM_EMPTY))) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        att_mma_kmn(tDQ, smem_u32(sDS), sK, j > 0);
        tc_commit(&k_empty[s]);
        tc_commit(dq_done);
      }
    }
  } else {
    const int q = warp & 3;
    const int c0 = ((warp - 2) >> 2) * 64;
    const int r = q * 32 + lane;
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    const long long grow = (long long)row0 + r;
    const bool row_valid = r < rows;
    bool ok = true;
    for (int hi = 0; ok && hi < group; ++hi) {
      const int h = h0 + hi;
      const float lse2 = row_valid ? p.lse[(long long)h * p.M_total + grow] * 1.4426950408889634f : 0.f;
      const float dlts = row_valid ? p.delta[(long long)h * p.M_total + grow] * p.scale : 0.f;  // delta * softmax scale
      for (int j = 0; j < n_kv; ++j) {
        const int J = hi * n_kv + j;
        const int sb = J & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&s_full[sb], (J >> 1) & 1, ctx, ERR_WAIT_TMEM_FULL))) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const bool diag = (j == n_kv - 1);
        // P of this thread's 64 columns from S alone, while the tensor pipe still produces dP
        float pv[64];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t(&dst)[32] = *reinterpret_cast<uint32_t(*)[32]>(&pv[cc * 32]);
          tmem_ld_32x32b_x32(tS[sb] + lane_addr + c0 + cc * 32, dst);
        }
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[sb]);
#pragma unroll
        for (int i = 0; i < 64; ++i) pv[i] = fast_exp2(pv[i] * p.scale_log2e - lse2);
        if (diag || rows < ATT_TILE) {   // uniform: only the diagonal tile and a ragged query tile mask anything
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (!row_valid || (diag && c0 + i > r)) pv[i] = 0.f;
        }
        if (!__all_sync(0xffffffffu, mbar_wait(dp_full, J & 1, ctx, ERR_WAIT_TMEM_FULL))) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {   // dS in registers (over P); dP's buffer is free right after
          uint32_t dv[32];
          tmem_ld_32x32b_x32(tDP + lane_addr + c0 + cc * 32, dv);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) pv[cc * 32 + i] *= fmaf(__uint_as_float(dv[i]), p.scale, -dlts);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(dp_empty);
        // sDS is still being read by the previous tile's dQ product (for j == 0 the previous
        // head's final store has already waited for it)
        if (j > 0 && !__all_sync(0xffffffffu, mbar_wait(dq_done, (J - 1) & 1, ctx, ERR_WAIT_MISC))) {
          ok = false;
          break;
        }
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          float(&src)[32] = *reinterpret_cast<float(*)[32]>(&pv[cc * 32]);
          att_store_row_chunk(sDS, r, c0 + cc * 32, src);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(ds_full);
      }
      if (!ok) break;
      if (!__all_sync(0xffffffffu, mbar_wait(dq_done, (hi * n_kv + n_kv - 1) & 1, ctx, ERR_WAIT_MISC))) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      __nv_bfloat16* orow = p.dqkv + grow * p.ld_qkv + p.q_col0 + h * ATT_D + c0;
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tDQ + lane_addr + c0 + cc * 32, o);
        tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int gq = 0; gq < 4; ++gq)
            st_global_v4(orow + cc * 32 + gq * 8,
                         pack_bf16x2(__uint_as_float(o[gq * 8 + 0]), __uint_as_float(o[gq * 8 + 1])),
                         pack_bf16x2(__uint_as_float(o[gq * 8 + 2]), __uint_as_float(o[gq * 8 + 3])),
                         pack_bf16x2(__uint_as_float(o[gq * 8 + 4]), __uint_as_float(o[gq * 8 + 5])),
                         pack_bf16x2(__uint_as_float(o[gq * 8 + 6]), __uint_as_float(o[gq * 8 + 7])));
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_empty);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ----------------------------------------------------------------------------------
// dK, dV
// ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_dkdv_kernel(const AttnBwdParams p, const __grid_constant__ CUtensorMap tmQKV,
                 const __grid_constant__ CUtensorMap tmDO) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + ATT_TILE_BYTES;
  uint8_t* sQD = smem + 2 * ATT_TILE_BYTES;  // stage s: Q, dO
  uint8_t* sPD = smem + 6 * ATT_TILE_BYTES;  // P, then dS
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 7 * ATT_TILE_BYTES);
  uint64_t* kv_full = bars;
  uint64_t* qd_full = bars + 1;
  uint64_t* qd_empty = bars + 3;
  // S and dP have barriers of their own (one TMEM buffer each): S of the next iteration is issued
  // as soon as P of this one has been formed, so the element-wise warps turn it into P while the
  // tensor pipe runs dK of this iteration and dP of the next.
  uint64_t* s_full = bars + 5;
  uint64_t* s_empty = bars + 6;
  uint64_t* p_full = bars + 7;
  uint64_t* dv_done = bars + 8;
  uint64_t* ds_full = bars + 9;
  uint64_t* dk_done = bars + 10;
  uint64_t* dp_full = bars + 11;
  uint64_t* dp_empty = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  AbortCtx ctx{p.err, abort_flag};
  const int4 tile = p.tiles[blockIdx.x];
  const int row0 = tile.x, rows = tile.y, seq_row0 = tile.z, seq_rows = tile.w;
  const int g = blockIdx.y;
  const int group = p.Hq / p.Hkv;
  const int i_kv = (row0 - seq_row0) / ATT_TILE;
  const int n_q_tiles = (seq_rows + ATT_TILE - 1) / ATT_TILE;
  const int per_head = n_q_tiles - i_kv;
  const int n_it = per_head * group;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qd_full[i], 1);
      mbar_init(&qd_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 8);  // one arrival per element-wise warp
    mbar_init(dp_full, 1);
    mbar_init(dp_empty, 8);
    mbar_init(p_full, 8);
    mbar_init(dv_done, 1);
    mbar_init(ds_full, 8);
    mbar_init(dk_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDV = tmem_base + 256, tDK = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * ATT_TILE_BYTES);
      att_load_tile(sK, &tmQKV, kv_full, p.k_col0 + g * ATT_D, row0);
      att_load_tile(sV, &tmQKV, kv_full, p.v_col0 + g * ATT_D, row0);
      for (int it = 0; it < n_it; ++it) {
        const int s = it & 1;
        const int h = g * group + it / per_head;
        const int qrow0 = seq_row0 + (i_kv + it % per_head) * ATT_TILE;
        if (!mbar_wait(&qd_empty[s], ((it >> 1) & 1) ^ 1, ctx, ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&qd_full[s], 2 * ATT_TILE_BYTES);
        uint8_t* sQ = sQD + s * 2 * ATT_TILE_BYTES;
        att_load_tile(sQ, &tmQKV, &qd_full[s], p.q_col0 + h * ATT_D, qrow0);
        att_load_tile(sQ + ATT_TILE_BYTES, &tmDO, &qd_full[s], h * ATT_D, qrow0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // Issue order per iteration: [P ready] dV(it), S(it + 1), dP(it + 1), [dS ready] dK(it).
      auto issue_s = [&](int i1) -> bool {   // S = Q K^T of iteration i1 (its Q / dO stage must have landed)
        const int s1 = i1 & 1;
        if (!mbar_wait(&qd_full[s1], (i1 >> 1) & 1, ctx, ERR_WAIT_FULL) ||
            !mbar_wait(s_empty, (i1 & 1) ^ 1, ctx, ERR_WAIT_TMEM_EMPTY))
          return false;
        tc_fence_after_sync();
        att_mma_kk(tS, smem_u32(sQD + s1 * 2 * ATT_TILE_BYTES), smem_u32(sK), false);
        tc_commit(s_full);
        return true;
      };
      auto issue_dp = [&](int i1) -> bool {  // dP = dO V^T of iteration i1 (stage awaited by issue_s(i1))
        if (!mbar_wait(dp_empty, (i1 & 1) ^ 1, ctx, ERR_WAIT_TMEM_EMPTY)) return false;
        tc_fence_after_sync();
        att_mma_kk(tDP, smem_u32(sQD + (i1 & 1) * 2 * ATT_TILE_BYTES + ATT_TILE_BYTES), smem_u32(sV), false);
        tc_commit(dp_full);
        return true;
      };
      bool ok = mbar_wait(kv_full, 0, ctx, ERR_WAIT_FULL);
      ok = ok && n_it > 0 && issue_s(0) && issue_dp(0);
      for (int it = 0; ok && it < n_it; ++it) {
        const int s = it & 1;
        const uint32_t sQ = smem_u32(sQD + s * 2 * ATT_TILE_BYTES);
        const uint32_t sDO = sQ + ATT_TILE_BYTES;
        if (!mbar_wait(p_full, it & 1, ctx, ERR_WAIT_READY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        att_mma_mnmn(tDV, smem_u32(sPD), sDO, it > 0);
        tc_commit(dv_done);
        if (it + 1 < n_it && !(issue_s(it + 1) && issue_dp(it + 1))) {
          ok = false;
          break;
        }
        if (!mbar_wait(ds_full, it & 1, ctx, ERR_WAIT_READY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        att_mma_mnmn(tDK, smem_u32(sPD), sQ, it > 0);
        tc_commit(&qd_empty[s]);
        tc_commit(dk_done);
      }
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int c0 = half * 64;
    const int r = q * 32 + lane;  // query row inside the current query tile
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    bool ok = true;
    // log-sum-exp and delta of this thread's query row: loaded one iteration ahead, so that the
    // two global loads are not on the critical path of every iteration
    auto row_stats = [&](int i1, float& lse2_out, float& dlt_out) {
      const int h1 = g * group + i1 / per_head;
      const int jq1 = i_kv + i1 % per_head;
      const bool valid1 = r < min(ATT_TILE, seq_rows - jq1 * ATT_TILE);
      const long long grow1 = (long long)seq_row0 + jq1 * ATT_TILE + r;
      lse2_out = valid1 ? p.lse[(long long)h1 * p.M_total + grow1] * 1.4426950408889634f : 0.f;
      dlt_out = valid1 ? p.delta[(long long)h1 * p.M_total + grow1] * p.scale : 0.f;
    };
    float lse2_next = 0.f, dlts_next = 0.f;
    if (n_it > 0) row_stats(0, lse2_next, dlts_next);
    for (int it = 0; it < n_it; ++it) {
      const int jq = i_kv + it % per_head;
      const int q_valid = min(ATT_TILE, seq_rows - jq * ATT_TILE);
      const bool row_valid = r < q_valid;
      const bool diag = (jq == i_kv);
      const bool need_mask = diag || q_valid < ATT_TILE;   // uniform over the CTA
      const float lse2 = lse2_next, dlts = dlts_next;       // dlts = delta * softmax scale
      if (it + 1 < n_it) row_stats(it + 1, lse2_next, dlts_next);
      if (!__all_sync(0xffffffffu, mbar_wait(s_full, it & 1, ctx, ERR_WAIT_TMEM_FULL))) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      // P of this thread's 64 columns in registers first; its store waits for the shared P / dS buffer
      float pv[64];
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t(&dst)[32] = *reinterpret_cast<uint32_t(*)[32]>(&pv[cc * 32]);
        tmem_ld_32x32b_x32(tS + lane_addr + c0 + cc * 32, dst);
      }
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty);   // S has been read: the next iteration's S may be issued
#pragma unroll
      for (int i = 0; i < 64; ++i) pv[i] = fast_exp2(pv[i] * p.scale_log2e - lse2);
      if (need_mask) {   // only the diagonal tile and a ragged last query tile have anything to mask
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (!row_valid || (diag && c0 + i > r)) pv[i] = 0.f;
      }
      // sPD still holds dS of the previous iteration until its dK product has read it
      if (it > 0 && !__all_sync(0xffffffffu, mbar_wait(dk_done, (it - 1) & 1, ctx, ERR_WAIT_MISC))) {
        ok = false;
        break;
      }
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        float(&src)[32] = *reinterpret_cast<float(*)[32]>(&pv[cc * 32]);
        att_store_row_chunk(sPD, r, c0 + cc * 32, src);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      // dS of this thread's 64 columns in registers while the dV product still reads P from sPD
      if (!__all_sync(0xffffffffu, mbar_wait(dp_full, it & 1, ctx, ERR_WAIT_TMEM_FULL))) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      // dS = P (.) (dP - delta) * scale, in place over P (fp32; the dV product saw the same P rounded to bf16)
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t dv[32];
        tmem_ld_32x32b_x32(tDP + lane_addr + c0 + cc * 32, dv);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) pv[cc * 32 + i] *= fmaf(__uint_as_float(dv[i]), p.scale, -dlts);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(dp_empty);
      if (!__all_sync(0xffffffffu, mbar_wait(dv_done, it & 1, ctx, ERR_WAIT_MISC))) {
        ok = false;
        break;
      }
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        float(&src)[32] = *reinterpret_cast<float(*)[32]>(&pv[cc * 32]);
        att_store_row_chunk(sPD, r, c0 + cc * 32, src);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (ok && n_it > 0 && __all_sync(0xffffffffu, mbar_wait(dk_done, (n_it - 1) & 1, ctx, ERR_WAIT_MISC))) {
      tc_fence_after_sync();
      const long long grow = (long long)row0 + r;  // key row owned by this thread
      __nv_bfloat16* krow = p.dqkv + grow * p.ld_qkv + p.k_col0 + g * ATT_D;
      __nv_bfloat16* vrow = p.dqkv + grow * p.ld_qkv + p.v_col0 + g * ATT_D;
      // the first half of the warps writes dV, the second dK
#pragma unroll 1
      for (int cc = half * 4; cc < half * 4 + 4; ++cc) {
        uint32_t o[32];
        const bool is_k = cc >= 4;
        tmem_ld_32x32b_x32((is_k ? tDK : tDV) + lane_addr + (cc & 3) * 32, o);
        tmem_ld_wait();
        if (r < rows) {
          __nv_bfloat16* dst = (is_k ? krow : vrow) + (cc & 3) * 32;
#pragma unroll
          for (int gq = 0; gq < 4; ++gq)
            st_global_v4(dst + gq * 8,
                         pack_bf16x2(__uint_as_float(o[gq * 8 + 0]), __uint_as_float(o[gq * 8 + 1])),
                         pack_bf16x2(__uint_as_float(o[gq * 8 + 2]), __uint_as_float(o[gq * 8 + 3])),
                         pack_bf16x2(__uint_as_float(o[gq * 8 + 4]), __uint_as_float(o[gq * 8 + 5])),
                         pack_bf16x2(__uint_as_float(o[gq * 8 + 6]), __uint_as_float(o[gq * 8 + 7])));
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace lf

using namespace lf;

// out / d_out: [M, Hq*128]; qkv and dqkv: [M, ld_qkv]; lse, delta: fp32 [Hq, M]
// (delta is scratch filled here).
extern "C" int lf_attn_bwd(const void* qkv, const void* out, const void* d_out, void* dqkv,
                           long long M, long long ld_qkv, int q_col0, int k_col0, int v_col0, int Hq,
                           int Hkv, const void* tiles, int num_tiles, long long ldo, const float* lse,
                           float* delta, float scale, int* err, void* stream) {
  if (num_tiles <= 0) return 0;
  if (Hq % Hkv != 0) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  CUtensorMap tmQKV, tmDO;
  int rc = make_tmap_2d_b16(&tmQKV, qkv, (uint64_t)M, (uint64_t)ld_qkv, (uint64_t)ld_qkv, 128, 64, true);
  if (rc != 0) return -20 + rc;
  rc = make_tmap_2d_b16(&tmDO, d_out, (uint64_t)M, (uint64_t)Hq * ATT_D, (uint64_t)ldo, 128, 64, true);
  if (rc != 0) return -30 + rc;
  static PerDeviceOnce dq_configured, dkdv_configured;
  if (ensure_max_dynamic_smem(dq_configured, attn_dq_kernel, BWD_SMEM) != cudaSuccess ||
      ensure_max_dynamic_smem(dkdv_configured, attn_dkdv_kernel, BWD_SMEM) != cudaSuccess)
    return -10;
  {
    const long long warps = M * Hq;
    const int block = 256;
    const long long grid = (warps * 32 + block - 1) / block;
    attn_delta_kernel<<<(unsigned)grid, block, 0, st>>>((const __nv_bfloat16*)out,
                                                         (const __nv_bfloat16*)d_out, delta, M, Hq, ldo);
  }
  AttnBwdParams p;
  p.tiles = (const int4*)tiles;
  p.num_tiles = num_tiles;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.q_col0 = q_col0;
  p.k_col0 = k_col0;
  p.v_col0 = v_col0;
  p.dqkv = (__nv_bfloat16*)dqkv;
  p.ld_qkv = ld_qkv;
  p.lse = lse;
  p.delta = delta;
  p.M_total = M;
  p.scale = scale;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.err = err;
  attn_dq_kernel<<<dim3(num_tiles, Hkv), BWD_THREADS, BWD_SMEM, st>>>(p, tmQKV, tmDO);  // walks the group's q heads
  attn_dkdv_kernel<<<dim3(num_tiles, Hkv), BWD_THREADS, BWD_SMEM, st>>>(p, tmQKV, tmDO);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// ------------------------------------------------------------------------------------
// Variant that allocates nothing: the delta scratch lives in the library image.
// See attn_noalloc.h for who needs this and for the rules of use.
// ------------------------------------------------------------------------------------
#include "attn_noalloc.h"

static __device__ __align__(256) float g_noalloc_delta[LF_ATTN_NOALLOC_MAX_DELTA];

namespace {
constexpr int kMaxDevices = 64;
std::atomic<float*> g_noalloc_delta_addr[kMaxDevices];  // zero-initialised (static storage)

// In host code `g_noalloc_delta` is only a handle for the symbol, not a device address;
// the real address has to be asked for once per device, with that device current.
int noalloc_delta_address(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  float* addr = g_noalloc_delta_addr[dev].load(std::memory_order_acquire);
  if (addr == nullptr) {  // two host threads may both look it up: they get the same answer
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_delta) != cudaSuccess || p == nullptr) return -1;
    addr = static_cast<float*>(p);
    g_noalloc_delta_addr[dev].store(addr, std::memory_order_release);
  }
  *out = addr;
  return 0;
}
}  // namespace

extern "C" int lf_attn_bwd_noalloc(const void* qkv, const void* out, const void* d_out, void* dqkv,
                                   long long M, long long ld_qkv, int q_col0, int k_col0, int v_col0,
                                   int Hq, int Hkv, const void* tiles, int num_tiles, long long ldo,
                                   const float* lse, float scale, int* err, void* stream) {
  if (num_tiles <= 0) return 0;
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || M <= 0) return -1;
  if ((long long)Hq * M > (long long)LF_ATTN_NOALLOC_MAX_DELTA) {
    fprintf(stderr,
            "lf_attn_bwd_noalloc: Hq * M = %lld exceeds the built-in scratch of %d floats; use "
            "lf_attn_bwd with a caller-provided delta buffer instead\n",
            (long long)Hq * M, LF_ATTN_NOALLOC_MAX_DELTA);
    return LF_ATTN_NOALLOC_TOO_LARGE;
  }
  float* delta = nullptr;
  if (noalloc_delta_address(&delta) != 0) {
    fprintf(stderr, "lf_attn_bwd_noalloc: could not resolve the scratch symbol on this device\n");
    return LF_ATTN_NOALLOC_SETUP_FAILED;
  }
  // Same launches as lf_attn_bwd, with the built-in array in place of the caller's scratch.
  return lf_attn_bwd(qkv, out, d_out, dqkv, M, ld_qkv, q_col0, k_col0, v_col0, Hq, Hkv, tiles, num_tiles, ldo,
                     lse, delta, scale, err, stream);
}
