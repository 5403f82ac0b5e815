// Causal, variable-length, grouped-query attention forward for head_dim 128 on sm_100a.
// Replaces the FlashAttention-2 varlen call of the reference
// (lorafusion/patch/patch_transformers.py:150-159).
//
// One CTA handles one 128-row query tile of one sequence for one KV head and walks the query
// heads of that head's group one after the other ("persistent" over the group): TMEM, the
// barriers and the K/V ring are set up once, and the next head's Q and first K/V tiles are
// already on their way while the current head is normalised and stored.  With one CTA per
// (tile, query head) the fixed cost per CTA was two thirds of the time on short sequences.
//   warp 0      TMA producer: per head Q, then K and V tiles through two 2-stage rings of their own
//   warp 1      tcgen05.mma issuer: S = Q K^T into one of two TMEM buffers, O += P V
//   warps 2..   softmax: read S from TMEM (FWD_PARTS threads per row, 128 / FWD_PARTS key columns
//               each), online max/sum with lazy rescaling of O (only when the running max grows
//               by more than 2^8), write bf16 P into swizzled shared memory for the second MMA,
//               final normalise.  This role sets the pace of the kernel: its per-tile latency
//               chain, not issue slots, the special-function unit or the tensor pipe (each about
//               one third busy), is the critical path.
// Q/K/V are read straight out of the packed, RoPE-rotated QKV projection with one tensor
// map; O is written token-major [M, Hq * 128]; the log-sum-exp is kept for the backward.
#include <stdio.h>

#include "../common/launch.h"
#include "../common/tensormap.h"
#include "attn_common.cuh"

namespace lf {

struct AttnFwdParams {
  const int4* tiles;
  int num_tiles;
  int Hq, Hkv;
  int q_col0, k_col0, v_col0;
  __nv_bfloat16* out;
  long long ldo;
  float* lse;
  long long M_total;
  float scale, scale_log2e;
  int* err;
};

// Threads per query row in the softmax (each takes 128 / FWD_PARTS key columns of a tile).
// Measured at 4 x 4096 tokens, 64 / 8 heads: 2 -> 700 TFLOP/s, 4 -> 669: the per-tile chain
// (TMEM load, row-max exchange, 1024 cycles of exponentials on the special-function unit, P
// store, proxy fence, hand-over to the MMA warp) is a latency chain that more warps do not shorten.
constexpr int FWD_PARTS = 2;
constexpr int FWD_COLS = ATT_TILE / FWD_PARTS;
constexpr int FWD_SOFTMAX_WARPS = 4 * FWD_PARTS;
constexpr int FWD_THREADS = 64 + 32 * FWD_SOFTMAX_WARPS;  // TMA warp, MMA warp, softmax warps
constexpr int FWD_XCHG_BYTES = 3 * FWD_PARTS * 128 * 4;  // row-max exchange (2 parities) + row-sum exchange
constexpr int FWD_SMEM = ATT_TILE_BYTES * (1 + 4 + 1) + 256 + FWD_XCHG_BYTES + 1024;

__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const AttnFwdParams p, const __grid_constant__ CUtensorMap tm) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + ATT_TILE_BYTES;            // stage s: K at s*64K, V at s*64K + 32K
  uint8_t* sP = smem + ATT_TILE_BYTES * 5;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ATT_TILE_BYTES * 6);
  uint64_t* q_full = bars;
  // K and V tiles travel through two rings of their own: a K slot is free again as soon as the
  // S = Q K^T that read it has completed, one whole softmax earlier than the V slot of the same
  // tile.  With one ring for both, the load of tile J + 1 could only start after P V of tile
  // J - 1, and its latency sat in the per-tile critical path (S of J + 1 is issued before P V of J).
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 15;   // [2]
  uint64_t* v_empty = bars + 17;  // [2]
  uint64_t* s_full = bars + 5;    // [2]
  uint64_t* s_empty = bars + 7;   // [2]
  uint64_t* p_full = bars + 9;
  uint64_t* pv_done = bars + 10;
  uint64_t* q_empty = bars + 12;  // every S = Q K^T of the current head has completed: sQ may be refilled
  uint64_t* o_empty = bars + 13;  // the softmax warps have read the finished O: the next head may overwrite it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xchg = reinterpret_cast<float*>(smem + ATT_TILE_BYTES * 6 + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  AbortCtx ctx{p.err, abort_flag};
  const int4 tile = p.tiles[blockIdx.x];
  const int row0 = tile.x, rows = tile.y, seq_row0 = tile.z;
  const int g = blockIdx.y;            // KV head
  const int group = p.Hq / p.Hkv;      // query heads that share it, walked in turn
  const int h0 = g * group;
  const int n_kv = (row0 - seq_row0) / ATT_TILE + 1;
  const int total = group * n_kv;      // the flat (head, key tile) sequence J = hi * n_kv + j

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], FWD_SOFTMAX_WARPS);  // one arrival per softmax warp
    }
    mbar_init(p_full, FWD_SOFTMAX_WARPS);
    mbar_init(pv_done, 1);
    mbar_init(q_empty, 1);
    mbar_init(o_empty, FWD_SOFTMAX_WARPS);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm);
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
  const uint32_t tO = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      for (int hi = 0; ok && hi < group; ++hi) {
        for (int j = 0; j < n_kv; ++j) {
          const int J = hi * n_kv + j;
          const int s = J & 1;
          if (!mbar_wait(&k_empty[s], ((J >> 1) & 1) ^ 1, ctx, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sK = sKV + s * 2 * ATT_TILE_BYTES;
          mbar_expect_tx(&k_full[s], ATT_TILE_BYTES);
          att_load_tile(sK, &tm, &k_full[s], p.k_col0 + g * ATT_D, seq_row0 + j * ATT_TILE);
          if (j == 0) {
            // Q of this head, right behind its first K/V tile; the single Q buffer is free once
            // the previous head's last S product has completed
            if (hi > 0 && !mbar_wait(q_empty, (hi - 1) & 1, ctx, ERR_WAIT_EMPTY)) {
              ok = false;
              break;
            }
            mbar_expect_tx(q_full, ATT_TILE_BYTES);
            att_load_tile(sQ, &tm, q_full, p.q_col0 + (h0 + hi) * ATT_D, row0);
          }
          if (!mbar_wait(&v_empty[s], ((J >> 1) & 1) ^ 1, ctx, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&v_full[s], ATT_TILE_BYTES);
          att_load_tile(sK + ATT_TILE_BYTES, &tm, &v_full[s], p.v_col0 + g * ATT_D, seq_row0 + j * ATT_TILE);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, ctx, ERR_WAIT_FULL);
      ok = ok && mbar_wait(&k_full[0], 0, ctx, ERR_WAIT_FULL);
      if (ok) {
        tc_fence_after_sync();
        att_mma_kk(tS[0], smem_u32(sQ), smem_u32(sKV), false);
        tc_commit(&s_full[0]);
        tc_commit(&k_empty[0]);
        if (n_kv == 1) tc_commit(q_empty);
      }
      for (int J = 0; ok && J < total; ++J) {
        const int hi = J / n_kv, j = J - hi * n_kv;
        if (J + 1 < total) {
          // S of the next element of the sequence goes out before this element's P V, so that
          // the softmax warps always have a tile waiting (two S buffers in TMEM)
          const int J1 = J + 1;
          const int hi1 = J1 / n_kv, j1 = J1 - hi1 * n_kv;
          const int s1 = J1 & 1;
          const uint32_t ph = (J1 >> 1) & 1;
          if ((j1 == 0 && !mbar_wait(q_full, hi1 & 1, ctx, ERR_WAIT_FULL)) ||
              !mbar_wait(&k_full[s1], ph, ctx, ERR_WAIT_FULL) ||
              !mbar_wait(&s_empty[s1], ph ^ 1, ctx, ERR_WAIT_TMEM_EMPTY)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          att_mma_kk(tS[s1], smem_u32(sQ), smem_u32(sKV + s1 * 2 * ATT_TILE_BYTES), false);
          tc_commit(&s_full[s1]);
          tc_commit(&k_empty[s1]);
          if (j1 == n_kv - 1) tc_commit(q_empty);  // last use of this head's Q
        }
        if (!mbar_wait(p_full, J & 1, ctx, ERR_WAIT_READY) ||
            !mbar_wait(&v_full[J & 1], (J >> 1) & 1, ctx, ERR_WAIT_FULL) ||
            (j == 0 && hi > 0 && !mbar_wait(o_empty, (hi - 1) & 1, ctx, ERR_WAIT_TMEM_EMPTY))) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        att_mma_kmn(tO, smem_u32(sP), smem_u32(sKV + (J & 1) * 2 * ATT_TILE_BYTES + ATT_TILE_BYTES),
                    j > 0);
        tc_commit(&v_empty[J & 1]);
        tc_commit(pv_done);
      }
    }
  } else {
    // FWD_PARTS threads per query row: warps 2-5 take the first FWD_COLS key columns of each tile,
    // warps 6-9 the next, ... (a warp may only touch the TMEM lane quarter warp % 4).  The parts
    // agree on the running maximum through shared memory once per tile, keep private partial
    // row sums, and each rescales / writes its own FWD_COLS columns of O.
    const int q = warp & 3;
    const int part = (warp - 2) >> 2;  // which FWD_COLS-wide slice of the key columns
    const int r = q * 32 + lane;       // row inside the tile
    const int c0 = part * FWD_COLS;
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    const float c = p.scale_log2e;
    constexpr uint32_t FULL = 0xffffffffu;
    // Synchronisation is kept cheap because it sits on the critical path of every key tile: the two
    // warps that share a row quarter meet in a hardware named barrier (id 1 + q, 64 threads) for
    // the row-max exchange, and every mbarrier gets ONE arrival per warp (256 arrivals on one
    // barrier word serialise).  `good` is warp-uniform (the tcgen05.ld/st below are .sync.aligned);
    // a failed wait is carried to the next named barrier, whose vote lets both warps leave together.
    bool good = true, ok = true;
    for (int hi = 0; ok && hi < group; ++hi) {
      const int h = h0 + hi;
      float m_ref = -INFINITY, l = 0.f;
      for (int j = 0; j < n_kv; ++j) {
        const int J = hi * n_kv + j;          // position in the flat sequence: S / P / K-V ring parities
        const int X = hi * (n_kv + 1) + j;    // exchanges through shared memory so far (one more per head)
        const int b = J & 1, xb = X & 1;
        good = __all_sync(FULL, good && mbar_wait(&s_full[b], (J >> 1) & 1, ctx, ERR_WAIT_TMEM_FULL));
        float s[FWD_COLS];
        if (good) {
          tc_fence_after_sync();
#pragma unroll
          for (int cc = 0; cc < FWD_COLS / 32; ++cc) {
            uint32_t(&dst)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[cc * 32]);
            tmem_ld_32x32b_x32(tS[b] + lane_addr + c0 + cc * 32, dst);
          }
          tmem_ld_wait();
          tc_fence_before_sync();
        } else {
#pragma unroll
          for (int col = 0; col < FWD_COLS; ++col) s[col] = 0.f;
        }
        __syncwarp();
        if (lane == 0 && good) mbar_arrive(&s_empty[b]);
        if (j == n_kv - 1) {
#pragma unroll
          for (int col = 0; col < FWD_COLS; ++col)
            if (c0 + col > r) s[col] = -INFINITY;
        }
        // four independent chains each for the maximum and the sum: one chain of 64 dependent
        // operations per row leaves the two warps of a scheduler waiting on fixed latencies
        float mx4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
        for (int col = 4; col < FWD_COLS; ++col) mx4[col & 3] = fmaxf(mx4[col & 3], s[col]);
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        xchg[xb * FWD_PARTS * 128 + part * 128 + r] = mx;
        good = named_bar_and_id(1 + q, 32 * FWD_PARTS, good);
        if (!good) {
          ok = false;
          break;
        }
#pragma unroll
        for (int o = 1; o < FWD_PARTS; ++o) mx = fmaxf(mx, xchg[xb * FWD_PARTS * 128 + ((part + o) % FWD_PARTS) * 128 + r]);
        float alpha = 1.f;
        bool need = false;
        if (j == 0) {
          m_ref = mx;
        } else {
          need = (mx - m_ref) * c > 8.f;
          if (need) {
            alpha = fast_exp2((m_ref - mx) * c);
            m_ref = mx;
            l *= alpha;
          }
        }
        const bool warp_need = __any_sync(FULL, need);
        const float mc = m_ref * c;
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int col = 0; col < FWD_COLS; ++col) {
          s[col] = fast_exp2(s[col] * c - mc);
          sum4[col & 3] += s[col];
        }
        l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        if (j > 0) {
          // (for j == 0 the previous head's last P V was awaited by that head's final store)
          good = __all_sync(FULL, mbar_wait(pv_done, (J - 1) & 1, ctx, ERR_WAIT_MISC));
        }
        if (good) {
          tc_fence_after_sync();
#pragma unroll
          for (int cc = 0; cc < FWD_COLS / 32; ++cc) {
            float(&src)[32] = *reinterpret_cast<float(*)[32]>(&s[cc * 32]);
            att_store_row_chunk(sP, r, c0 + cc * 32, src);
          }
          if (warp_need) {
#pragma unroll 1
            for (int cc = 0; cc < FWD_COLS / 32; ++cc) {
              uint32_t o[32];
              tmem_ld_32x32b_x32(tO + lane_addr + c0 + cc * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st_32x32b_x32(tO + lane_addr + c0 + cc * 32, o);
            }
            tmem_st_wait();
          }
          fence_proxy_async_smem();
          tc_fence_before_sync();
        }
        __syncwarp();
        if (lane == 0 && good) mbar_arrive(p_full);
      }
      if (!ok) break;
      // ---- this head is complete: combine the two partial row sums (both relative to the same
      // m_ref), normalise, store, and hand the O accumulator to the next head
      xchg[2 * FWD_PARTS * 128 + part * 128 + r] = l;
      good = named_bar_and_id(1 + q, 32 * FWD_PARTS, good);
      if (!good) break;
      {
        // every thread of the row adds the partial sums in the same order (part 0 first)
        float tot = 0.f;
#pragma unroll
        for (int o = 0; o < FWD_PARTS; ++o) tot += xchg[2 * FWD_PARTS * 128 + o * 128 + r];
        l = tot;
      }
      good = __all_sync(FULL, mbar_wait(pv_done, (hi * n_kv + n_kv - 1) & 1, ctx, ERR_WAIT_MISC));
      if (good) {
        tc_fence_after_sync();
        const float inv_l = 1.f / l;
        const long long grow = (long long)row0 + r;
        __nv_bfloat16* orow = p.out + grow * p.ldo + h * ATT_D + c0;
#pragma unroll 1
        for (int cc = 0; cc < FWD_COLS / 32; ++cc) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(tO + lane_addr + c0 + cc * 32, o);
          tmem_ld_wait();
          if (r < rows) {
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
              st_global_v4(orow + cc * 32 + gq * 8,
                           pack_bf16x2(__uint_as_float(o[gq * 8 + 0]) * inv_l, __uint_as_float(o[gq * 8 + 1]) * inv_l),
                           pack_bf16x2(__uint_as_float(o[gq * 8 + 2]) * inv_l, __uint_as_float(o[gq * 8 + 3]) * inv_l),
                           pack_bf16x2(__uint_as_float(o[gq * 8 + 4]) * inv_l, __uint_as_float(o[gq * 8 + 5]) * inv_l),
                           pack_bf16x2(__uint_as_float(o[gq * 8 + 6]) * inv_l, __uint_as_float(o[gq * 8 + 7]) * inv_l));
            }
          }
        }
        if (part == 0 && r < rows) p.lse[(long long)h * p.M_total + grow] = m_ref * p.scale + __logf(l);
        tc_fence_before_sync();
      }
      __syncwarp();
      if (lane == 0 && good) mbar_arrive(o_empty);
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

// qkv: packed [M, ld_qkv] bf16 (q heads, then k heads, then v heads at the given column
// offsets); tiles: device int32 [num_tiles, 4]; out [M, Hq*128]; lse fp32 [Hq, M].
extern "C" int lf_attn_fwd(const void* qkv, long long M, long long ld_qkv, int q_col0, int k_col0,
                           int v_col0, int Hq, int Hkv, const void* tiles, int num_tiles, void* out,
                           long long ldo, float* lse, float scale, int* err, void* stream) {
  if (num_tiles <= 0) return 0;
  if (Hq % Hkv != 0 || (q_col0 | k_col0 | v_col0) % 64 != 0) return -1;
  CUtensorMap tm;
  int rc = make_tmap_2d_b16(&tm, qkv, (uint64_t)M, (uint64_t)ld_qkv, (uint64_t)ld_qkv, 128, 64, true);
  if (rc != 0) return -20 + rc;
  static PerDeviceOnce configured;
  if (ensure_max_dynamic_smem(configured, attn_fwd_kernel, FWD_SMEM) != cudaSuccess) return -10;
  AttnFwdParams p;
  p.tiles = (const int4*)tiles;
  p.num_tiles = num_tiles;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.q_col0 = q_col0;
  p.k_col0 = k_col0;
  p.v_col0 = v_col0;
  p.out = (__nv_bfloat16*)out;
  p.ldo = ldo;
  p.lse = lse;
  p.M_total = M;
  p.scale = scale;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.err = err;
  dim3 grid(num_tiles, Hkv);  // one CTA per (query tile, KV head); it walks the group's query heads
  attn_fwd_kernel<<<grid, FWD_THREADS, FWD_SMEM, (cudaStream_t)stream>>>(p, tm);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
