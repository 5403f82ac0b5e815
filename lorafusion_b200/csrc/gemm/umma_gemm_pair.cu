// CTA-pair (tcgen05 cta_group::2) version of the hot base+LoRA GEMMs: a cluster of two CTAs
// on neighbouring SMs computes one 256 x 256 output tile.  Each CTA stages only its own 128
// rows of A and its own 128 of the 256 B rows (32 KB per 64-deep k-block instead of 48 KB
// for the single-CTA 128 x 256 tile), the pair MMA reads both halves of B from both CTAs'
// shared memory, and each CTA ends up with its 128 x 256 fp32 slice in its own TMEM.  The
// single-CTA kernel (umma_gemm.cu) is operand-bandwidth bound -- 910 TFLOP/s with 128-wide,
// 1300 with 256-wide tiles on the same problem -- so halving the B traffic per CTA is what
// moves it towards the tensor-core bound.  No cluster-multicast load is used anywhere: every
// CTA fetches its own tiles with ordinary tiled TMA loads.
//
// Covered ops (the ones that dominate a training step):
//   forward  Y  = X W^T + S' B_a^T (+ bias)                 B K-major,  one accumulator
//   dX       dX = dY W + dS A_a                             B MN-major, one accumulator
//   dX with dropout: the slab dS A_a goes into the accumulator first, is masked in place in
//                    TMEM by the epilogue warps (Philox mask regenerated), dY W lands on top
// Adapters are chosen per 128-row tile, so the two CTAs of a pair may need different LoRA
// weights: the LoRA slab is issued once per distinct adapter of the pair, and a CTA whose
// rows belong to another adapter loads zeros for its S' rows (an out-of-range TMA box).
//
// Roles per CTA: warp 0 = TMA producer (both CTAs), warp 1 = TMEM allocator (both) and MMA
// issuer (leader CTA only), warps 2..9 = epilogue (both).  Barriers: "stage full" lives in
// the leader and is credited by both CTAs' loads; "stage empty" and "accumulator full" exist
// in both CTAs and are signalled by two tcgen05.commit (own + peer address); "accumulator
// empty" lives in the leader and collects one arrival per epilogue warp of both CTAs.  All waits are bounded.
#include <stdio.h>

#include "../common/launch.h"
#include "../common/philox.cuh"
#include "../common/ptx.cuh"
#include "../common/tensormap.h"
#include "gemm_api.h"
#include "tp_params.cuh"

namespace lf {
namespace pair {

constexpr int BM = 128;        // rows per CTA
constexpr int BN = 256;        // columns of the pair tile
constexpr int BNH = 128;       // B rows staged per CTA
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BNH * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 6;
constexpr int PAIR_EPI_WARPS = 8;                    // two per TMEM lane quarter
constexpr int PAIR_THREADS = 64 + 32 * PAIR_EPI_WARPS;  // TMA warp, MMA warp, epilogue warps
constexpr int SMEM_TOTAL = STAGES * STAGE_BYTES + 512 + 1024;

struct Params {
  int M, N;
  int nkb_main, nkb2;
  int num_pair_m, num_n_tiles, num_tiles, group_m;
  const int* tile_adapter;  // per 128-row tile, may be null (= adapter 0)
  int b2_adapter_rows;
  __nv_bfloat16* out;
  long long ldo;
  const __nv_bfloat16* bias;
  const uint32_t* adapter_thresh16;
  const float* adapter_inv_keep;
  uint32_t thresh16;
  float inv_keep;
  uint32_t seed_lo, seed_hi, stream_id;
  int row_offset, col_offset;
  int zero_row;  // a row coordinate outside A2: TMA reads zeros there
  int m_rotate;  // pair rows the tile order is rotated by (tensor-parallel variants start / end with the own shard)
  int* err;
};

struct Tile {
  int pm, n_tile;   // pair-row index (256 rows) and column tile
  int a0, a1;       // adapters of the leader's and the peer's 128 rows (-1 = none)
};

__device__ __forceinline__ Tile decode(const Params& p, int idx) {
  Tile t;
  const int per_group = p.group_m * p.num_n_tiles;
  const int g = idx / per_group;
  const int first = g * p.group_m;
  const int gsz = min(p.group_m, p.num_pair_m - first);
  const int r = idx - g * per_group;
  t.pm = first + r % gsz + p.m_rotate;
  if (t.pm >= p.num_pair_m) t.pm -= p.num_pair_m;
  t.n_tile = r / gsz;
  const int mt0 = 2 * t.pm, mt1 = 2 * t.pm + 1;
  const int n_mt = (p.M + BM - 1) / BM;
  if (p.nkb2 == 0) {
    t.a0 = t.a1 = -1;
  } else if (p.tile_adapter == nullptr) {
    t.a0 = 0;
    t.a1 = mt1 < n_mt ? 0 : -1;
  } else {
    t.a0 = p.tile_adapter[mt0];
    t.a1 = mt1 < n_mt ? p.tile_adapter[mt1] : -1;
  }
  return t;
}

// Slab passes of a tile: one per distinct adapter of the pair.
__device__ __forceinline__ int slab_passes(const Tile& t, int (&ad)[2]) {
  int n = 0;
  if (t.a0 >= 0) ad[n++] = t.a0;
  if (t.a1 >= 0 && t.a1 != t.a0) ad[n++] = t.a1;
  return n;
}

// TP = 0: plain.  TP = 1: all-gather -> GEMM (four extra warps per CTA push this rank's token
// shard to the peers; a CTA's producer waits for the flag of its own 128-row tile before the first
// load).  TP = 2: GEMM -> reduce-scatter (each CTA leaves its 128 x 256 partial in this GPU's stage
// and flags it at the owner of the rows; four extra warps per CTA pull and sum the partials of the
// rows this rank owns).  Same protocol, flags and buffers as the single-CTA template in
// umma_gemm.cu; 128-row tile granularity is kept because each CTA of a pair owns one such tile.
//
// EPI = LF_EPI_BF16: per tile the main product, then the LoRA slab on top; two accumulator
// buffers, the epilogue of tile j drains one while the main loop of tile j + 1 fills the other.
//
// EPI = LF_EPI_BF16_DROPMIX ("slab first"): dX = dY W + keep (.) (dS A) / (1 - p).  The slab
// product of tile j + 1 is issued in the MIDDLE of tile j's main loop into the other accumulator
// buffer; the epilogue warps multiply it by the regenerated dropout mask IN PLACE in TMEM
// (tcgen05.ld -> Philox -> tcgen05.st) while tile j's main loop goes on, and tile j + 1's main
// product then accumulates on top of the masked slab.  Both passes of the epilogue warps (mask
// of the next tile, drain of the current one) are hidden behind a main loop, so the kernel keeps
// ONE accumulator per tile, double-buffered, exactly like the plain variant.  Barriers added for
// this: "slab full" (both CTAs, tcgen05.commit) and "slab masked" (leader, every epilogue thread
// of both CTAs arrives).
template <bool B_MN, int EPI, int TP = 0>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS + (TP != 0 ? 32 * kNumCommWarps : 0), 1)
    umma_gemm_pair_kernel(const Params p, const __grid_constant__ CUtensorMap tmA,
                          const __grid_constant__ CUtensorMap tmB,
                          const __grid_constant__ CUtensorMap tmA2,
                          const __grid_constant__ CUtensorMap tmB2, const TpParams tp) {
  constexpr bool SLAB_FIRST = (EPI == LF_EPI_BF16_DROPMIX);
  constexpr int NBUF = 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                 // used in the leader
  uint64_t* empty = bars + STAGES;       // both
  uint64_t* tfull = bars + 2 * STAGES;   // both [2]
  uint64_t* tempty = tfull + 2;          // leader [2]
  uint64_t* sfull = tempty + 2;          // both [2]: the slab product of a tile is in its buffer
  uint64_t* masked = sfull + 2;          // leader [2]: ... and has been masked in place
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(masked + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  AbortCtx ctx{p.err, abort_flag, TP != 0 ? kPeerWaitNs + kLocalWaitNs : kLocalWaitNs};
  // main-loop block before which the next tile's slab is slipped in (slab-first variant)
  const int ks = SLAB_FIRST ? p.nkb_main / 2 : p.nkb_main;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], 2 * PAIR_EPI_WARPS);  // lane 0 of every epilogue warp of both CTAs
      mbar_init(&sfull[b], 1);
      mbar_init(&masked[b], 2 * PAIR_EPI_WARPS);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();   // the peer's barriers exist before anything is signalled remotely
  cluster_wait();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ producer (both CTAs) ------------------------------
    if (lane == 0) {
      int it = 0;
      // one 64-deep k-block into the next free stage: block `kb` of the main product, or block
      // `slab_idx` (>= 0) of the tile's slab passes
      auto load_block = [&](const Tile& t, const int (&ad)[2], int kb, int slab_idx) -> bool {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, ctx, ERR_WAIT_EMPTY)) return false;
        ++it;
        const int m0 = (2 * t.pm + int(cta)) * BM;
        const int n0 = t.n_tile * BN + int(cta) * BNH;
        uint8_t* sA = smem + s * STAGE_BYTES;
        uint8_t* sB = sA + A_BYTES;
        const uint32_t fbar = mapa_shared(&full[s], 0);
        if (cta == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
        if (slab_idx < 0) {
          const int kk = kb * BK;
          tma_load_2d_pair(sA, &tmA, fbar, kk, m0);
          if (!B_MN) {
            tma_load_2d_pair(sB, &tmB, fbar, kk, n0);
          } else {
            tma_load_2d_pair(sB, &tmB, fbar, n0, kk);
            tma_load_2d_pair(sB + 8192, &tmB, fbar, n0 + 64, kk);
          }
        } else {
          const int sp = slab_idx / p.nkb2;
          const int kk2 = (slab_idx - sp * p.nkb2) * BK;
          const int a = ad[sp];
          const int my_adapter = cta == 0 ? t.a0 : t.a1;
          // rows of another adapter contribute nothing to this pass: read zeros
          tma_load_2d_pair(sA, &tmA2, fbar, kk2, my_adapter == a ? m0 : p.zero_row);
          const int by2 = a * p.b2_adapter_rows;
          if (!B_MN) {
            tma_load_2d_pair(sB, &tmB2, fbar, kk2, by2 + n0);
          } else {
            tma_load_2d_pair(sB, &tmB2, fbar, n0, by2 + kk2);
            tma_load_2d_pair(sB + 8192, &tmB2, fbar, n0 + 64, by2 + kk2);
          }
        }
        return true;
      };
      // all-gather variant: the rows of this CTA's A tile (and of its slab tile) come from rank
      // `src`; they are in LOCAL memory once that rank has pushed them and raised the tile's flag
      auto rows_ready = [&](const Tile& t) -> bool {
        if (TP == 1) {
          const int mt = 2 * t.pm + int(cta);
          const int src = mt / tp.tiles_per_shard;
          if (src != tp.rank) {
            if (!wait_flag_ge(tp.ag_flags + src * tp.tiles_per_shard + (mt - src * tp.tiles_per_shard), tp.epoch,
                              ctx))
              return false;
            fence_proxy_async_all();
          }
        }
        return true;
      };
      auto load_slabs = [&](const Tile& t) -> bool {
        int ad[2] = {0, 0};
        const int n = slab_passes(t, ad) * p.nkb2;
        for (int i = 0; i < n; ++i)
          if (!load_block(t, ad, 0, i)) return false;
        return true;
      };
      auto load_main = [&](const Tile& t, int kb0, int kb1) -> bool {
        const int ad[2] = {0, 0};
        for (int kb = kb0; kb < kb1; ++kb)
          if (!load_block(t, ad, kb, -1)) return false;
        return true;
      };
      bool ok = true;
      if (SLAB_FIRST && pair_id < p.num_tiles) {
        const Tile t = decode(p, pair_id);
        ok = rows_ready(t) && load_slabs(t);
      }
      for (int tile = pair_id; ok && tile < p.num_tiles; tile += num_pairs) {
        const Tile t = decode(p, tile);
        if (!SLAB_FIRST) ok = rows_ready(t);
        ok = ok && load_main(t, 0, ks);
        if (SLAB_FIRST) {
          if (ok && tile + num_pairs < p.num_tiles) {
            const Tile tn = decode(p, tile + num_pairs);
            ok = rows_ready(tn) && load_slabs(tn);
          }
        } else {
          ok = ok && load_slabs(t);
        }
        ok = ok && load_main(t, ks, p.nkb_main);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader only) ------------------------------
    if (cta == 0 && lane == 0) {
      constexpr uint32_t IDESC = make_idesc_bf16(256, BN, 0, B_MN ? 1 : 0);
      int it = 0;
      // one k-block from the next full stage into accumulator `d`; `fresh` = overwrite it
      auto issue_block = [&](uint32_t d, bool fresh) -> bool {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(&full[s], ph, ctx, ERR_WAIT_FULL)) return false;
        ++it;
        tc_fence_after_sync();
        const uint32_t sA = smem_u32(smem + s * STAGE_BYTES);
        const uint32_t sB = sA + A_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
          const uint64_t da = make_smem_desc_sw128(sA + kk * 32, 16, 1024);
          const uint64_t db = B_MN ? make_smem_desc_sw128(sB + kk * 2048, 8192, 1024)
                                   : make_smem_desc_sw128(sB + kk * 32, 16, 1024);
          umma_bf16_ss_pair(d, da, db, IDESC, uint32_t(!(fresh && kk == 0)));
        }
        tc_commit_pair(mapa_shared(&empty[s], 0));
        tc_commit_pair(mapa_shared(&empty[s], 1));
        return true;
      };
      // slab passes of a tile; in the slab-first variant they open the accumulator
      auto issue_slabs = [&](const Tile& t, uint32_t d) -> bool {
        int ad[2] = {0, 0};
        const int n = slab_passes(t, ad) * p.nkb2;
        for (int i = 0; i < n; ++i)
          if (!issue_block(d, SLAB_FIRST && i == 0)) return false;
        return true;
      };
      auto issue_main = [&](uint32_t d, int kb0, int kb1, bool opens) -> bool {
        for (int kb = kb0; kb < kb1; ++kb)
          if (!issue_block(d, opens && kb == 0)) return false;
        return true;
      };
      int tile_iter = 0;
      bool ok = true;
      if (SLAB_FIRST && pair_id < p.num_tiles) {
        const Tile t = decode(p, pair_id);
        ok = mbar_wait(&tempty[0], 1, ctx, ERR_WAIT_TMEM_EMPTY);   // fresh barrier: passes at once
        if (ok) {
          tc_fence_after_sync();
          ok = issue_slabs(t, tmem_base);
        }
        if (ok) {
          tc_commit_pair(mapa_shared(&sfull[0], 0));
          tc_commit_pair(mapa_shared(&sfull[0], 1));
        }
      }
      for (int tile = pair_id; ok && tile < p.num_tiles; tile += num_pairs, ++tile_iter) {
        const Tile t = decode(p, tile);
        const int buf = tile_iter % NBUF;
        const uint32_t bph = (tile_iter / NBUF) & 1;
        const uint32_t acc = tmem_base + uint32_t(buf * BN);
        bool opens = true;   // does the main product start from a fresh accumulator?
        if (SLAB_FIRST) {
          int ad[2];
          opens = slab_passes(t, ad) * p.nkb2 == 0;
          ok = mbar_wait(&masked[buf], bph, ctx, ERR_WAIT_READY);
        } else {
          ok = mbar_wait(&tempty[buf], bph ^ 1, ctx, ERR_WAIT_TMEM_EMPTY);
        }
        if (!ok) break;
        tc_fence_after_sync();
        ok = issue_main(acc, 0, ks, opens);
        if (SLAB_FIRST) {
          if (ok && tile + num_pairs < p.num_tiles) {
            const Tile tn = decode(p, tile + num_pairs);
            const int nbuf = (tile_iter + 1) % NBUF;
            const uint32_t nph = ((tile_iter + 1) / NBUF) & 1;
            ok = mbar_wait(&tempty[nbuf], nph ^ 1, ctx, ERR_WAIT_TMEM_EMPTY);
            if (ok) {
              tc_fence_after_sync();
              ok = issue_slabs(tn, tmem_base + uint32_t(nbuf * BN));
            }
            if (ok) {
              tc_commit_pair(mapa_shared(&sfull[nbuf], 0));
              tc_commit_pair(mapa_shared(&sfull[nbuf], 1));
            }
          }
        } else {
          ok = ok && issue_slabs(t, acc);
        }
        // with ks == 0 (a single main block) the main product opens here instead
        ok = ok && issue_main(acc, ks, p.nkb_main, opens && ks == 0);
        if (!ok) break;
        tc_commit_pair(mapa_shared(&tfull[buf], 0));
        tc_commit_pair(mapa_shared(&tfull[buf], 1));
      }
    }
  } else if (threadIdx.x < PAIR_THREADS) {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    // Eight warps: two per TMEM lane quarter (a warp may only touch quarter warp % 4), each
    // taking half of the tile's columns.
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int CHUNKS_PER_HALF = BN / 32 / (PAIR_EPI_WARPS / 4);
    const int c_begin = half * CHUNKS_PER_HALF, c_end = (half + 1) * CHUNKS_PER_HALF;
    const uint32_t lane_addr = uint32_t(q * 32) << 16;

    // Slab-first variant: multiply the slab product of tile `t` (in buffer `iter % 2`) by its
    // dropout mask, in place.  A CTA whose rows have no adapter (or an adapter without dropout)
    // only reports in.
    auto mask_slab = [&](const Tile& t, int iter) -> bool {
      const int buf = iter % NBUF;
      // warp-uniform: the tcgen05.ld/st below are .sync.aligned, and the warp reports in as one
      bool got = __all_sync(0xffffffffu, mbar_wait(&sfull[buf], uint32_t(iter / NBUF) & 1, ctx, ERR_WAIT_TMEM_FULL));
      // the reduce-scatter epilogue meets in named barriers: one answer for all 256 threads
      if (TP == 2) got = named_bar_and<1, 32 * PAIR_EPI_WARPS>(got);
      if (!got) return false;
      tc_fence_after_sync();
      const int my_adapter = cta == 0 ? t.a0 : t.a1;
      uint32_t thresh = p.thresh16;
      float inv_keep = p.inv_keep;
      if (my_adapter >= 0 && p.adapter_thresh16 != nullptr) {
        thresh = p.adapter_thresh16[my_adapter];
        inv_keep = p.adapter_inv_keep[my_adapter];
      }
      if (p.nkb2 > 0 && my_adapter >= 0 && thresh != 0) {
        const int row = (2 * t.pm + int(cta)) * BM + q * 32 + lane;
        const uint32_t acc = tmem_base + uint32_t(buf * BN) + lane_addr;
        uint32_t r[32];
        tmem_ld_32x32b_x32(acc + c_begin * 32, r);
#pragma unroll 1
        for (int c = c_begin; c < c_end; ++c) {
          tmem_ld_wait();
          uint32_t w[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) w[j] = r[j];
          if (c + 1 < c_end) tmem_ld_32x32b_x32(acc + (c + 1) * 32, r);
          const int col0 = t.n_tile * BN + c * 32;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint32_t keep = dropout_keep8(uint32_t(row + p.row_offset),
                                                uint32_t((col0 + p.col_offset) >> 3) + g, p.stream_id,
                                                p.seed_lo, p.seed_hi, thresh);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              w[g * 8 + j] = ((keep >> j) & 1u) ? __float_as_uint(inv_keep * __uint_as_float(w[g * 8 + j])) : 0u;
          }
          tmem_st_32x32b_x32(acc + c * 32, w);
        }
        tmem_st_wait();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(&masked[buf], 0));
      return true;
    };

    int tile_iter = 0;
    bool ok = true;
    if (SLAB_FIRST && pair_id < p.num_tiles) ok = mask_slab(decode(p, pair_id), 0);
    for (int tile = pair_id; ok && tile < p.num_tiles; tile += num_pairs, ++tile_iter) {
      const Tile t = decode(p, tile);
      if (SLAB_FIRST && tile + num_pairs < p.num_tiles) {
        if (!mask_slab(decode(p, tile + num_pairs), tile_iter + 1)) {
          ok = false;
          break;
        }
      }
      const int buf = tile_iter % NBUF;
      const uint32_t bph = (tile_iter / NBUF) & 1;
      bool got = __all_sync(0xffffffffu, mbar_wait(&tfull[buf], bph, ctx, ERR_WAIT_TMEM_FULL));
      // the reduce-scatter epilogue ends in a named barrier of its 256 threads: one answer for all
      if (TP == 2) got = named_bar_and<1, 32 * PAIR_EPI_WARPS>(got);
      if (!got) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int row = (2 * t.pm + int(cta)) * BM + q * 32 + lane;
      const uint32_t acc = tmem_base + uint32_t(buf * BN) + lane_addr;
      // the TMEM load of chunk c + 1 is in flight while chunk c is converted and stored
      uint32_t r[32];
      tmem_ld_32x32b_x32(acc + c_begin * 32, r);
#pragma unroll 1
      for (int c = c_begin; c < c_end; ++c) {
        tmem_ld_wait();
        const int col0 = t.n_tile * BN + c * 32;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (c + 1 < c_end) tmem_ld_32x32b_x32(acc + (c + 1) * 32, r);
        if (EPI == LF_EPI_BF16 && p.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
        }
        if (row < p.M) {
          // reduce-scatter: the partial tile stays in THIS GPU's stage [M, N]; the owner pulls it
          __nv_bfloat16* out = (TP == 2) ? tp.rs_peer_stage[tp.rank] + (long long)row * p.N
                                         : p.out + (long long)row * p.ldo;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = col0 + g * 8;
            if (col + 8 <= p.N) {
              st_global_v4(out + col, pack_bf16x2(v[g * 8 + 0], v[g * 8 + 1]),
                           pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]), pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]),
                           pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]));
            } else {
              for (int j = 0; j < 8; ++j)
                if (col + j < p.N) out[col + j] = __float2bfloat16(v[g * 8 + j]);
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(&tempty[buf], 0));
      if (TP == 2) {
        // all 256 epilogue threads of this CTA have stored their part of the 128 x 256 partial
        __threadfence_system();
        asm volatile("bar.sync 1, %0;" ::"n"(32 * PAIR_EPI_WARPS) : "memory");
        if (threadIdx.x == 64) {
          const int mt = 2 * t.pm + int(cta);
          const int owner = mt / tp.tiles_per_shard;
          st_release_sys(tp.rs_peer_cnt[owner] +
                             (tp.rank * tp.tiles_per_shard + (mt - owner * tp.tiles_per_shard)) * p.num_n_tiles +
                             t.n_tile,
                         tp.epoch);
        }
      }
    }
  } else if (TP == 2) {
    // ---- reduce the partials of the rows this rank owns, as they arrive ----
    // Four dedicated warps, concurrent with the GEMM of the other warps: they poll the
    // per-(source, row tile, column tile) flags and sum the bf16 partials in fp32 (+ residual).
    // Every thread keeps the loads of several output vectors from all sources in flight (tp_reduce_item).
    const int et = threadIdx.x - PAIR_THREADS;  // 0..127
    const int items = tp.tiles_per_shard * p.num_n_tiles;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < items; item += gridDim.x) {
      const int lt = item / p.num_n_tiles, nt = item - lt * p.num_n_tiles;
      if (et < tp.world) {
        if (!wait_flag_ge(tp.rs_cnt + (et * tp.tiles_per_shard + lt) * p.num_n_tiles + nt, tp.epoch, ctx))
          ok = false;
      }
      // one agreed answer for the 128 reduce threads (see named_bar_and)
      ok = named_bar_and<2, 128>(ok && !aborted(ctx));
      if (!ok) break;
      tp_reduce_item_any<BM, BN>(tp, et, lt, nt, p.N);
    }
  } else if (TP == 1) {
    // ------------- push this rank's token shard to every peer's gathered buffer -------------
    const int ct = threadIdx.x - PAIR_THREADS;  // 0..127
    const int tps = tp.tiles_per_shard;
    const int ms = tps * BM;
    // A row tile is pushed by up to eight CTAs (row slices), so that every SM's copy warps take
    // part even when the shard has fewer row tiles than the grid has CTAs.  The slices of a
    // tile count themselves as (epoch << 4 | arrivals) in a counter region that follows the
    // flags in the same local buffer (`rs_target` = its offset in ints in this mode; the
    // counters must never share words with flags: a stale count would read as a huge epoch);
    // whoever completes the count raises the tile's flag at the peers.
    int parts = 1;
    if (tp.rs_target > 0)
      while (parts < 8 && parts * 2 * tps <= int(gridDim.x)) parts *= 2;
    const int rows_per = BM / parts;
    int* my_cnt = const_cast<int*>(tp.ag_flags) + tp.rs_target;
    for (int u = blockIdx.x; u < tps * parts; u += gridDim.x) {
      const int lt = u / parts, part = u - lt * parts;
      const long long row0 = (long long)tp.rank * ms + lt * BM + part * rows_per;
      const int vec_per_row = tp.ag_cols / 8;
      const int nvec = rows_per * vec_per_row;
      for (int v0 = ct; v0 < nvec; v0 += 4 * 32 * kNumCommWarps) {
        uint4 val[4];
        long long off[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // four local loads in flight before the first peer store
          const int v = v0 + i * 32 * kNumCommWarps;
          off[i] = (row0 + v / vec_per_row) * tp.ag_ld + (v % vec_per_row) * 8;
          if (v < nvec) val[i] = *reinterpret_cast<const uint4*>(tp.ag_src + off[i]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (v0 + i * 32 * kNumCommWarps < nvec) {
            for (int d = 1; d < tp.world; ++d) {
              const int q = (tp.rank + d) % tp.world;
              *reinterpret_cast<uint4*>(tp.ag_peer_dst[q] + off[i]) = val[i];
            }
          }
        }
      }
      if (tp.ag2_src != nullptr) {
        const int vec2 = tp.ag2_cols / 8;
        for (int v = ct; v < rows_per * vec2; v += 32 * kNumCommWarps) {
          const long long off = (row0 + v / vec2) * tp.ag2_ld + (v % vec2) * 8;
          const uint4 val = *reinterpret_cast<const uint4*>(tp.ag2_src + off);
          for (int d = 1; d < tp.world; ++d) {
            const int q = (tp.rank + d) % tp.world;
            *reinterpret_cast<uint4*>(tp.ag2_peer_dst[q] + off) = val;
          }
        }
      }
      __threadfence_system();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (ct == 0) {
        bool last = true;
        if (parts > 1) {
          int seen = *reinterpret_cast<volatile int*>(my_cnt + lt);
          for (;;) {
            const int want = ((seen >> 4) == tp.epoch) ? seen + 1 : ((tp.epoch << 4) | 1);
            const int prev = atomicCAS(my_cnt + lt, seen, want);
            if (prev == seen) {
              last = (want & 15) == parts;
              break;
            }
            seen = prev;
          }
        }
        if (last) {
          __threadfence_system();
          for (int d = 1; d < tp.world; ++d) {
            const int q = (tp.rank + d) % tp.world;
            st_release_sys(tp.ag_peer_flags[q] + tp.rank * tps + lt, tp.epoch);
          }
        }
      }
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  // neither CTA may exit (and release shared memory / barriers) while its partner can still
  // signal into it
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <bool B_MN, int EPI, int TP = 0>
static int launch(const Params& p, const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2,
                  const CUtensorMap& tB2, int pairs, cudaStream_t st, const TpParams& tp = TpParams()) {
  auto kern = umma_gemm_pair_kernel<B_MN, EPI, TP>;
  static lf::PerDeviceOnce configured;  // one per template instantiation
  if (lf::ensure_max_dynamic_smem(configured, kern, SMEM_TOTAL) != cudaSuccess) {
    fprintf(stderr, "lf_gemm_pair: cudaFuncSetAttribute failed\n");
    return -10;
  }
  kern<<<2 * pairs, PAIR_THREADS + (TP != 0 ? 32 * kNumCommWarps : 0), SMEM_TOTAL, st>>>(p, tA, tB, tA2, tB2, tp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "lf_gemm_pair: launch failed: %s\n", cudaGetErrorString(e));
    return -11;
  }
  return 0;
}

}  // namespace pair
}  // namespace lf

// Same argument struct as lf_gemm.  Supported: a / a2 K-major; b and b2 both K-major or both
// MN-major; bn = 256; epilogues LF_EPI_BF16 (nacc 1) and LF_EPI_BF16_DROPMIX (callers pass nacc 2,
// the layout of the single-CTA kernel; here the slab is masked in place in one accumulator); dense
// mode only.  Returns -5 for anything else so that callers can fall back to lf_gemm.
static int pair_entry(const LfGemmArgs* a, const LfTpArgs* t) {
  using namespace lf;
  using namespace lf::pair;
  if (a == nullptr || a->a == nullptr || a->b == nullptr || a->out == nullptr) return -1;
  if (a->a_mn || a->seg_tiles != nullptr || a->mask_a || a->b_adapter_rows != 0) return -5;
  if (a->K2 % BK != 0 || (a->K2 > 0 && (a->b_mn != a->b2_mn))) return -5;
  const bool dropmix = a->epi == LF_EPI_BF16_DROPMIX && a->nacc == 2;
  if (!dropmix && !(a->epi == LF_EPI_BF16 && a->nacc == 1)) return -5;
  if (a->scale != 1.0f) return -5;

  CUtensorMap tA, tB, tA2, tB2;
  int rc = make_tmap_2d_b16(&tA, a->a, a->a_rows, a->a_cols, a->a_ld, BM, 64, true);
  if (rc != 0) return -20 + rc;
  rc = make_tmap_2d_b16(&tB, a->b, a->b_rows, a->b_cols, a->b_ld, a->b_mn ? 64 : BNH, 64, true);
  if (rc != 0) return -30 + rc;
  if (a->K2 > 0) {
    rc = make_tmap_2d_b16(&tA2, a->a2, a->a2_rows, a->a2_cols, a->a2_ld, BM, 64, true);
    if (rc != 0) return -40 + rc;
    rc = make_tmap_2d_b16(&tB2, a->b2, a->b2_rows, a->b2_cols, a->b2_ld, a->b2_mn ? 64 : BNH, 64, true);
    if (rc != 0) return -50 + rc;
  } else {
    tA2 = tA;
    tB2 = tB;
  }
  Params p;
  p.M = a->M;
  p.N = a->N;
  p.nkb_main = (a->K + BK - 1) / BK;
  p.nkb2 = a->K2 / BK;
  p.num_pair_m = (a->M + 2 * BM - 1) / (2 * BM);
  p.num_n_tiles = (a->N + BN - 1) / BN;
  p.num_tiles = p.num_pair_m * p.num_n_tiles;
  p.group_m = a->group_m > 0 ? a->group_m : 4;
  p.tile_adapter = a->tile_adapter;
  p.b2_adapter_rows = a->b2_adapter_rows;
  p.out = (__nv_bfloat16*)a->out;
  p.ldo = a->ldo;
  p.bias = (const __nv_bfloat16*)a->bias;
  p.adapter_thresh16 = a->adapter_thresh16;
  p.adapter_inv_keep = a->adapter_inv_keep;
  p.thresh16 = a->thresh16;
  p.inv_keep = a->inv_keep;
  p.seed_lo = a->seed_lo;
  p.seed_hi = a->seed_hi;
  p.stream_id = a->stream_id;
  p.row_offset = a->row_offset;
  p.col_offset = a->col_offset;
  p.zero_row = int(a->a2_rows) + BM;  // beyond the last row of S': the TMA box reads zeros
  p.err = a->err;
  p.m_rotate = 0;
  if (p.num_tiles <= 0) return 0;
  TpParams tp{};
  const int mode = (t != nullptr) ? t->mode : 0;
  if (mode != 0) {
    if (t->world < 1 || t->world > 8 || t->rank < 0 || t->rank >= t->world) return -7;
    // a pair owns two 128-row tiles of ONE rank's shard: whole pairs per shard, no ragged last pair
    if (t->tiles_per_shard % 2 != 0 || a->M != (long long)t->world * t->tiles_per_shard * BM) return -5;
    if (a->bn != BN) return -5;
    tp = make_tp_params(t);
    // all-gather: start with this rank's own rows; reduce-scatter: finish with them
    const int pairs_per_shard = t->tiles_per_shard / 2;
    p.m_rotate = (mode == 1 ? t->rank : (t->rank + 1) % t->world) * pairs_per_shard;
    if (pairs_per_shard < p.group_m) p.group_m = pairs_per_shard;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int pairs = sms / 2;
  if (a->max_ctas > 0 && a->max_ctas / 2 < pairs) pairs = a->max_ctas / 2;
  if (p.num_tiles < pairs) pairs = p.num_tiles;
  if (pairs < 1) pairs = 1;
  cudaStream_t st = (cudaStream_t)a->stream;
  if (dropmix && !a->b_mn) return -5;
#define LF_PAIR_DISPATCH(TPV)                                                                                  \
  do {                                                                                                         \
    if (dropmix) return launch<true, LF_EPI_BF16_DROPMIX, TPV>(p, tA, tB, tA2, tB2, pairs, st, tp);         \
    if (a->b_mn) return launch<true, LF_EPI_BF16, TPV>(p, tA, tB, tA2, tB2, pairs, st, tp);                 \
    return launch<false, LF_EPI_BF16, TPV>(p, tA, tB, tA2, tB2, pairs, st, tp);                             \
  } while (0)
  if (mode == 1) LF_PAIR_DISPATCH(1);
  if (mode == 2) LF_PAIR_DISPATCH(2);
  LF_PAIR_DISPATCH(0);
#undef LF_PAIR_DISPATCH
}

extern "C" int lf_gemm_pair(const LfGemmArgs* a) { return pair_entry(a, nullptr); }

// CTA-pair variants of the tensor-parallel fused kernels (see lf_gemm_tp).  Returns -5 for
// shapes the pair kernels do not cover (odd number of 128-row tiles per shard, ...): the caller
// falls back to lf_gemm_tp.
extern "C" int lf_gemm_pair_tp(const LfGemmArgs* a, const LfTpArgs* t) {
  if (t == nullptr || t->mode == 0) return -5;
  return pair_entry(a, t);
}
