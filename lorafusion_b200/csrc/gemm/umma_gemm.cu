// Persistent, warp-specialised bf16 GEMM family for sm_100a built directly on tcgen05.mma
// with fp32 accumulators in TMEM and TMA-fed 128-byte-swizzled shared-memory stages.
//
// One kernel template covers every GEMM-shaped op of the fused LoRA linear layer:
//   * forward  Y = X W^T + S' B_a^T        (main loop over W, one extra "slab" of k-blocks
//                                           over the rank dimension, adapter chosen per
//                                           128-row tile)           -- reference K4/K5/K9
//   * dX       dX = dY W + keep (.) (dS A_a) / (1 - p)              -- reference K6/K7/K10
//   * the skinny LoRA products S' = a * drop(X) A_a^T, dS = a * dY B_a, dB, dA, with the
//     dropout mask regenerated from Philox inside shared memory (never stored)
//                                           -- reference K1-K3, K8, K11 and cuBLAS calls
// (file:line citations of the reference live in lorafusion_b200/ops/lora.py).
//
// Roles inside a CTA (1 CTA per SM, grid = min(#tiles, #SMs)):
//   warp 0      : TMA producer (one elected lane)
//   warp 1      : TMEM allocator + single-thread tcgen05.mma issuer
//   warps 2..5  : epilogue (each warp owns one 32-lane TMEM quarter)
//   warps 6..13 : only when MASK_A: apply the dropout mask to the A stage in place
// Accumulators are double-buffered in TMEM so the epilogue of tile i overlaps the main loop
// of tile i+1.
#include <stdio.h>

#include "../common/launch.h"
#include "../common/philox.cuh"
#include "../common/ptx.cuh"
#include "../common/tensormap.h"
#include "gemm_api.h"
#include "tp_params.cuh"

namespace lf {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kNumMaskWarps = 8;
// The dropout warps work in groups on DIFFERENT stages at the same time: one stage's rewrite is a
// chain of latencies (barrier poll, shared-memory load, seven Philox rounds, store, proxy fence),
// and eight warps on one stage at a time left the kernel bound by that chain, not by issue slots.
constexpr int kMaskGroups = 4;

struct GemmKParams {
  int M, N;
  int nkb_main, nkb2;
  int num_m_tiles, num_n_tiles, num_tiles, group_m;
  const int* tile_adapter;
  const int4* seg_tiles;
  int b_adapter_rows, b2_adapter_rows;
  void* out;
  long long ldo;
  long long out_adapter_stride;
  int out_transposed;
  const float* adapter_scale;
  float scale;
  const __nv_bfloat16* bias;
  const uint32_t* adapter_thresh16;
  const float* adapter_inv_keep;
  uint32_t thresh16;
  float inv_keep;
  uint32_t seed_lo, seed_hi, stream_id;
  int row_offset, col_offset;
  int m_rotate;  // dense mode: M tiles are visited starting from this tile (wraps around)
  int* err;
  // NF4 main loop: fp32 scale of every 64-element block of the [nf4_rows, 64 * blocks] weight
  const float* nf4_scales;
  long long nf4_rows, nf4_blocks_per_row;
};

// The sixteen NF4 code values (bitsandbytes' normal-float table).
__constant__ float kNf4Values[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f,
};

// Tensor-parallel fusion (TP != 0).  Token rows are split in `world` shards of
// `tiles_per_shard` 128-row tiles; shard q belongs to rank q.
//  TP == 1  all-gather -> GEMM: the A operand (and the LoRA S' operand) of the other ranks'
//           shards is pushed into this GPU's gathered buffer by their kernels while this one
//           computes; extra warps push this rank's shard to every peer with plain stores over
//           NVLink and raise one flag per row tile; the TMA producer waits for the flag of a
//           tile's source rank before loading it (own shard first).
//  TP == 2  GEMM -> reduce-scatter: the epilogue stores each bf16 partial tile into this GPU's
//           own staging buffer and raises a per-(source, row tile, column tile) epoch flag in
//           the memory of the rank that owns those token rows; four extra warps, concurrent
//           with the GEMM, pull the partials of the rows this rank owns from every source with
//           coalesced peer loads as their flags arrive and sum them in fp32 (+ residual).
struct TileCoord {
  int m0, n0, k0, nkb, adapter;
};

__device__ __forceinline__ TileCoord decode_tile(const GemmKParams& p, int idx) {
  TileCoord t;
  if (p.seg_tiles != nullptr) {
    const int4 s = p.seg_tiles[idx];
    t.m0 = s.x;
    t.n0 = 0;
    t.k0 = s.y;
    t.nkb = s.z;
    t.adapter = s.w;
    return t;
  }
  const int per_group = p.group_m * p.num_n_tiles;
  const int g = idx / per_group;
  const int first_m = g * p.group_m;
  const int gsz = min(p.group_m, p.num_m_tiles - first_m);
  const int r = idx - g * per_group;
  int m_tile = first_m + r % gsz;
  const int n_tile = r / gsz;
  m_tile += p.m_rotate;
  if (m_tile >= p.num_m_tiles) m_tile -= p.num_m_tiles;
  t.m0 = m_tile * BM;
  t.n0 = n_tile;  // multiplied by BN by the caller (BN is a template constant there)
  t.k0 = 0;
  t.nkb = p.nkb_main;
  t.adapter = (p.tile_adapter != nullptr) ? p.tile_adapter[m_tile] : 0;
  return t;
}

template <int BN, bool NF4B = false>
struct SmemPlan {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  // NF4 variant: the packed 4-bit B tile lands behind the bf16 tile it is expanded into
  static constexpr int PACK_BYTES = NF4B ? BN * BK / 2 : 0;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + PACK_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 192 ? 5 : (BN == 128 ? 6 : 8));
  static constexpr int BAR_BYTES = 512;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // + alignment slack
};


template <int BN, int NACC, bool A_MN, bool B_MN, bool B2_MN, int EPI, bool MASK_A, int TP = 0,
          bool NF4B = false>
__global__ void __launch_bounds__(192 + ((MASK_A || NF4B) ? 32 * kNumMaskWarps : 0) +
                                      (TP != 0 ? 32 * kNumCommWarps : 0), 1)
    umma_gemm_kernel(const GemmKParams p, const __grid_constant__ CUtensorMap tmA,
                     const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmA2,
                     const __grid_constant__ CUtensorMap tmB2, const TpParams tp) {
  static_assert(!(MASK_A && TP != 0), "dropout-in-smem and TP fusion are not combined");
  static_assert(!NF4B || (BN == 256 && !MASK_A && !A_MN),
                "the NF4 main loop exists for 256-wide dense tiles only");
  // Thread layout: warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, then (if any) the eight warps
  // that rewrite a stage (dropout mask or NF4 expansion), then (if any) the four warps that
  // move data between GPUs.  COMM_T0 = first thread of the latter.
  constexpr int COMM_T0 = 192 + ((MASK_A || NF4B) ? 32 * kNumMaskWarps : 0);
  using Plan = SmemPlan<BN, NF4B>;
  constexpr bool XFORM = MASK_A || NF4B;  // extra warps rewrite a stage before the MMA reads it
  __shared__ float nf4_lut[16];
  if (NF4B && threadIdx.x < 16) nf4_lut[threadIdx.x] = kNf4Values[threadIdx.x];
  constexpr int STAGES = Plan::STAGES;
  // Two accumulator buffers whenever TMEM (512 columns) has room; the 256-wide
  // two-accumulator variant runs single-buffered.
  constexpr int NBUF = (BN * NACC * 2 <= 512) ? 2 : 1;
  constexpr int TMEM_COLS = BN * NACC * NBUF;
  static_assert(TMEM_COLS <= 512, "TMEM budget");
  constexpr uint32_t TMEM_ALLOC = TMEM_COLS <= 32 ? 32 : TMEM_COLS <= 64 ? 64 : TMEM_COLS <= 128 ? 128 : TMEM_COLS <= 256 ? 256 : 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Plan::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* ready = bars + 2 * STAGES;
  uint64_t* tfull = bars + 3 * STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  AbortCtx ctx{p.err, abort_flag, TP != 0 ? kPeerWaitNs + kLocalWaitNs : kLocalWaitNs};

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      // lane 0 of every warp that rewrites the stage reports for its warp
      mbar_init(&ready[s], MASK_A ? kNumMaskWarps / kMaskGroups : kNumMaskWarps);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (p.nkb2 > 0) {
      tma_prefetch_desc(&tmA2);
      tma_prefetch_desc(&tmB2);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_ALLOC);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        TileCoord t = decode_tile(p, tile);
        const int n0 = (p.seg_tiles != nullptr) ? 0 : t.n0 * BN;
        const int nkb2 = (t.adapter >= 0) ? p.nkb2 : 0;
        const int by = (t.adapter >= 0) ? t.adapter * p.b_adapter_rows : 0;
        const int by2 = (t.adapter >= 0) ? t.adapter * p.b2_adapter_rows : 0;
        const int nkb = (t.adapter < 0 && p.b_adapter_rows > 0) ? 0 : t.nkb;
        const int total = nkb + nkb2;
        if (TP == 1) {
          const int mt = t.m0 / BM;
          const int src = mt / tp.tiles_per_shard;
          if (src != tp.rank) {
            if (!wait_flag_ge(tp.ag_flags + src * tp.tiles_per_shard + (mt - src * tp.tiles_per_shard),
                              tp.epoch, ctx)) {
              ok = false;
              break;
            }
            fence_proxy_async_all();
          }
        }
        for (int kb = 0; kb < total; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, ctx, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + s * Plan::STAGE_BYTES;
          uint8_t* sB = sA + Plan::A_BYTES;
          mbar_expect_tx(&full[s], (NF4B && kb < nkb) ? Plan::A_BYTES + Plan::PACK_BYTES
                                                       : Plan::A_BYTES + Plan::B_BYTES);
          if (kb < nkb) {
            const int kk = t.k0 + kb * BK;
            if (!A_MN) {
              tma_load_2d(sA, &tmA, &full[s], kk, t.m0);
            } else {
              tma_load_2d(sA, &tmA, &full[s], t.m0, kk);
              tma_load_2d(sA + 8192, &tmA, &full[s], t.m0 + 64, kk);
            }
            if (NF4B) {
              // packed bytes (two codes each): K-major W -> [256 rows x 32 B],
              // MN-major W -> [64 rows x 128 B]; tmB is a byte map here
              uint8_t* sP = sB + Plan::B_BYTES;
              if (!B_MN) tma_load_2d(sP, &tmB, &full[s], kk >> 1, n0);
              else tma_load_2d(sP, &tmB, &full[s], n0 >> 1, kk);
            } else if (!B_MN) {
              tma_load_2d(sB, &tmB, &full[s], kk, by + n0);
            } else {
#pragma unroll
              for (int h = 0; h < BN / 64; ++h)
                tma_load_2d(sB + h * 8192, &tmB, &full[s], n0 + 64 * h, by + kk);
            }
          } else {
            const int kk2 = (kb - nkb) * BK;
            tma_load_2d(sA, &tmA2, &full[s], kk2, t.m0);
            if (!B2_MN) {
              tma_load_2d(sB, &tmB2, &full[s], kk2, by2 + n0);
            } else {
#pragma unroll
              for (int h = 0; h < BN / 64; ++h)
                tma_load_2d(sB + h * 8192, &tmB2, &full[s], n0 + 64 * h, by2 + kk2);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t IDESC_MAIN = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint32_t IDESC_SLAB = make_idesc_bf16(BM, BN, 0, B2_MN ? 1 : 0);
      int it = 0;
      int tile_iter = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tile_iter) {
        TileCoord t = decode_tile(p, tile);
        const int nkb2 = (t.adapter >= 0) ? p.nkb2 : 0;
        const int nkb = (t.adapter < 0 && p.b_adapter_rows > 0) ? 0 : t.nkb;
        const int total = nkb + nkb2;
        const int buf = tile_iter % NBUF;
        const uint32_t bph = (tile_iter / NBUF) & 1;
        if (!mbar_wait(&tempty[buf], bph ^ 1, ctx, ERR_WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t acc0 = tmem_base + uint32_t(buf * BN * NACC);
        const uint32_t acc1 = acc0 + BN;
        for (int kb = 0; kb < total; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(XFORM ? &ready[s] : &full[s], ph, ctx,
                         XFORM ? ERR_WAIT_READY : ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sA = smem_u32(smem + s * Plan::STAGE_BYTES);
          const uint32_t sB = sA + Plan::A_BYTES;
          const bool slab = kb >= nkb;
          const bool a_mn = slab ? false : A_MN;
          const bool b_mn = slab ? B2_MN : B_MN;
          const uint32_t d = (NACC == 2 && slab) ? acc1 : acc0;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t da = a_mn ? make_smem_desc_sw128(sA + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sA + kk * 32, 16, 1024);
            const uint64_t db = b_mn ? make_smem_desc_sw128(sB + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sB + kk * 32, 16, 1024);
            const uint32_t accum =
                (NACC == 2 && slab) ? uint32_t(kb > nkb || kk > 0) : uint32_t(kb > 0 || kk > 0);
            umma_bf16_ss(d, da, db, slab ? IDESC_SLAB : IDESC_MAIN, accum);
          }
          tc_commit(&empty[s]);
        }
        if (!ok) break;
        if (total > 0) {
          tc_commit(&tfull[buf]);
        } else {
          mbar_arrive(&tfull[buf]);
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int tile_iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tile_iter) {
      TileCoord t = decode_tile(p, tile);
      const int n0 = (p.seg_tiles != nullptr) ? 0 : t.n0 * BN;
      const int nkb2 = (t.adapter >= 0) ? p.nkb2 : 0;
      const int nkb = (t.adapter < 0 && p.b_adapter_rows > 0) ? 0 : t.nkb;
      const bool has_work = (nkb + nkb2) > 0;
      const bool has_slab = nkb2 > 0;
      const int buf = tile_iter % NBUF;
      const uint32_t bph = (tile_iter / NBUF) & 1;
      bool got = mbar_wait(&tfull[buf], bph, ctx, ERR_WAIT_TMEM_FULL);
      // The reduce-scatter epilogue ends in a named barrier of its 128 threads: they must all
      // take the same branch here, or one that saw an abort earlier would leave the others
      // waiting for its arrival.
      if (TP == 2) got = named_bar_and<1, 128>(got);
      if (!got) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int row = t.m0 + q * 32 + lane;
      const uint32_t lane_addr = uint32_t(q * 32) << 16;
      const uint32_t acc0 = tmem_base + uint32_t(buf * BN * NACC) + lane_addr;
      const uint32_t acc1 = acc0 + BN;

      float tile_scale = p.scale;
      if (EPI == LF_EPI_BF16_ADAPTER_SCALE) {
        tile_scale = (t.adapter >= 0 && p.adapter_scale != nullptr) ? p.adapter_scale[t.adapter]
                                                                    : (t.adapter >= 0 ? p.scale : 0.f);
      }
      uint32_t thresh = p.thresh16;
      float inv_keep = p.inv_keep;
      if (EPI == LF_EPI_BF16_DROPMIX && t.adapter >= 0 && p.adapter_thresh16 != nullptr) {
        thresh = p.adapter_thresh16[t.adapter];
        inv_keep = p.adapter_inv_keep[t.adapter];
      }

#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        uint32_t r2[32];
        if (has_work) {
          tmem_ld_32x32b_x32(acc0 + c * 32, r);
          if (NACC == 2 && has_slab) tmem_ld_32x32b_x32(acc1 + c * 32, r2);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        const int col0 = n0 + c * 32;
        if (EPI == LF_EPI_F32_ACCUM) {
          if (has_work && row < p.M) {
            float* out = reinterpret_cast<float*>(p.out) +
                         (t.adapter >= 0 ? t.adapter * p.out_adapter_stride : 0);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int col = col0 + j;
              if (col < p.N) {
                float* dst = p.out_transposed ? (out + (long long)col * p.ldo + row)
                                              : (out + (long long)row * p.ldo + col);
                *dst += tile_scale * __uint_as_float(r[j]);
              }
            }
          }
        } else {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * tile_scale;
          if (EPI == LF_EPI_BF16_DROPMIX) {
            if (NACC == 2 && has_slab) {
              if (thresh == 0) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += __uint_as_float(r2[j]);
              } else {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const uint32_t keep =
                      dropout_keep8(uint32_t(row + p.row_offset),
                                    uint32_t((col0 + p.col_offset) >> 3) + g, p.stream_id,
                                    p.seed_lo, p.seed_hi, thresh);
#pragma unroll
                  for (int j = 0; j < 8; ++j)
                    if ((keep >> j) & 1u) v[g * 8 + j] += inv_keep * __uint_as_float(r2[g * 8 + j]);
                }
              }
            }
          }
          if (EPI == LF_EPI_BF16 && p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int col = col0 + j;
              if (col < p.N) v[j] += __bfloat162float(p.bias[col]);
            }
          }
          if (row < p.M) {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)row * p.ldo;
            if (TP == 2) {
              // partial tiles stay in THIS GPU's stage [M, N]; the owner of the rows pulls them
              // (row-per-thread stores are merged in the local L2; pushed over NVLink they
              // would travel as 16-byte writes)
              out = tp.rs_peer_stage[tp.rank] + (long long)row * p.N;
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = col0 + g * 8;
              if (col + 8 <= p.N) {
                st_global_v4(out + col, pack_bf16x2(v[g * 8 + 0], v[g * 8 + 1]),
                             pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]),
                             pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]),
                             pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]));
              } else {
                for (int j = 0; j < 8; ++j)
                  if (col + j < p.N) out[col + j] = __float2bfloat16(v[g * 8 + j]);
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&tempty[buf]);
      if (TP == 2) {
        // all 128 epilogue threads have stored their rows of this partial tile
        __threadfence_system();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          const int mt = t.m0 / BM;
          const int owner = mt / tp.tiles_per_shard;
          st_release_sys(tp.rs_peer_cnt[owner] +
                             (tp.rank * tp.tiles_per_shard + (mt - owner * tp.tiles_per_shard)) * p.num_n_tiles +
                             t.n0,
                         tp.epoch);
        }
      }
    }
  } else if (TP == 2 && int(threadIdx.x) >= COMM_T0) {
    // ---- reduce the partials of the rows this rank owns, as they arrive ----
    // Four dedicated warps, concurrent with the GEMM of the other warps: they poll the
    // per-(source, row tile, column tile) flags and sum the bf16 partials in fp32 (+ residual).
    // Every thread keeps the loads of several output vectors from all sources in flight (tp_reduce_item).
    const int et = threadIdx.x - COMM_T0;  // 0..127
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
      tp_reduce_item_any<BM, BN, !NF4B>(tp, et, lt, nt, p.N);
    }
  } else if (TP == 1 && !MASK_A && int(threadIdx.x) >= COMM_T0) {
    // ------------- push this rank's token shard to every peer's gathered buffer -------------
    const int ct = threadIdx.x - COMM_T0;  // 0..127
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
  } else if (NF4B) {
    // ------------- NF4 -> bf16 expansion of the main-loop B stage (256 threads) -------------
    // Thread tt owns 64 consecutive codes along the quantisation direction: one row of a
    // K-major tile, or a quarter row (one 64-column block) of an MN-major tile.  They share
    // one block scale, fetched before the wait so that its latency hides behind the TMA.
    const int tt = threadIdx.x - 192;
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
      TileCoord t = decode_tile(p, tile);
      const int n0 = t.n0 * BN;
      const int nkb2 = (t.adapter >= 0) ? p.nkb2 : 0;
      const int nkb = t.nkb;
      const int total = nkb + nkb2;
      for (int kb = 0; kb < total; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        float scale = 0.f;
        if (kb < nkb) {
          const int kk = kb * BK;
          long long wrow, wblk;
          if (!B_MN) {
            wrow = n0 + tt;
            wblk = kk >> 6;
          } else {
            wrow = kk + (tt >> 2);
            wblk = (n0 >> 6) + (tt & 3);
          }
          if (wrow < p.nf4_rows && wblk < p.nf4_blocks_per_row)
            scale = __ldg(p.nf4_scales + wrow * p.nf4_blocks_per_row + wblk);
        }
        // one answer per warp: its lanes meet again in __syncwarp below
        if (!__all_sync(0xffffffffu, mbar_wait(&full[s], ph, ctx, ERR_WAIT_FULL))) {
          ok = false;
          break;
        }
        if (kb < nkb) {
          uint8_t* sB = smem + s * Plan::STAGE_BYTES + Plan::A_BYTES;
          const uint8_t* sP = sB + Plan::B_BYTES;
          const uint8_t* src;
          uint8_t* dst;
          int sw;
          if (!B_MN) {
            src = sP + tt * 32;
            dst = sB + tt * 128;
            sw = tt & 7;
          } else {
            const int kr = tt >> 2, h = tt & 3;
            src = sP + kr * 128 + h * 32;
            dst = sB + h * 8192 + kr * 128;
            sw = kr & 7;
          }
          const uint4 w0 = *reinterpret_cast<const uint4*>(src);
          const uint4 w1 = *reinterpret_cast<const uint4*>(src + 16);
          const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t byte = (w[c] >> (8 * i)) & 0xffu;
              // even element in the high nibble
              o[i] = pack_bf16x2(nf4_lut[byte >> 4] * scale, nf4_lut[byte & 15u] * scale);
            }
            *reinterpret_cast<uint4*>(dst + ((c ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
          fence_proxy_async_smem();
        }
        // one arrival per warp: 256 arrivals on one barrier word serialise and cost as much as
        // the rewrite itself
        __syncwarp();
        if (lane == 0) mbar_arrive(&ready[s]);
      }
    }
  } else if (MASK_A) {
    // ------------------- dropout mask applied to the A stage in place -------------------
    constexpr int NMT = 32 * kNumMaskWarps / kMaskGroups;  // threads that share one stage
    const int grp = (threadIdx.x - 192) / NMT;             // this thread's group takes stages grp, grp + kMaskGroups, ...
    const int mt = (threadIdx.x - 192) % NMT;
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
      TileCoord t = decode_tile(p, tile);
      const int nkb2 = (t.adapter >= 0) ? p.nkb2 : 0;
      const int nkb = (t.adapter < 0 && p.b_adapter_rows > 0) ? 0 : t.nkb;
      const int total = nkb + nkb2;
      uint32_t thresh = p.thresh16;
      float inv_keep = p.inv_keep;
      if (t.adapter >= 0 && p.adapter_thresh16 != nullptr) {
        thresh = p.adapter_thresh16[t.adapter];
        inv_keep = p.adapter_inv_keep[t.adapter];
      }
      for (int kb = 0; kb < total; ++kb, ++it) {
        if (it % kMaskGroups != grp) continue;
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        // one answer per warp: its lanes meet again in __syncwarp below
        if (!__all_sync(0xffffffffu, mbar_wait(&full[s], ph, ctx, ERR_WAIT_FULL))) {
          ok = false;
          break;
        }
        if (kb < nkb && thresh != 0) {
          uint8_t* sA = smem + s * Plan::STAGE_BYTES;
          const int kk = t.k0 + kb * BK;
#pragma unroll
          for (int i = 0; i < (Plan::A_BYTES / 16) / NMT; ++i) {
            const int qd = mt + i * NMT;  // 16-byte chunk index inside the A stage
            int token, feature;
            if (!A_MN) {
              const int r = qd >> 3;
              const int c = (qd & 7) ^ (r & 7);
              token = t.m0 + r;
              feature = kk + 8 * c;
            } else {
              const int h = qd >> 9;
              const int kr = (qd & 511) >> 3;
              const int c = (qd & 7) ^ (kr & 7);
              token = kk + kr;
              feature = t.m0 + 64 * h + 8 * c;
            }
            const uint32_t keep =
                dropout_keep8(uint32_t(token + p.row_offset), uint32_t((feature + p.col_offset) >> 3),
                              p.stream_id, p.seed_lo, p.seed_hi, thresh);
            uint4* ptr = reinterpret_cast<uint4*>(sA + qd * 16);
            uint4 x = *ptr;
            uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float2 f = unpack_bf16x2(w[j]);
              f.x = ((keep >> (2 * j)) & 1u) ? f.x * inv_keep : 0.f;
              f.y = ((keep >> (2 * j + 1)) & 1u) ? f.y * inv_keep : 0.f;
              w[j] = pack_bf16x2(f.x, f.y);
            }
            *ptr = make_uint4(w[0], w[1], w[2], w[3]);
          }
          fence_proxy_async_smem();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&ready[s]);
      }
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    // Give copies that may still be in flight a bounded time to land before the shared
    // memory and TMEM of this CTA are released.
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_ALLOC);
  }
}

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
template <int BN, int NACC, bool A_MN, bool B_MN, bool B2_MN, int EPI, bool MASK_A, int TP = 0,
          bool NF4B = false>
static int launch_variant(const GemmKParams& kp, const CUtensorMap& tA, const CUtensorMap& tB,
                          const CUtensorMap& tA2, const CUtensorMap& tB2, int grid,
                          cudaStream_t stream, const TpParams& tp = TpParams()) {
  auto kern = umma_gemm_kernel<BN, NACC, A_MN, B_MN, B2_MN, EPI, MASK_A, TP, NF4B>;
  constexpr int smem = SmemPlan<BN, NF4B>::TOTAL;
  static PerDeviceOnce configured;  // one per template instantiation
  {
    cudaError_t e = ensure_max_dynamic_smem(configured, kern, smem);
    if (e != cudaSuccess) {
      fprintf(stderr, "lf_gemm: cudaFuncSetAttribute failed: %s\n", cudaGetErrorString(e));
      return -10;
    }
  }
  const int threads = 192 + ((MASK_A || NF4B) ? 32 * kNumMaskWarps : 0) + (TP != 0 ? 32 * kNumCommWarps : 0);
  kern<<<grid, threads, smem, stream>>>(kp, tA, tB, tA2, tB2, tp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "lf_gemm: launch failed: %s\n", cudaGetErrorString(e));
    return -11;
  }
  return 0;
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace lf

static int gemm_entry(const LfGemmArgs* a, const LfTpArgs* t, const LfNf4Args* q);

extern "C" int lf_gemm(const LfGemmArgs* a) { return gemm_entry(a, nullptr, nullptr); }

// Tensor-parallel fused variants (all-gather -> GEMM, GEMM -> reduce-scatter).
extern "C" int lf_gemm_tp(const LfGemmArgs* a, const LfTpArgs* t) { return gemm_entry(a, t, nullptr); }

// Base weight read as NF4 and expanded to bf16 inside the main loop (no bf16 copy of the
// weight ever exists in global memory).
extern "C" int lf_gemm_nf4(const LfGemmArgs* a, const LfNf4Args* q) {
  if (q == nullptr || q->block_scales == nullptr) return -1;
  return gemm_entry(a, nullptr, q);
}

// Both at once: the tensor-parallel fused kernels with the NF4 weight shard expanded in their
// main loop (the QLoRA configuration of the tensor-parallel layouts).
extern "C" int lf_gemm_tp_nf4(const LfGemmArgs* a, const LfTpArgs* t, const LfNf4Args* q) {
  if (t == nullptr || q == nullptr || q->block_scales == nullptr) return -1;
  return gemm_entry(a, t, q);
}

static int gemm_entry(const LfGemmArgs* a, const LfTpArgs* t, const LfNf4Args* q) {
  using namespace lf;
  if (a == nullptr || a->a == nullptr || a->b == nullptr || a->out == nullptr) return -1;
  if (a->bn != 64 && a->bn != 128 && a->bn != 192 && a->bn != 256) return -2;
  if (a->K2 % BK != 0) return -3;
  const int BN = a->bn;
  if (q != nullptr) {
    // whole 64-code blocks per tile row, dense tiles, adapters only on the slab operand
    if (BN != 256 || a->a_mn || a->mask_a || a->seg_tiles != nullptr || a->b_adapter_rows != 0) return -12;
    if (q->w_cols % 256 != 0 || q->w_rows % 64 != 0 || a->K % BK != 0) return -13;
    if (a->b_mn ? (a->N != q->w_cols || a->K != q->w_rows) : (a->N != q->w_rows || a->K != q->w_cols)) return -14;
    if (!a->b_mn && a->N % 256 != 0) return -13;
  }

  CUtensorMap tA, tB, tA2, tB2;
  int rc;
  // A: K-major box = [128 rows x 64 cols]; MN-major box = [64 rows(k) x 64 cols(mn)]
  rc = make_tmap_2d_b16(&tA, a->a, a->a_rows, a->a_cols, a->a_ld, a->a_mn ? 64 : BM, 64, true);
  if (rc != 0) return -20 + rc;
  if (q == nullptr) {
    rc = make_tmap_2d_b16(&tB, a->b, a->b_rows, a->b_cols, a->b_ld, a->b_mn ? 64 : BN, 64, true);
  } else {
    // byte view of the packed weight [w_rows, w_cols / 2]
    rc = make_tmap_2d_u8(&tB, a->b, (uint64_t)q->w_rows, (uint64_t)q->w_cols / 2, (uint64_t)q->w_cols / 2,
                         a->b_mn ? 64 : 256, a->b_mn ? 128 : 32);
  }
  if (rc != 0) return -30 + rc;
  if (a->K2 > 0) {
    if (a->a2 == nullptr || a->b2 == nullptr) return -4;
    rc = make_tmap_2d_b16(&tA2, a->a2, a->a2_rows, a->a2_cols, a->a2_ld, BM, 64, true);
    if (rc != 0) return -40 + rc;
    rc = make_tmap_2d_b16(&tB2, a->b2, a->b2_rows, a->b2_cols, a->b2_ld, a->b2_mn ? 64 : BN, 64,
                          true);
    if (rc != 0) return -50 + rc;
  } else {
    tA2 = tA;
    tB2 = tB;
  }

  GemmKParams kp;
  kp.M = a->M;
  kp.N = a->N;
  kp.nkb_main = (a->K + BK - 1) / BK;
  kp.nkb2 = a->K2 / BK;
  kp.num_m_tiles = (a->M + BM - 1) / BM;
  kp.num_n_tiles = (a->N + BN - 1) / BN;
  kp.seg_tiles = reinterpret_cast<const int4*>(a->seg_tiles);
  kp.num_tiles = (a->seg_tiles != nullptr) ? a->num_seg_tiles : kp.num_m_tiles * kp.num_n_tiles;
  kp.group_m = a->group_m > 0 ? a->group_m : 8;
  kp.tile_adapter = a->tile_adapter;
  kp.b_adapter_rows = a->b_adapter_rows;
  kp.b2_adapter_rows = a->b2_adapter_rows;
  kp.out = a->out;
  kp.ldo = a->ldo;
  kp.out_adapter_stride = a->out_adapter_stride;
  kp.out_transposed = a->out_transposed;
  kp.adapter_scale = a->adapter_scale;
  kp.scale = a->scale;
  kp.bias = reinterpret_cast<const __nv_bfloat16*>(a->bias);
  kp.adapter_thresh16 = a->adapter_thresh16;
  kp.adapter_inv_keep = a->adapter_inv_keep;
  kp.thresh16 = a->thresh16;
  kp.inv_keep = a->inv_keep;
  kp.seed_lo = a->seed_lo;
  kp.seed_hi = a->seed_hi;
  kp.stream_id = a->stream_id;
  kp.row_offset = a->row_offset;
  kp.col_offset = a->col_offset;
  kp.err = a->err;
  kp.m_rotate = 0;
  kp.nf4_scales = q != nullptr ? q->block_scales : nullptr;
  kp.nf4_rows = q != nullptr ? q->w_rows : 0;
  kp.nf4_blocks_per_row = q != nullptr ? q->w_cols / 64 : 0;
  if (kp.num_tiles <= 0) return 0;

  int grid = sm_count();
  if (a->max_ctas > 0 && a->max_ctas < grid) grid = a->max_ctas;
  if (kp.num_tiles < grid) grid = kp.num_tiles;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);

  if (t != nullptr && t->mode != 0) {
    if (a->seg_tiles != nullptr || a->mask_a) return -6;
    if (t->world < 1 || t->world > 8 || t->rank < 0 || t->rank >= t->world) return -7;
    if (kp.num_m_tiles != t->world * t->tiles_per_shard) return -8;
    TpParams tp = make_tp_params(t);
    // all-gather: start with this rank's own rows; reduce-scatter: finish with them
    kp.m_rotate = (t->mode == 1 ? t->rank : (t->rank + 1) % t->world) * t->tiles_per_shard;
    kp.group_m = t->tiles_per_shard < kp.group_m ? t->tiles_per_shard : kp.group_m;
    const int tkey = (t->mode << 8) | (a->nacc << 4) | ((a->b_mn ? 1 : 0) << 1) | (a->epi == LF_EPI_BF16_DROPMIX);
    if (BN != 256 || a->a_mn) return -9;
    if (q != nullptr) {
      // NF4 weight expanded inside the main loop of the fused compute + collective kernel
      if (a->K2 > 0 && (a->b2_mn != a->b_mn)) return -5;
      switch (tkey) {
        case (1 << 8) | (1 << 4) | 0:
          return launch_variant<256, 1, false, false, false, LF_EPI_BF16, false, 1, true>(kp, tA, tB, tA2, tB2, grid, st, tp);
        case (1 << 8) | (1 << 4) | 2:
          return launch_variant<256, 1, false, true, true, LF_EPI_BF16, false, 1, true>(kp, tA, tB, tA2, tB2, grid, st, tp);
        case (1 << 8) | (2 << 4) | 3:
          return launch_variant<256, 2, false, true, true, LF_EPI_BF16_DROPMIX, false, 1, true>(kp, tA, tB, tA2, tB2, grid, st, tp);
        case (2 << 8) | (1 << 4) | 0:
          return launch_variant<256, 1, false, false, false, LF_EPI_BF16, false, 2, true>(kp, tA, tB, tA2, tB2, grid, st, tp);
        case (2 << 8) | (1 << 4) | 2:
          return launch_variant<256, 1, false, true, true, LF_EPI_BF16, false, 2, true>(kp, tA, tB, tA2, tB2, grid, st, tp);
        case (2 << 8) | (2 << 4) | 3:
          return launch_variant<256, 2, false, true, true, LF_EPI_BF16_DROPMIX, false, 2, true>(kp, tA, tB, tA2, tB2, grid, st, tp);
        default:
          fprintf(stderr, "lf_gemm_tp_nf4: no kernel variant for key 0x%x\n", tkey);
          return -5;
      }
    }
    switch (tkey) {
      case (1 << 8) | (1 << 4) | 0:
        return launch_variant<256, 1, false, false, false, LF_EPI_BF16, false, 1>(kp, tA, tB, tA2, tB2, grid, st, tp);
      case (1 << 8) | (1 << 4) | 2:
        return launch_variant<256, 1, false, true, true, LF_EPI_BF16, false, 1>(kp, tA, tB, tA2, tB2, grid, st, tp);
      case (1 << 8) | (2 << 4) | 3:
        return launch_variant<256, 2, false, true, true, LF_EPI_BF16_DROPMIX, false, 1>(kp, tA, tB, tA2, tB2, grid, st, tp);
      case (2 << 8) | (1 << 4) | 0:
        return launch_variant<256, 1, false, false, false, LF_EPI_BF16, false, 2>(kp, tA, tB, tA2, tB2, grid, st, tp);
      case (2 << 8) | (1 << 4) | 2:
        return launch_variant<256, 1, false, true, true, LF_EPI_BF16, false, 2>(kp, tA, tB, tA2, tB2, grid, st, tp);
      case (2 << 8) | (2 << 4) | 3:
        return launch_variant<256, 2, false, true, true, LF_EPI_BF16_DROPMIX, false, 2>(kp, tA, tB, tA2, tB2, grid, st, tp);
      default:
        fprintf(stderr, "lf_gemm_tp: no kernel variant for key 0x%x\n", tkey);
        return -5;
    }
  }

  if (q != nullptr) {
    const int qkey = (a->nacc << 4) | ((a->b_mn ? 1 : 0) << 1) | (a->epi == LF_EPI_BF16_DROPMIX);
    if (a->K2 > 0 && (a->b2_mn != a->b_mn)) return -5;
    switch (qkey) {
      case (1 << 4) | 0:
        if (a->epi != LF_EPI_BF16) return -5;
        return launch_variant<256, 1, false, false, false, LF_EPI_BF16, false, 0, true>(kp, tA, tB, tA2, tB2, grid, st);
      case (1 << 4) | 2:
        if (a->epi != LF_EPI_BF16) return -5;
        return launch_variant<256, 1, false, true, true, LF_EPI_BF16, false, 0, true>(kp, tA, tB, tA2, tB2, grid, st);
      case (2 << 4) | 3:
        return launch_variant<256, 2, false, true, true, LF_EPI_BF16_DROPMIX, false, 0, true>(kp, tA, tB, tA2, tB2, grid, st);
      default:
        fprintf(stderr, "lf_gemm_nf4: no kernel variant for key 0x%x\n", qkey);
        return -5;
    }
  }

  const int key = (BN << 16) | (a->nacc << 12) | ((a->a_mn ? 1 : 0) << 11) |
                  ((a->b_mn ? 1 : 0) << 10) | ((a->b2_mn ? 1 : 0) << 9) | (a->epi << 4) |
                  (a->mask_a ? 1 : 0);
#define LF_KEY(bn, nacc, amn, bmn, b2mn, epi, mask) \
  (((bn) << 16) | ((nacc) << 12) | ((amn) << 11) | ((bmn) << 10) | ((b2mn) << 9) | ((epi) << 4) | (mask))
#define LF_CASE(bn, nacc, amn, bmn, b2mn, epi, mask)                                         \
  case LF_KEY(bn, nacc, amn, bmn, b2mn, epi, mask):                                          \
    return launch_variant<bn, nacc, (amn) != 0, (bmn) != 0, (b2mn) != 0, epi, (mask) != 0>(  \
        kp, tA, tB, tA2, tB2, grid, st);
  switch (key) {
    // forward base+LoRA and plain NT GEMM
    LF_CASE(256, 1, 0, 0, 0, LF_EPI_BF16, 0)
    LF_CASE(128, 1, 0, 0, 0, LF_EPI_BF16, 0)
    // dX without dropout and plain NN GEMM
    LF_CASE(256, 1, 0, 1, 1, LF_EPI_BF16, 0)
    LF_CASE(128, 1, 0, 1, 1, LF_EPI_BF16, 0)
    // dX with the dropout mask regenerated in the epilogue
    LF_CASE(128, 2, 0, 1, 1, LF_EPI_BF16_DROPMIX, 0)
    LF_CASE(256, 2, 0, 1, 1, LF_EPI_BF16_DROPMIX, 0)
#define LF_SKINNY(bn)                                                \
    /* S' = alpha * dropout(X) A^T */                                  \
    LF_CASE(bn, 1, 0, 0, 0, LF_EPI_BF16_ADAPTER_SCALE, 0)              \
    LF_CASE(bn, 1, 0, 0, 0, LF_EPI_BF16_ADAPTER_SCALE, 1)              \
    /* dS = alpha * dY B */                                            \
    LF_CASE(bn, 1, 0, 1, 0, LF_EPI_BF16_ADAPTER_SCALE, 0)              \
    /* dB += dY^T S'   and   dA += dS^T dropout(X) */                  \
    LF_CASE(bn, 1, 1, 1, 0, LF_EPI_F32_ACCUM, 0)                       \
    LF_CASE(bn, 1, 1, 1, 0, LF_EPI_F32_ACCUM, 1)
    LF_SKINNY(64)
    LF_SKINNY(128)
    LF_SKINNY(192)
    LF_SKINNY(256)
#undef LF_SKINNY
    default:
      fprintf(stderr, "lf_gemm: no kernel variant for key 0x%x\n", key);
      return -5;
  }
#undef LF_CASE
#undef LF_KEY
}
