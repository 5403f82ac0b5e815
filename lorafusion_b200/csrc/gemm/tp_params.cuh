// Device-side description of one tensor-parallel fused launch (all-gather -> GEMM or
// GEMM -> reduce-scatter), shared by the single-CTA template (umma_gemm.cu) and the CTA-pair
// kernels (umma_gemm_pair.cu), plus its conversion from the C ABI struct.
#pragma once
#include <cuda_bf16.h>

#include "gemm_api.h"

namespace lf {

constexpr int kNumCommWarps = 4;  // warps that move data between GPUs next to the GEMM roles

struct TpParams {
  int rank, world, tiles_per_shard, epoch;
  const int* ag_flags;
  int* ag_peer_flags[8];
  const __nv_bfloat16* ag_src;
  long long ag_ld;
  int ag_cols;
  __nv_bfloat16* ag_peer_dst[8];
  const __nv_bfloat16* ag2_src;
  long long ag2_ld;
  int ag2_cols;
  __nv_bfloat16* ag2_peer_dst[8];
  __nv_bfloat16* rs_peer_stage[8];
  int* rs_peer_cnt[8];
  const int* rs_cnt;
  int rs_target;
  __nv_bfloat16* rs_out;
  long long rs_ldo;
  const __nv_bfloat16* rs_residual;
};

// Copies the pointers and sizes of the C ABI struct; the caller has validated rank / world.
inline TpParams make_tp_params(const LfTpArgs* t) {
  TpParams tp;
  tp.rank = t->rank;
  tp.world = t->world;
  tp.tiles_per_shard = t->tiles_per_shard;
  tp.epoch = t->epoch;
  tp.ag_flags = (const int*)t->ag_flags;
  tp.ag_src = (const __nv_bfloat16*)t->ag_src;
  tp.ag_ld = t->ag_ld;
  tp.ag_cols = t->ag_cols;
  tp.ag2_src = (const __nv_bfloat16*)t->ag2_src;
  tp.ag2_ld = t->ag2_ld;
  tp.ag2_cols = t->ag2_cols;
  for (int r = 0; r < 8; ++r) {
    tp.ag_peer_flags[r] = (int*)t->ag_peer_flags[r];
    tp.ag_peer_dst[r] = (__nv_bfloat16*)t->ag_peer_dst[r];
    tp.ag2_peer_dst[r] = (__nv_bfloat16*)t->ag2_peer_dst[r];
    tp.rs_peer_stage[r] = (__nv_bfloat16*)t->rs_peer_stage[r];
    tp.rs_peer_cnt[r] = (int*)t->rs_peer_cnt[r];
  }
  tp.rs_cnt = (const int*)t->rs_cnt;
  tp.rs_target = t->rs_target;
  tp.rs_out = (__nv_bfloat16*)t->rs_out;
  tp.rs_ldo = t->rs_ldo;
  tp.rs_residual = (const __nv_bfloat16*)t->rs_residual;
  return tp;
}

#ifdef __CUDACC__
// GEMM -> reduce-scatter, consumer side: sum of all ranks' bf16 partials (+ residual) of one
// ROWS x COLS item of the rows this rank owns, by the 128 threads of the reduce warps (`et` =
// thread index among them).  The loads cross NVLink (2-3 us), so the bytes in flight per SM, not
// the adds, set the pace: every thread keeps U output vectors of 16 bytes from W sources in flight
// at once, and walks the sources W at a time (rank order, so the sum does not depend on U or W).
template <int U, int W, int ROWS, int COLS>
__device__ __forceinline__ void tp_reduce_item(const TpParams& tp, int et, int lt, int nt, int n_cols) {
  constexpr int VEC_PER_ROW = COLS / 8;
  constexpr int NV = ROWS * VEC_PER_ROW;
  const long long grow0 = (long long)tp.rank * tp.tiles_per_shard * ROWS;  // first own row in every source's stage [M, N]
  for (int v0 = et; v0 < NV; v0 += 128 * U) {
    float acc[U][8];
    int row[U], col[U];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * 128;
      row[u] = lt * ROWS + v / VEC_PER_ROW;
      col[u] = nt * COLS + (v % VEC_PER_ROW) * 8;
      live[u] = v < NV && col[u] < n_cols;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
    }
    uint4 res[U];   // the residual travels with the first round of source loads
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (live[u] && tp.rs_residual != nullptr)
        res[u] = ld_global_v4(tp.rs_residual + (long long)row[u] * tp.rs_ldo + col[u]);
    for (int s0 = 0; s0 < tp.world; s0 += W) {
      uint4 raw[U][W];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int i = 0; i < W; ++i)
          if (live[u] && s0 + i < tp.world)
            raw[u][i] = ld_global_v4(tp.rs_peer_stage[s0 + i] + (grow0 + row[u]) * n_cols + col[u]);
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int i = 0; i < W; ++i)
          if (live[u] && s0 + i < tp.world) {
            const uint32_t w[4] = {raw[u][i].x, raw[u][i].y, raw[u][i].z, raw[u][i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = unpack_bf16x2(w[j]);
              acc[u][2 * j] += f.x;
              acc[u][2 * j + 1] += f.y;
            }
          }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!live[u]) continue;
      const long long off = (long long)row[u] * tp.rs_ldo + col[u];
      if (tp.rs_residual != nullptr) {
        const uint32_t w[4] = {res[u].x, res[u].y, res[u].z, res[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(w[j]);
          acc[u][2 * j] += f.x;
          acc[u][2 * j + 1] += f.y;
        }
      }
      st_global_v4(tp.rs_out + off, pack_bf16x2(acc[u][0], acc[u][1]), pack_bf16x2(acc[u][2], acc[u][3]),
                   pack_bf16x2(acc[u][4], acc[u][5]), pack_bf16x2(acc[u][6], acc[u][7]));
    }
  }
}

// Depth by world size: two ranks -> four vectors from both sources at once; more ranks -> two
// vectors from four sources per round.
// DEEP = false for kernels with a tight register budget (the NF4-expanding variants).
template <int ROWS, int COLS, bool DEEP = true>
__device__ __forceinline__ void tp_reduce_item_any(const TpParams& tp, int et, int lt, int nt, int n_cols) {
  if (DEEP && tp.world <= 2)
    tp_reduce_item<4, 2, ROWS, COLS>(tp, et, lt, nt, n_cols);
  else
    tp_reduce_item<2, 4, ROWS, COLS>(tp, et, lt, nt, n_cols);
}
#endif  // __CUDACC__

}  // namespace lf
