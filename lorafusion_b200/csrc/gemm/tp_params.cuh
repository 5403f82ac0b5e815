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

}  // namespace lf
