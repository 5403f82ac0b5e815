// C ABI of the tcgen05 GEMM family.  Python fills LfGemmArgs through ctypes; the layout
// below (all 8-byte fields first, then 4-byte fields) must stay in sync with
// lorafusion_b200/ops/_native.py.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Epilogue selectors.
enum LfGemmEpi {
  LF_EPI_BF16 = 0,           // out[m, n] = bf16(acc * scale + bias[n])
  LF_EPI_BF16_DROPMIX = 1,   // out[m, n] = bf16(acc0 + keep(m, n) * inv_keep * acc1)   (nacc == 2)
  LF_EPI_F32_ACCUM = 2,      // out_f32[adapter][m, n] (or [n, m]) += scale * acc
  LF_EPI_BF16_ADAPTER_SCALE = 3,  // out[m, n] = bf16(acc * adapter_scale[adapter(m tile)])
};

// D[M, N] = sum_k A[m, k] * B[n, k]  (+ second "slab" product A2[m, k2] * B2[n, k2]).
// Operands are 2-D row-major bf16 tensors described as stored in memory:
//   K-major operand : [rows = M or N, cols = K]   (reduction index contiguous)
//   MN-major operand: [rows = K, cols = M or N]   (reduction index strided)
typedef struct LfGemmArgs {
  const void* a;
  int64_t a_rows, a_cols, a_ld;
  const void* b;
  int64_t b_rows, b_cols, b_ld;
  const void* a2;  // slab A operand, always K-major [M, K2]
  int64_t a2_rows, a2_cols, a2_ld;
  const void* b2;  // slab B operand
  int64_t b2_rows, b2_cols, b2_ld;
  const int32_t* tile_adapter;  // adapter id per 128-row M tile (dense mode), <0 = none; may be null
  const int32_t* seg_tiles;     // segment mode: int4 {m0, k0, num_k_blocks, adapter} per tile
  void* out;
  int64_t ldo;
  int64_t out_adapter_stride;   // elements between adapters in `out` (F32_ACCUM)
  const float* adapter_scale;   // per-adapter scalar (ADAPTER_SCALE epilogue)
  const void* bias;             // bf16 [N] or null
  const uint32_t* adapter_thresh16;  // per-adapter dropout threshold (keep iff lane >= thresh) or null
  const float* adapter_inv_keep;     // per-adapter 1 / (1 - p) or null
  int32_t* err;                 // device error word
  void* stream;
  int32_t a_mn, b_mn, b2_mn;
  int32_t M, N, K, K2;
  int32_t bn, nacc, epi, mask_a;
  int32_t b_adapter_rows, b2_adapter_rows;
  int32_t num_seg_tiles;
  int32_t out_transposed;
  float scale;
  float inv_keep;
  uint32_t thresh16;
  uint32_t seed_lo, seed_hi, stream_id;
  int32_t row_offset, col_offset;
  int32_t group_m, max_ctas;
} LfGemmArgs;

// Returns 0 on success, negative on argument/launch errors.
int lf_gemm(const LfGemmArgs* args);

// Extra arguments of the tensor-parallel fused variants.  Token rows are split into `world`
// shards of `tiles_per_shard` 128-row tiles.  All "peer" arrays hold, per rank of the TP
// group, that rank's device pointer to the same symmetric buffer (entry `rank` is local).
//   mode 1 (all-gather -> GEMM): `ag_src` is this rank's gathered A buffer [M, ag_cols]
//     (own shard already in place); the kernel pushes the own shard to `ag_peer_dst[q]` and
//     signals `ag_peer_flags[q][rank * tiles_per_shard + tile] = epoch`; it waits on its own
//     `ag_flags`.  `ag2_*` optionally gathers the LoRA slab operand the same way.  `rs_target`
//     (> 0) is the offset in ints, inside the `ag_flags` buffer, of tiles_per_shard local
//     arrival counters that let several CTAs share the push of one row tile; 0 = one CTA per tile.
//   mode 2 (GEMM -> reduce-scatter): partial tiles go to this rank's own `rs_peer_stage[rank]`
//     ([M, N] bf16; the owner of a row reads it from every source's stage), the flag
//     `rs_peer_cnt[owner][(rank * tiles_per_shard + tile) * num_n_tiles + n_tile]` is set to
//     `epoch`, and rows owned by this rank are reduced into `rs_out` (+ optional
//     `rs_residual`) once the matching flags in `rs_cnt` carry `epoch` (`rs_target` is unused).
typedef struct LfTpArgs {
  const void* ag_flags;
  void* ag_peer_flags[8];
  const void* ag_src;
  int64_t ag_ld;
  void* ag_peer_dst[8];
  const void* ag2_src;
  int64_t ag2_ld;
  void* ag2_peer_dst[8];
  void* rs_peer_stage[8];
  void* rs_peer_cnt[8];
  const void* rs_cnt;
  void* rs_out;
  int64_t rs_ldo;
  const void* rs_residual;
  int32_t mode, rank, world, tiles_per_shard, epoch, rs_target, ag_cols, ag2_cols;
} LfTpArgs;

int lf_gemm_tp(const LfGemmArgs* args, const LfTpArgs* tp);
// CTA-pair (256 x 256 tile) variants of the same; -5 = shape not covered, use lf_gemm_tp.
int lf_gemm_pair_tp(const LfGemmArgs* args, const LfTpArgs* tp);

// NF4 main loop: `args->b` points at the PACKED weight (uint8 [w_rows, w_cols / 2], two 4-bit
// codes per byte, even element in the high nibble) while b_rows / b_cols / b_ld / b_mn describe
// it as if it were the bf16 [w_rows, w_cols] matrix.  `block_scales` holds one fp32 scale per
// 64 consecutive elements of a row (double quantisation already undone).  bn must be 256;
// variants: K-major weight (forward) and MN-major weight (input gradient, with or without
// the dropout-mixing epilogue).
typedef struct LfNf4Args {
  const float* block_scales;
  int64_t w_rows, w_cols;
} LfNf4Args;

int lf_gemm_nf4(const LfGemmArgs* args, const LfNf4Args* nf4);
// Tensor-parallel fused variants reading an NF4 weight shard (see lf_gemm_tp and lf_gemm_nf4).
int lf_gemm_tp_nf4(const LfGemmArgs* args, const LfTpArgs* tp, const LfNf4Args* nf4);

#ifdef __cplusplus
}
#endif
