// Shared pieces of the causal varlen GQA attention kernels (head_dim 128, 128x128 tiles).
//
// Tile bookkeeping: the host cuts every sequence of the packed batch into 128-row tiles
// starting at the sequence start, so a query tile and the key tile with the same index are
// aligned and only that diagonal tile needs the causal mask.  A work item is
//   {row0, rows, seq_row0, seq_rows}
// (global row of the tile's first token, valid rows in the tile, global row where the
// sequence starts, sequence length).  Rows of a tile beyond `rows` belong to another
// sequence (or lie past the end of the buffer, where TMA reads zeros); they are computed
// and discarded.
//
// Shared-memory operand layout: a [128 rows x 128 cols] bf16 tile is stored as two
// "panels" of [128 rows x 64 cols] (128-byte rows, TMA 128-byte swizzle, 16 KB each).
//   * used K-major (reduction over the 128 columns): per 16-column step the descriptor
//     start advances 32 B inside a panel, SBO = 1024;
//   * used MN-major (reduction over the 128 rows): per 16-row step the start advances
//     2048 B, LBO = panel stride (16 KB), SBO = 1024.
#pragma once
#include "../common/ptx.cuh"

namespace lf {

constexpr int ATT_D = 128;
constexpr int ATT_TILE = 128;
constexpr int ATT_PANEL_BYTES = ATT_TILE * 128;     // 16 KB
constexpr int ATT_TILE_BYTES = 2 * ATT_PANEL_BYTES; // 32 KB

// Loads a [128 x 128] tile (two panels) whose first element is (row, col) of the 2-D map.
__device__ __forceinline__ void att_load_tile(uint8_t* smem_tile, const CUtensorMap* tm,
                                              uint64_t* bar, int col, int row) {
  tma_load_2d(smem_tile, tm, bar, col, row);
  tma_load_2d(smem_tile + ATT_PANEL_BYTES, tm, bar, col + 64, row);
}

// D[128 x 128] (+)= A * B^T over 128 reduction elements, both operands K-major tiles.
__device__ __forceinline__ void att_mma_kk(uint32_t tmem_d, uint32_t sA, uint32_t sB,
                                           bool accumulate) {
  constexpr uint32_t IDESC = make_idesc_bf16(128, 128, 0, 0);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t off = (k >> 2) * ATT_PANEL_BYTES + (k & 3) * 32;
    umma_bf16_ss(tmem_d, make_smem_desc_sw128(sA + off, 16, 1024),
                 make_smem_desc_sw128(sB + off, 16, 1024), IDESC, (accumulate || k > 0) ? 1u : 0u);
  }
}
// D (+)= A * B with A K-major [128 x 128(k)], B MN-major [128(k) rows x 128(n) cols].
__device__ __forceinline__ void att_mma_kmn(uint32_t tmem_d, uint32_t sA, uint32_t sB,
                                            bool accumulate) {
  constexpr uint32_t IDESC = make_idesc_bf16(128, 128, 0, 1);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t offA = (k >> 2) * ATT_PANEL_BYTES + (k & 3) * 32;
    umma_bf16_ss(tmem_d, make_smem_desc_sw128(sA + offA, 16, 1024),
                 make_smem_desc_sw128(sB + k * 2048, ATT_PANEL_BYTES, 1024), IDESC,
                 (accumulate || k > 0) ? 1u : 0u);
  }
}
// D (+)= A^T * B with A MN-major [128(k) rows x 128(m) cols], B MN-major [128(k) x 128(n)].
__device__ __forceinline__ void att_mma_mnmn(uint32_t tmem_d, uint32_t sA, uint32_t sB,
                                             bool accumulate) {
  constexpr uint32_t IDESC = make_idesc_bf16(128, 128, 1, 1);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    umma_bf16_ss(tmem_d, make_smem_desc_sw128(sA + k * 2048, ATT_PANEL_BYTES, 1024),
                 make_smem_desc_sw128(sB + k * 2048, ATT_PANEL_BYTES, 1024), IDESC,
                 (accumulate || k > 0) ? 1u : 0u);
  }
}

// 2^x on the special-function unit, one instruction (relative error about 2^-22, results below
// 2^-126 flush to zero): exp2f() wraps the same instruction in range handling that the softmax
// does not need (its arguments are bounded above by the lazy-rescaling threshold).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Writes 32 consecutive values of row `r` (columns [c0, c0+32), c0 a multiple of 32) of a
// [128 x 128] bf16 tile into its swizzled two-panel shared-memory layout.
__device__ __forceinline__ void att_store_row_chunk(uint8_t* smem_tile, int r, int c0,
                                                    const float (&v)[32]) {
  uint8_t* panel = smem_tile + (c0 >> 6) * ATT_PANEL_BYTES + r * 128;
  const int chunk0 = (c0 & 63) >> 3;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int phys = (chunk0 + g) ^ (r & 7);
    uint4 q = make_uint4(pack_bf16x2(v[g * 8 + 0], v[g * 8 + 1]), pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]),
                         pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]), pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]));
    *reinterpret_cast<uint4*>(panel + phys * 16) = q;
  }
}

}  // namespace lf
