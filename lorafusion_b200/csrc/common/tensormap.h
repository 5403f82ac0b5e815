// Host-side creation of TMA tensor maps without linking libcuda: the encoder is fetched
// through the runtime's driver-entry-point query, so the library builds on a machine with
// no driver installed.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace lf {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "lorafusion_b200: cuTensorMapEncodeTiled entry point unavailable (%d)\n",
              int(e));
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// The encoder is a driver call and wants a context current in the calling thread.  A thread that
// has made no runtime call yet has none: PyTorch's autograd worker threads are the case that
// matters (a custom Function's backward whose first CUDA call is this encoder; seen as
// CUDA_ERROR_INVALID_CONTEXT when an attention backward was the first backward of a process).
// Binds the primary context of the device that owns `base`.
inline void bind_context_of(const void* base) {
  cudaPointerAttributes attr;
  int dev = -1;
  if (cudaPointerGetAttributes(&attr, base) == cudaSuccess && attr.type == cudaMemoryTypeDevice)
    dev = attr.device;
  else
    cudaGetLastError();
  if (dev >= 0) cudaSetDevice(dev);
  cudaFree(nullptr);
}

// 2-D row-major tensor [rows, cols] (cols contiguous, row pitch ld elements) of 2-byte
// elements, box [box_rows, box_cols], 128-byte swizzle (box_cols * 2 must be 128) or none.
// Out-of-range elements read as zero.  Returns 0 on success.
inline int make_tmap_2d_b16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                            uint64_t ld_elems, uint32_t box_rows, uint32_t box_cols,
                            bool swizzle128) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld_elems * 2) % 16 != 0) return -2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_elems * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_ERROR_INVALID_CONTEXT && r != CUDA_ERROR_NOT_INITIALIZED) break;
    bind_context_of(base);   // no context in this thread yet: bind one and encode again
  }
  if (r != CUDA_SUCCESS)
    fprintf(stderr,
            "lorafusion_b200: cuTensorMapEncodeTiled failed (%d): base %p, [%llu x %llu], pitch %llu B, box [%u x %u]\n",
            int(r), base, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)(ld_elems * 2),
            box_rows, box_cols);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// Same for 1-byte elements (packed NF4 bytes); no swizzle.
inline int make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                           uint64_t ld_bytes, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ld_bytes % 16 != 0) return -2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_ERROR_INVALID_CONTEXT && r != CUDA_ERROR_NOT_INITIALIZED) break;
    bind_context_of(base);
  }
  return r == CUDA_SUCCESS ? 0 : -3;
}

}  // namespace lf
