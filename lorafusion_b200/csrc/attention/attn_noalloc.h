// Attention backward for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference framework; it exists for hosts of
// this library that run with a fixed memory budget or inside a region where the CUDA
// allocator must not be touched -- for example a serving process that pre-partitions the
// whole GPU at start-up, a plugin called from another runtime's stream callback, or code
// that has frozen its allocator before entering a latency-critical loop.  Such callers can
// hand over input and output buffers they already own but cannot provide (or let us create)
// the temporary "delta" array the backward needs.
//
// lf_attn_bwd_noalloc does the same work as lf_attn_bwd, but keeps delta
// (sum_d O * dO per head and token, fp32) in a fixed array that lives inside the library
// image, so it calls no cudaMalloc / cudaFree and no allocating library routine.
//
// Limits and rules
//   * Hq * M (query heads times tokens) must not exceed LF_ATTN_NOALLOC_MAX_DELTA
//     (1,048,576 floats = 4 MiB, e.g. 64 heads x 16,384 tokens).  Larger problems are
//     rejected with LF_ATTN_NOALLOC_TOO_LARGE and nothing is launched.
//   * Every GPU that loads the library carries those 4 MiB until the process exits.
//   * The first call on each device looks up the device address of the array (with that
//     device current).  Make that first call outside of any stream capture.  Two host
//     threads that make their first calls at the same time both do the look-up and get the
//     same address; the ordering of their launches is still the callers' business (below).
//   * All calls on a device share the one array.  It is fully rewritten by each call, so
//     nothing has to be cleared, but two calls whose kernels overlap on the GPU (different
//     streams without ordering between them) race on it: serialise them.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define LF_ATTN_NOALLOC_MAX_DELTA (1 << 20)
#define LF_ATTN_NOALLOC_TOO_LARGE (-40)
#define LF_ATTN_NOALLOC_SETUP_FAILED (-41)

// Arguments as for lf_attn_bwd, without the delta scratch pointer:
// qkv, dqkv: [M, ld_qkv] bf16; out, d_out: [M, Hq*128] bf16 with row pitch ldo;
// tiles: device int32 [num_tiles, 4]; lse: fp32 [Hq, M]; err: device error word.
// Returns 0 on success, a negative code otherwise.
int lf_attn_bwd_noalloc(const void* qkv, const void* out, const void* d_out, void* dqkv, long long M,
                        long long ld_qkv, int q_col0, int k_col0, int v_col0, int Hq, int Hkv,
                        const void* tiles, int num_tiles, long long ldo, const float* lse, float scale,
                        int* err, void* stream);

#ifdef __cplusplus
}
#endif
