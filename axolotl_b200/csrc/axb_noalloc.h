// Allocation-free entry point (this one has no counterpart in the reference project).
//
// Who needs it: code that drives these kernels from a place where it may not call cudaMalloc or
// any allocating library routine -- a real-time or signal-handling thread, a plugin running
// inside another framework's memory pool with a fixed budget, a host callback, or an embedder
// that links this library without PyTorch's caching allocator. Such a caller can still own its
// input and output buffers, but it has nowhere to get the temporary buffers the attention
// backward pass needs (the fp32 dQ accumulator and the per-row delta vector).
//
// axb_flash_varlen_bwd_noalloc is the attention backward pass with those temporaries placed in a
// fixed array that lives inside the library image on every GPU that loads it (about 16.3 MB,
// held until the process exits). Everything else -- inputs, outputs, semantics, tolerances -- is
// that of axb_flash_varlen_bwd.
//
// Limits and rules:
//   * T * Hq * D  <= AXB_NOALLOC_MAX_DQ_FLOATS   (4,194,304; e.g. 1024 tokens x 32 heads x 128)
//     Hq * T      <= AXB_NOALLOC_MAX_DELTA_FLOATS (65,536)
//     Larger problems are rejected with AXB_NOALLOC_TOO_LARGE and a message in `err`.
//     An empty problem (T == 0 or no tiles) returns 0 without launching anything; a negative T or
//     a non-positive Hq / D is rejected with AXB_NOALLOC_BAD_SIZE.
//   * The first call on a device looks up the device address of the array (a one-time set-up
//     with that device current). Make that first call outside of any stream capture. Two host
//     threads that make their first call on the same device at the same time both look the
//     address up and store the same value into the per-device cache, which is harmless.
//   * All calls share the one array and it keeps whatever the previous call left in it; each
//     call clears the part that must start at zero. Two calls that overlap on the GPU (different
//     streams, or different host threads without ordering) race on it: serialise them.
//   * Nothing is allocated or freed: no cudaMalloc / cudaFree, no allocating library call.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define AXB_NOALLOC_MAX_DQ_FLOATS 4194304
#define AXB_NOALLOC_MAX_DELTA_FLOATS 65536
#define AXB_NOALLOC_TOO_LARGE (-20)
#define AXB_NOALLOC_SETUP_FAILED (-21)
#define AXB_NOALLOC_BAD_SIZE (-22)

// Same arguments as axb_flash_varlen_bwd without the two scratch pointers; `err` (optional,
// `err_len` bytes) receives a human-readable reason when the return value is negative.
int axb_flash_varlen_bwd_noalloc(const void* qkv, long long ld, const void* dout, const void* out,
                                 long long o_ld, const float* lse2, long long T, int Hq, int Hk,
                                 int D, int q_col0, int k_col0, int v_col0, const void* tiles,
                                 int n_tiles, void* dqkv, long long dqkv_ld, float softmax_scale,
                                 int* status, void* stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
