// Allocation-free entry point of the paged-attention kernel.
//
// This entry point has no counterpart in the reference engine.
//
// Who needs it: code that drives this library from a place where device memory cannot be
// requested — a host callback or signal-safe path, a process whose memory budget was handed out
// up front to other components, or an embedding runtime that forbids cudaMalloc after start-up.
// The regular entry point (msgl_paged_attention) needs a caller-provided workspace whenever the
// KV range is split across CTAs; such callers have nowhere to get one from.
//
// What it does: msgl_paged_attention_noalloc runs the same kernels as msgl_paged_attention but
// keeps the split-KV partial results in a fixed array that is part of the loaded library image
// (MSGL_ATTN_NOALLOC_WS_BYTES bytes of device memory per GPU, held from the moment the library
// is loaded on that GPU until the process exits). It calls no cudaMalloc / cudaFree and no
// allocating library routine; inputs and outputs are still passed by the caller.
//
// Rules for callers:
//   * A problem whose partials do not fit (splits * total_q * hq * (head_dim + 1) floats more
//     than the array holds) is rejected with MSGL_BAD_ARG and a message in msgl_last_error();
//     lower `splits` or the batch.
//   * The first call on each device that actually splits the KV range (splits > 1) looks up the
//     device address of the array (a blocking runtime query). Make that first call outside of
//     any stream capture. The looked-up address is remembered per device in a plain table that
//     is written without a lock: two threads racing on the first call both store the same value,
//     which is harmless, but do not rely on more than that.
//   * All calls on one device share the one array, and it keeps whatever the previous call left
//     in it. Nothing in it has to be cleared between calls: for every query row that belongs to
//     a request (the rows below cu_q[B]) each slot the merge step reads is written earlier in
//     the same call; rows past cu_q[B] are padding and come back as zeros without touching the
//     array. Two calls that overlap in time on the same device (different streams, or different
//     threads) would trample each other's partials, so serialise them.
#pragma once
#include <cuda_runtime.h>

#define MSGL_ATTN_NOALLOC_WS_BYTES (16u << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments as msgl_paged_attention without the `workspace` pointer.
__attribute__((visibility("default"))) int msgl_paged_attention_noalloc(
    const void* kv_map, const void* q, void* out, const void* block_table, int bt_stride, const void* cu_q,
    const void* seq_lens, const void* k_scale, const void* v_scale, const void* mask, long long mask_stride, int B,
    int total_q, int max_q, int hq, int hk, int head_dim, int page_size, int num_pages, int layer, int num_layers,
    int kv_fp8, int causal, int window, int splits, float scale, int dtype, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
