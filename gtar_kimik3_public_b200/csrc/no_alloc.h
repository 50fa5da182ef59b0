// Entry points of the kernel library that allocate no device memory.
//
// This interface has no counterpart in the reference (qtris123/gtar-kimik3-public has no native
// code and lets PyTorch allocate whatever its attention needs): it exists for callers of THIS
// library that cannot, or must not, allocate while they decode:
//
//   * a serving process that has given every free byte of the GPU to its key/value cache, so a
//     cudaMalloc for a few megabytes of scratch fails or forces it to shrink the cache;
//   * a C or C++ host that links the library without PyTorch and owns nothing but its inputs and
//     outputs: there is no caching allocator to borrow scratch from;
//   * a latency-critical decode loop: cudaMalloc and cudaFree synchronise the whole device, which
//     stalls every stream for far longer than the attention itself takes.
//
// What is given up in exchange: the scratch is one fixed array inside the library (see the limit
// below), every GPU that loads the library holds it until the process exits, and all calls share it.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest scratch the entry point below can use, in bytes.  A call needs
//   n_seqs * n_q * n_splits * (head_dim + 2) * 4   bytes
// (e.g. 64 sequences x 16 query heads x 8 splits x 130 floats = 4.1 MiB) and is refused with a
// clear error beyond this.
#define GK_NO_ALLOC_SCRATCH_BYTES (8u << 20)

// Split-KV decode attention over the paged cache in bfloat16 — the same computation, arguments and
// results as gk_attention_decode_bf16 — except that the partial results of the splits live in a
// file-scope device array of GK_NO_ALLOC_SCRATCH_BYTES instead of caller-provided scratch.  The
// function calls no cudaMalloc, cudaFree or other allocating routine.
//
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress) and
//     raises the kernel's shared-memory limit; make that first call with the device current and
//     before any stream capture begins.
//   * The array keeps whatever the previous call left in it.  Nothing in it has to start at zero:
//     every entry a call reads is written earlier in the same call.
//   * Calls share the one array: two calls whose kernels can overlap on the GPU (different streams,
//     or a launch order that lets a later call start before an earlier one has finished) race on it.
//     Issue them in one stream.
//
// Returns 0 on success; otherwise gk_last_error() describes the refusal.
int gk_attention_decode_bf16_no_alloc(const void* q, const void* k_pages, const void* v_pages, void* out,
                                      const int* kv_len, const int* slots, const int* block_table, int n_seqs,
                                      int n_q, int n_kv, int head_dim, int max_pages, int page_size, float scale,
                                      int window, int n_splits, void* stream);

#ifdef __cplusplus
}
#endif
