// A decode-attention entry point that allocates nothing.
//
// This entry point has no counterpart in the reference engine; it exists for embedders of this
// library.
//
// Who it is for: code that drives the decode attention kernel from a place where it may not ask
// the CUDA runtime for memory - a real-time or safety-partitioned process whose device memory was
// carved up once at start-up, a plug-in running inside someone else's allocator discipline, a
// caller in the middle of work during which a cudaMalloc (which may synchronise the device or
// fail under fragmentation) is not acceptable.  The ordinary entry point,
// xb_attn_decode_bf16, wants three scratch buffers from its caller (partial outputs, their
// (max, sum) pairs, and the tickets that elect the merging CTA).  Such a caller has nowhere to get
// them from, so this variant keeps the scratch inside the library: a fixed array in device memory
// that is part of the loaded module.
//
// What that costs and what to watch:
//   * The array is XB_NOALLOC_SCRATCH_BYTES (8 MiB) of device memory on every GPU that loads the
//     library, held until the process exits, whether or not this entry point is ever called.
//   * A call whose scratch need exceeds the array is refused with XB_NOALLOC_TOO_LARGE and does
//     nothing.  The need is tokens * heads * num_splits * (head_dim + 2) * 4 bytes plus the
//     tickets; xb_attn_decode_bf16_noalloc_need() computes it.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress,
//     with that device current).  That first call per device should be made before any stream
//     capture is begun.  Later calls only read the cached address (an atomic: host threads that
//     make a device's first call at the same moment both look the address up and agree).
//   * There is ONE array per device and every call uses it.  It still holds whatever the last call
//     left there.  The part that must start as zeros (the tickets) is cleared on the stream at
//     the start of every call; the rest is fully overwritten before it is read.  Two calls whose
//     kernels may overlap on the GPU (different streams, or no ordering between them) race on the
//     array and give wrong results: serialise them.
//   * It calls no cudaMalloc, cudaFree or any allocating library routine.
//
// Arguments are those of xb_attn_decode_bf16 without part_o, part_ml and tickets; inputs and
// outputs stay the caller's.
#pragma once
#include <cuda_runtime.h>

#define XB_NOALLOC_SCRATCH_BYTES (8u << 20)
#define XB_NOALLOC_TOO_LARGE (-2)   // the call needs more scratch than the built-in array holds
#define XB_NOALLOC_NO_SYMBOL (-3)   // the array's device address could not be obtained

extern "C" {
// Returns 0 on success, a positive cudaError_t of a failed launch or argument check, or one of the
// negative codes above.
int xb_attn_decode_bf16_noalloc(void* out, const void* q, const void* kc, const void* vc, const int* positions,
                                const int* req_of_token, const int* q_start, int num_entries, const int* table,
                                int stride, int nh, int nkv, int d, int ps, int num_pages, int window, float scale,
                                int dec_max, int direct, int split, int num_splits, int tokens, int* err,
                                cudaStream_t stream);
}
