// Paged attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for one kind of caller of
// this library.  The ordinary entry point, vapi_paged_attention, needs two scratch buffers
// when the keys of a sequence are divided among several blocks (`splits` > 1), and expects
// the caller to allocate them.  Some callers cannot do that at the moment they need attention:
// a latency-critical serving loop that must never enter the device allocator (its cost is
// unbounded and it may synchronise the device), a host program that was handed a fixed memory
// budget and no allocator of its own, or a plug-in inside another runtime in which device
// memory belongs to the host application.  For them the scratch lives inside the library, in a
// device array of fixed size.
//
//   * The array holds VAPI_ATTN_NOALLOC_MAX_FLOATS floats (8 MiB).  Every GPU on which this
//     library is loaded keeps those 8 MiB until the process exits, whether or not this entry
//     point is ever called.
//   * A call needs n * nh * splits * (d + 2) floats (n query tokens, nh query heads, head size d).
//     A call that needs more is refused with an error message; nothing is launched.
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress) and
//     remembers it for that device.  That first call should be made before any stream capture
//     begins; later calls do no set-up at all.  No call allocates or frees memory, in this
//     library or through any other.
//   * All calls share the one array, and it keeps whatever the last call left in it.  Nothing in
//     it has to start at zero: every slot the combining kernel reads is written earlier in the
//     same call.  For the same reason two calls whose kernels may run at the same time on one
//     GPU (different streams, or different host threads) would overwrite each other's partial
//     results: keep calls on one device in one stream, or otherwise ordered.
//   * With splits == 1 the array is not touched.
//
// Arguments and result are those of vapi_paged_attention (attention.cu) without the two scratch
// pointers: 0 on success, a negative code otherwise, the message through vapi_last_error().
#pragma once
#include <cuda_runtime.h>

#define VAPI_ATTN_NOALLOC_MAX_FLOATS (2 * 1024 * 1024)

extern "C" int vapi_paged_attention_noalloc(const void* q, long long q_row_stride, const void* cache,
                                            int dtype, const int* block_table, int table_stride,
                                            const int* cu_q, const int* seqlens_k, void* out, int n,
                                            int num_seqs, int max_q, int nh, int nkv, int d,
                                            int page_size, int num_pages, float scale, int window,
                                            int splits, int impl, int* status, cudaStream_t stream);
