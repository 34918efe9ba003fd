// C interface of the paged decode-attention kernels in attention_decode.cu.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Split-KV decode attention over one layer of the paged cache. The caller supplies the fp32 workspace for the
// per-split partial results. See attention_decode.cu for the argument contract.
int ksana_paged_decode(const void* q, int ldq, const void* cache, int cache_kind, const int* block_tables,
                       int max_blocks, const int* cu_q, const int* kv_lens, int seq_base, int num_seqs, int max_q_len,
                       int max_kv_len, int h, int hk, int d, int block_size, float scale, const float* alibi,
                       float k_scale, float v_scale, void* out, int ldo, float* workspace, long long workspace_floats,
                       cudaStream_t stream);

// Same computation and same arguments as ksana_paged_decode, minus the workspace: nothing is allocated, by this
// function or on its behalf. (This entry point has no counterpart in the reference engine.)
//
// Who it is for: code that drives the kernels but is not in a position to call cudaMalloc or to go through an
// allocating framework - a real-time serving loop that must never block on the allocator, a plug-in running
// inside another program's memory budget, or a host that hands this library nothing but finished input and output
// buffers. Such a caller cannot provide the scratch space that splitting the KV range across thread blocks needs,
// so the scratch is a fixed 8 MiB array compiled into the library (ksana_paged_decode_static_scratch_floats()
// floats). Every GPU on which the library is loaded carries those 8 MiB until the process exits.
//
// Rules that follow from the shared array:
//  * A problem needing more than the array holds (num_seqs * max_q_len * h * kv_splits * 129 floats) is refused
//    with -7 and nothing is launched; ksana_paged_decode_static_error(code) returns the explanation as text.
//  * All calls on a device use the same array. Calls that can overlap on the GPU (different streams, or
//    different host threads on different streams) overwrite each other's partial results: keep them on one
//    stream or order them with events.
//  * The array keeps whatever the previous call left in it. Nothing in it has to start at zero: every slot the
//    merge step reads is first written by the same call, so no clearing pass is needed between calls.
//  * The first call made on a device looks up the array's device address (cudaGetSymbolAddress, with that device
//    current) and remembers it. Make that first call outside of any stream capture; later calls only launch.
// Returns 0 on success, a negative code otherwise.
int ksana_paged_decode_static(const void* q, int ldq, const void* cache, int cache_kind, const int* block_tables,
                              int max_blocks, const int* cu_q, const int* kv_lens, int seq_base, int num_seqs,
                              int max_q_len, int max_kv_len, int h, int hk, int d, int block_size, float scale,
                              const float* alibi, float k_scale, float v_scale, void* out, int ldo,
                              cudaStream_t stream);

// Capacity of the built-in scratch array, in floats.
long long ksana_paged_decode_static_scratch_floats(void);
// Human-readable text for a return code of ksana_paged_decode_static.
const char* ksana_paged_decode_static_error(int code);

#ifdef __cplusplus
}
#endif
