// Allocation-free entry point. No counterpart in the reference: this is an addition of this library.
//
// Who it is for: callers that drive the kernels from a context where device memory cannot be requested — a host
// thread inside a real-time serving loop that must not take the allocator's locks or trigger a synchronising
// cudaMalloc, or a plugin loaded into another runtime that owns the whole memory pool and forbids foreign
// allocations. Such callers own their input and output buffers already; the only thing the split-KV decode attention
// needs beyond them is scratch for the per-split partial results, and this entry point takes that scratch from an
// array that is part of the loaded library image instead of from an allocator.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Size of the built-in scratch in bytes (8 MiB). Every GPU that loads the library holds this much memory until the
// process exits, whether or not the entry point below is ever called.
long fb_attn_decode_static_scratch_bytes(void);

// Bytes of scratch a call with these sizes needs: rows * nq * nsplit * (hd + 2) floats. Saturates at 2^52 for absurd
// sizes instead of wrapping, and returns -1 for a negative one.
long fb_attn_decode_static_need_bytes(int rows, int nq, int hd, int nsplit);

// Same computation, same arguments and same results as fb_attn_decode (api.h), without the two scratch pointers.
//
// Returns 0 on success; a CUDA error code (> 0) if a runtime call failed; -1 / -2 for the same shape errors as
// fb_attn_decode, and -1 also for sizes outside rows <= 2^20, nq <= 4096, nsplit <= 1024, hd in {64, 128, 256};
// -20 if the call needs more scratch than the built-in array holds (the message from
// fb_attn_decode_static_error() then names both numbers); -21 if the device ordinal is beyond the table of
// per-device set-up records (64 devices).
//
// Device: the entry point works on the CURRENT device (cudaGetDevice) and assumes that the stream `s` and every
// pointer belong to it; it does not check the stream's device. Make the device of `s` current before calling.
//
// Set-up: the first call on each device looks up the device address of the scratch array (with that device current)
// and remembers it. That first call should be made before any stream capture begins; later calls do no set-up.
// The entry point calls no cudaMalloc, cudaFree or other allocating routine, of CUDA, of torch or of any library.
//
// Sharing: every call on a device uses the same array, and the array keeps whatever the previous call left in it.
// Nothing in it needs to start at zero — each call writes every partial result it later reads — but two calls that
// overlap on the GPU (different streams, or different host threads with different streams) race on it. Serialise
// them on one stream or with events.
int fb_attn_decode_static(void* out, const void* q, const void* k_cache, const void* v_cache, const void* proj,
                          long proj_stride, const int* row_slot, const int* row_kvlen, const int* row_base,
                          const unsigned long long* row_mask, const int* block_table, int max_blocks, int kv_block,
                          int rows, int nq, int nkv, int hd, int nsplit, int gated, cudaStream_t s);

// Text of the last error THIS THREAD got from fb_attn_decode_static ("" if none). The buffer is per thread: a thread
// other than the one that made the failing call reads an empty string.
const char* fb_attn_decode_static_error(void);

#ifdef __cplusplus
}
#endif
