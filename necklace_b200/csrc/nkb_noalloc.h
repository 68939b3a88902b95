// Allocation-free entry point of the native library.
//
// This has no counterpart in the reference framework.  It exists for callers that
// are not allowed to allocate device memory at the moment they need the result:
// code running between a framework's "memory plan frozen" point and the end of a
// step (for example inside a region whose allocator is locked down for CUDA graph
// capture set-up or by a host application that pre-partitions the GPU's memory and
// forbids cudaMalloc afterwards), plug-ins loaded into a process that owns the
// whole device heap, and latency-critical callers for which a cudaMalloc (which may
// synchronise the device) is unacceptable.  Those callers still own their inputs
// and outputs; what they cannot provide is the temporary fp32 accumulator the
// column-sum kernel needs, so this variant keeps that accumulator inside the
// library image.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

// Largest number of columns the built-in scratch can serve.
#define NKB_NOALLOC_MAX_COLS 65536

// out[c] = sum over r < rows of dy[r * ld + c], c < C (bias gradient of a linear layer).
//   dy  : bf16 device pointer, row pitch ld elements (ld and C even)
//   out : bf16 device pointer, C elements (overwritten)
//   stream : cudaStream_t passed as void*
// Same arithmetic as nkb_colsum + nkb_f32_to_bf16 (fp32 partial sums, atomically
// combined, rounded once to bf16), but the fp32 partial-sum buffer is a file-scope
// `static __device__` array of 2 * NKB_NOALLOC_MAX_COLS floats (512 KiB) that every
// GPU loading this library holds until the process exits.  The function performs no
// cudaMalloc / cudaFree and calls no allocating library routine.
//
// Returns 0 on success, -4 if C > NKB_NOALLOC_MAX_COLS (the caller must split the
// columns or use the allocating path), -3 for odd C / ld, or a positive cudaError_t.
//
// First call on each device: looks the array's device address up with
// cudaGetSymbolAddress (with that device current) and caches it.  Make that first
// call before starting any stream capture on that device.  The cached address is an
// atomic pointer: host threads may race on the first call (both look up and store the
// same value).
//
// The scratch is shared by every call in the process and keeps the previous call's
// contents; each call clears the part it uses on `stream` before accumulating.
// Calls that may overlap on the GPU (different streams without ordering between
// them) race on it: serialise them.
int nkb_colsum_bf16_noalloc(const void* dy, void* out, int rows, int C, long long ld,
                            void* stream);

#ifdef __cplusplus
}
#endif
