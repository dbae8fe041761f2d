// C interface for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference library.  It exists for hosts that hand a
// GPU to this library with the memory budget already spent or fenced off: an inference or
// training server that carved the whole device into its own arena at start-up, a plug-in host
// whose contract forbids allocator calls from extension code, or a latency-critical path that
// must never reach the driver's allocation lock.  Such a caller cannot let the split-K
// statistics kernel obtain its scratch buffer from an allocator, so this variant keeps the
// scratch inside the library image itself.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest scratch request this entry point can serve, in bytes.  The buffer is a static device
// array inside the shared object: every GPU that loads the library holds these bytes until the
// process exits, whether or not the function is ever called.
#define ASDL_B200_NOALLOC_SCRATCH_BYTES (32u << 20)

// C <- alpha * X^T X + beta * C          (symmetric n x n fp32 result, both triangles written)
//
//   x      device pointer, bf16, `rows` x `n` row-major with row pitch `ldx` elements;
//          16-byte aligned, `ldx` a multiple of 8
//   c      device pointer, fp32, n x n with row pitch `ldc` (>= n); read only when beta != 0;
//          16-byte aligned whenever `ldc` is a multiple of 4 (the kernel then uses 16-byte
//          accesses), 4-byte aligned otherwise
//   rows   at most 2^31 - 65; n at most 65536
//   nsplit number of row slices reduced through the scratch buffer; 0 picks one automatically
//   stream a cudaStream_t (0 = the default stream); the call only enqueues work on it
//   err / err_len  optional buffer that receives a message when the call fails
//
// Returns 0 on success.  Nothing is allocated or freed, neither through the CUDA runtime nor
// through any library.  A request whose partial tiles do not fit into
// ASDL_B200_NOALLOC_SCRATCH_BYTES (ceil(n/128) * (ceil(n/128)+1) / 2 * nsplit * 64 KiB) is
// refused with a non-zero return value and a message; pick a smaller nsplit.
//
// Set-up: the first call on a device resolves the device address of the scratch array, which
// takes a short synchronising runtime query.  Make that first call during initialisation, before
// any stream capture is started on that device.
//
// Sharing: all calls use the same scratch array, which keeps whatever the previous call left in
// it.  Every partial tile is completely rewritten before it is read, so nothing has to be
// cleared between calls; but two calls whose kernels can overlap on the GPU (different streams
// without an ordering between them, or different host threads) race on the array and must be
// serialised by the caller.
int asdl_b200_syrk_bf16_noalloc(const void* x, long long rows, int n, long long ldx, float* c,
                                int ldc, float alpha, float beta, int nsplit, void* stream,
                                char* err, int err_len);


// Every wait inside the kernels is bounded; one that runs out leaves its output tile unwritten
// and records a code in a status word of the library image.  This function waits for the work
// enqueued so far on the current device, copies that word to *code (0 = no problem, otherwise
// 1..3 = a wait for a load stage / a free stage / the accumulator ran out) and clears it.
// Returns 0 when *code was written.  Allocates nothing.  Call it after the stream that ran
// asdl_b200_syrk_bf16_noalloc has been synchronised, or simply when the results are needed.
int asdl_b200_noalloc_status(int* code);

#ifdef __cplusplus
}
#endif
