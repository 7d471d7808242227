// Allocation-free entry point (this one has no counterpart in the reference package).
//
// Some hosts embed these kernels where device memory cannot be requested at call time: a
// process whose memory pool was sized and frozen at start-up, a real-time control loop that may
// not take the driver's allocation lock, or a plugin running inside another runtime that owns
// the allocator.  For them the library keeps the scratch it needs in a fixed array that is part
// of the loaded module itself, so the call below touches only memory the caller passes in plus
// that array.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest batch the built-in scratch can serve (one float per matrix, 64 KiB per GPU that loads
// the library, held until the process exits).
#define DION_NOALLOC_MAX_MATRICES 16384

// Return codes.
#define DION_NOALLOC_OK 0
#define DION_NOALLOC_ERR_LAUNCH (-1)     // a CUDA call failed (set-up, memset or launch)
#define DION_NOALLOC_ERR_TOO_LARGE (-2)  // n > DION_NOALLOC_MAX_MATRICES
#define DION_NOALLOC_ERR_BAD_ARGS (-3)   // null pointer or non-positive size

// Newton-Schulz input normalisation without any allocation:
//
//     scale_out[i] = 1 / (sqrt(sum(X_i ** 2)) * mult + eps),   i = 0 .. n-1
//
// X      : n contiguous bf16 matrices of `numel` elements each (device pointer)
// scale_out : n floats (device pointer), written by the call
// stream : cudaStream_t of the caller (may be 0)
//
// The per-matrix sums are accumulated in the module's built-in scratch array, which this call
// zeroes before use.  All calls on one GPU share that array: two calls whose kernels can run at
// the same time (different streams, no ordering between them) race on it and give wrong
// results; serialise them.  The first call on each GPU looks the array's device address up
// (cudaGetSymbolAddress, with that GPU current) and remembers it; make that first call outside
// of any stream capture and before other threads call in on the same GPU.  No cudaMalloc,
// cudaFree or allocating library routine is called on any path.
int dion_frobenius_scale_noalloc(const void* X, int n, long long numel, float mult, float eps,
                                 float* scale_out, void* stream);

#ifdef __cplusplus
}
#endif
