// Allocation-free entry point (this has no counterpart in the reference project).
//
// Who needs it: code that is not allowed to allocate device memory at the point where it
// must run the norm backward pass — for example a host that pre-sizes all GPU memory at
// start-up and forbids later cudaMalloc calls, a plugin running inside another framework's
// memory pool, or a latency-critical loop where an allocator call (and the implicit
// synchronisation a raw cudaMalloc/cudaFree carries) is unacceptable. The regular entry
// point icb_norm_bwd() needs a caller-provided scratch buffer for the per-CTA partial sums
// of the weight/bias gradients; such callers cannot produce one.
//
// icb_norm_bwd_noalloc() runs the same kernels, but its scratch lives in a fixed array inside
// the library's device image (ICB_NOALLOC_PARTS x ICB_NOALLOC_MAX_D x 2 floats = 4 MiB).
// Every GPU that loads the library holds that array until the process exits.
//
// Rules for callers:
//  * D must be a multiple of 8 and at most ICB_NOALLOC_MAX_D; larger rows are rejected with
//    return code ICB_NOALLOC_TOO_LARGE and a message on stderr (use icb_norm_bwd instead).
//  * The first call on each device looks up the device address of the array (with that device
//    current) and caches it. Make that first call outside of any stream capture.
//  * All calls on one device share the one array. Its contents are whatever the previous call
//    left; the kernels overwrite every partial row they later read, so nothing has to be
//    cleared between calls — but two calls that overlap on the GPU (different streams, no
//    ordering between them) race on it. Serialise them.
//  * No cudaMalloc, cudaFree or allocating library routine is called; inputs and outputs are
//    the caller's buffers exactly as for icb_norm_bwd (dw/db are written, or accumulated into).
#pragma once

#define ICB_NOALLOC_PARTS 128
#define ICB_NOALLOC_MAX_D 4096
#define ICB_NOALLOC_TOO_LARGE (-20)
#define ICB_NOALLOC_SETUP_FAILED (-21)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments as icb_norm_bwd without the scratch pointer. Returns 0 on success.
int icb_norm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                         const void* dres_in, void* dx, void* dw, void* db, int M, int D, float w_offset, int rms,
                         int dtype, int grad_f32, int accumulate, void* stream);

#ifdef __cplusplus
}
#endif
