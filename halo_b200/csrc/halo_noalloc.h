// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference framework. It exists for callers that are
// not allowed to allocate device memory at the moment they need the kernel: code running inside
// another allocator's critical section or under a fixed memory plan, a host callback or a
// serving loop that must not touch cudaMalloc / the framework's caching allocator, or a plain C
// program that links this library without PyTorch. For them the RMSNorm backward - which
// normally asks its caller for a scratch buffer of per-block partial sums - is offered in a form
// that carries its scratch inside the library.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest hidden size the built-in scratch serves. The scratch is a file-scope device array of
// HALO_NOALLOC_MAX_BLOCKS * HALO_NOALLOC_MAX_HIDDEN floats (9.25 MiB); every GPU that loads the
// library holds it until the process exits.
#define HALO_NOALLOC_MAX_HIDDEN 4096
#define HALO_NOALLOC_MAX_BLOCKS 592

// RMSNorm backward without any allocation:
//   dx = rstd * (g*w - xhat * mean(g*w*xhat)) (+ dres),   dw = sum over rows of g * xhat
// with the same arguments and results as halo_rmsnorm_bwd, except that no scratch pointer is
// passed. g, h, dres (optional), dx: [rows, H] bf16; w: [H] bf16; rstd: [rows] fp32;
// dw_f32 / dw_bf16: [H] outputs (either may be null); accumulate != 0 adds into them.
//
// Returns 0 on success, -1 if H is not a shape the kernel supports, -3 if H exceeds
// HALO_NOALLOC_MAX_HIDDEN (the message goes to stderr), -4 if the scratch symbol could not be
// resolved on the current device, -11 if a launch failed.
//
// The first call on each device resolves the device address of the scratch array (a
// cudaGetSymbolAddress call, made with that device current); make that first call before any
// stream capture begins. The function itself calls no cudaMalloc, cudaFree or allocating library
// routine. All calls on one device share the one scratch array: the array keeps whatever the
// previous call left in it (each call overwrites every partial it later reads, so nothing needs
// clearing), and two calls whose kernels overlap on the GPU - different streams without an
// ordering between them - race on it. Order such calls on one stream or with events.
// The per-device address cache is filled without a lock: two host threads that make their first
// call on one device at the same time both resolve the same address and store the same value.
int halo_rmsnorm_bwd_noalloc(const void* g, const void* h, const void* w, const float* rstd,
                             const void* dres, void* dx, float* dw_f32, void* dw_bf16,
                             int accumulate, long long rows, int H, void* stream);

#ifdef __cplusplus
}
#endif
