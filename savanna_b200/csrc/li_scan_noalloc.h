// Allocation-free entry point of the Hyena-LI forward scan.  (This entry point has no counterpart in the
// reference; it exists for embedders of this library.)
//
// Who needs it: host programs that must not allocate device memory when they call into this library —
// for example a serving process that has handed all of the GPU's memory to its own pool at start-up, or a
// control loop that cannot afford the device-wide synchronisation a cudaMalloc / cudaFree may imply.  The
// regular entry point `sb_li_fwd` asks its caller for a scratch buffer of B * ceil(L/TC) * D * 16 floats (the
// per-chunk recurrence states); such callers have nowhere to get it from.
//
// `sb_li_fwd_noalloc` does the same work but keeps that scratch in a fixed array inside the library's device
// image: SB_LI_NOALLOC_SCRATCH_BYTES (16 MiB) per GPU that loads the library, held until the process exits.
// The caller passes only inputs and outputs (same meaning and layout as for `sb_li_fwd`).
//
//   * Limit: B * ceil(L/TC) * D * 16 * 4 bytes must not exceed SB_LI_NOALLOC_SCRATCH_BYTES
//     (e.g. B = 1, L = 8192, TC = 128, D = 4096 fits exactly).  Larger problems are rejected with return
//     code SB_LI_NOALLOC_TOO_LARGE and a message on stderr; nothing is launched.
//   * The first call on each device looks up the array's device address (no allocation, but a runtime query):
//     make that first call during set-up, with the device current, before any stream capture.
//   * The function calls no cudaMalloc / cudaFree and no allocating library routine.
//   * All calls on a device share the one array and it keeps the previous call's contents.  Nothing in it has
//     to start at zero: every entry a call reads was written by the same call's first kernel.  Two calls whose
//     kernels overlap on the GPU (different streams, no ordering between them) race on the array — serialise them.
#pragma once
#include <cuda_runtime.h>

#define SB_LI_NOALLOC_SCRATCH_BYTES (16u * 1024u * 1024u)
#define SB_LI_NOALLOC_TOO_LARGE (-20)
#define SB_LI_NOALLOC_SETUP_FAILED (-21)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0 on success, SB_LI_NOALLOC_TOO_LARGE, SB_LI_NOALLOC_SETUP_FAILED, or a negative launch error.
int sb_li_fwd_noalloc(const void* feat, const float* loglam, const float* R, const float* bias, const float* state_in,
                      float* state_out, void* z, int B, int L, int D, int TC, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
