/* Allocation-free MoE routing entry point.
 *
 * This entry point has no counterpart in the reference runtime.  It exists for callers that are not
 * allowed to allocate device memory at the point where they need a routing decision: code running
 * inside a memory-budgeted host (an embedding application that handed all device memory to its own
 * pools), latency-critical callers for which cudaMalloc's implicit device synchronisation is not
 * acceptable, and callers on threads that must not take the allocator's locks.  The regular entry
 * point (nrt_router) expects the caller to provide a scratch buffer for the [rows x experts] score
 * matrix and the grid's arrival counter; this one keeps that scratch inside the library.
 *
 * Scratch: one file-scope device array of NRT_NOALLOC_SCRATCH_BYTES (17 KiB) per GPU that loads the
 * library, held until the process exits.  Limits: rows <= 16, experts <= 256, top_k <= 32,
 * hidden a multiple of 4.  Larger problems are rejected with NRT_NOALLOC_E_LIMIT and nothing is launched.
 *
 * Set-up: the first call on each device resolves the device address of the scratch array (with that
 * device current) and caches it; make that first call before any stream capture begins on the device.
 * Every call clears the arrival counter on `stream` before the kernel, so a call never depends on what
 * the previous one left behind; the score matrix keeps the last call's values until overwritten.
 * All calls on one device share the one scratch array: two calls whose kernels may overlap on the GPU
 * (different streams without an ordering between them) race - serialise them.
 *
 * No cudaMalloc / cudaFree / allocating library routine is called on any path of this function.
 */
#ifndef NAIVERT_B200_NO_ALLOC_H
#define NAIVERT_B200_NO_ALLOC_H

#ifdef __cplusplus
extern "C" {
#endif

#define NRT_NOALLOC_MAX_ROWS 16
#define NRT_NOALLOC_MAX_EXPERTS 256
#define NRT_NOALLOC_SCRATCH_BYTES (NRT_NOALLOC_MAX_ROWS * NRT_NOALLOC_MAX_EXPERTS * 4 + 1024)

#define NRT_NOALLOC_E_LIMIT (-10)     /* a size exceeds the compiled-in maximum */
#define NRT_NOALLOC_E_ARG (-11)       /* null pointer or inconsistent argument */
#define NRT_NOALLOC_E_SETUP (-12)     /* the scratch symbol could not be resolved on this device */

/* Top-k expert routing of `rows` normalised token rows.
 *   xn          bf16 [16][hidden] (rows beyond `rows` are ignored); 8-byte aligned (the kernel reads 4 elements at a time)
 *   w, bias     fp32 router weight [experts][hidden], 16-byte aligned (read as float4), optional choice bias [experts]
 *   sigmoid     1: sigmoid scores (+ bias for the choice), 0: softmax scores
 *   outputs     n_active [1], active_ids [max_slots] (ascending distinct experts), probs [max_slots][16] - all
 *               max_slots * 16 floats are written (zero-filled first), also when rows < 16 -,
 *               topk_ids [16][top_k], topk_p [16][top_k]
 * Returns 0, one of the codes above, or a positive cudaError_t. */
int nrt_router_route_noalloc(const void* xn, const float* w, const float* bias, int hidden, int experts, int rows, int top_k,
                             int sigmoid, int normalize, float route_scale, int* n_active, int* active_ids, float* probs,
                             int* topk_ids, float* topk_p, int max_slots, void* stream);

#ifdef __cplusplus
}
#endif
#endif
