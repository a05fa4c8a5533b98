/* Column sums of a bf16 matrix with no allocation anywhere on the call path.
 *
 * This entry point has no counterpart in the reference library; it exists for
 * callers of this library that are not in a position to allocate device memory:
 * a host program that hands the GPU's whole memory to its own arena at start-up
 * and forbids later cudaMalloc calls, a real-time or serving loop where an
 * allocator call could stall or fail at a bad moment, or code that runs where the
 * process's allocator must not be touched.  cgk_colsum_bf16 needs the caller to
 * provide a scratch buffer for its per-CTA partial sums; this variant keeps that
 * buffer inside the library image instead, so the caller passes only the input and
 * the output.
 *
 *   out[n] (+)= sum over m of x[m, n]      x: bf16 [M, N], leading dimension ld
 *                                           out: fp32 [N]
 *
 * Limits and rules:
 *  - N <= CGK_COLSUM_NOALLOC_MAX_COLS (16384).  Larger N returns CGK_E_LIMIT (-3)
 *    with a message from cgk_last_error(); M is unlimited.
 *  - The built-in scratch is 4 MiB of device memory (64 x 16384 floats) and stays
 *    resident on every GPU that loads the library until the process exits.
 *  - The first call on a device looks up the device address of the scratch
 *    (cudaGetSymbolAddress).  Make that first call on each device before any
 *    stream capture begins.
 *  - Every call on a device uses the same scratch and leaves its partial sums
 *    there.  Each call overwrites every slot it later reads, so nothing needs
 *    clearing between calls, but two calls that overlap on the GPU (different
 *    streams, or concurrent host threads on the same device) race on it: run
 *    calls to this function on one stream, or order them with events.
 *  - No cudaMalloc, cudaFree or other allocating routine is called, by this
 *    function or by anything it calls.
 *
 * Returns 0, or a negative CGK_E_* code.
 */
#ifndef COGITO_COLSUM_NOALLOC_H
#define COGITO_COLSUM_NOALLOC_H

#define CGK_COLSUM_NOALLOC_MAX_COLS 16384

#ifdef __cplusplus
extern "C" {
#endif

int cgk_colsum_bf16_noalloc(const void* x, long long M, int N, long long ld, float* out,
                            int accumulate, void* stream);

#ifdef __cplusplus
}
#endif
#endif
