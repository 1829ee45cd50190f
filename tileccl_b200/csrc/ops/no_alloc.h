/* Allocation-free verification entry point.
 *
 * This entry point has no counterpart in the reference: it exists for callers of this library
 * that are not allowed to allocate device memory at the moment they want to verify a result.
 * Typical cases: an inference server that handed its whole device-memory budget to its own arena
 * at start-up and treats any later cudaMalloc as a fault; a plug-in running inside a host
 * application that forbids allocator calls on its worker threads; a latency-critical loop in
 * which cudaMalloc / cudaFree (which synchronise the device) would stall every other stream.
 *
 * tcl_max_rel_err_static computes the same number as tcl_max_rel_err (tileccl_ops.h):
 *     max over i of |got[i] - ref[i]| / (|ref[i]| + 1),   got bf16, ref fp32, NaN counts as worst
 * but keeps its scratch (one partial maximum per block of 4096 elements) in a fixed array that
 * lives inside the library image: TCL_STATIC_SCRATCH_FLOATS floats = 64 KiB on every GPU that
 * loads the library, held until the process exits.  The caller still passes the inputs and the
 * one-float result buffer; the call itself performs no cudaMalloc, no cudaFree and calls no
 * allocating library routine.
 *
 * Limits and rules
 *   - n must be at most TCL_STATIC_MAX_ELEMS (= 16384 blocks x 4096 elements = 67,108,864);
 *     a larger n is rejected with TCL_ERR_STATIC_TOO_LARGE before anything is launched.
 *   - The first call on each device looks up the device address of the scratch array
 *     (cudaGetSymbolAddress, with that device current) and caches it.  Make that first call
 *     during set-up, before any stream capture begins on that device.
 *   - All calls on one GPU share the one array.  A call overwrites exactly the slots it later
 *     reads, so nothing needs clearing between calls, but two calls that overlap in time on the
 *     same GPU (different streams, or different host threads) race on it: serialise them.
 *   - got and ref must be readable on the current device; result receives one float.
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TCL_STATIC_SCRATCH_FLOATS 16384
#define TCL_STATIC_ELEMS_PER_BLOCK 4096
#define TCL_STATIC_MAX_ELEMS ((int64_t)TCL_STATIC_SCRATCH_FLOATS * TCL_STATIC_ELEMS_PER_BLOCK)

#define TCL_ERR_STATIC_TOO_LARGE (-2)  /* n exceeds TCL_STATIC_MAX_ELEMS */
#define TCL_ERR_STATIC_BAD_ARG (-3)    /* null pointer or n <= 0 */
#define TCL_ERR_STATIC_SETUP (-4)      /* the scratch array's device address could not be obtained */

/* Returns 0, one of the TCL_ERR_STATIC_* codes, or a positive cudaError_t from the launches. */
int tcl_max_rel_err_static(const void* got_bf16, const float* ref, int64_t n, float* result, void* stream);

/* Human-readable text for a return value of tcl_max_rel_err_static. */
const char* tcl_max_rel_err_static_strerror(int code);

#ifdef __cplusplus
}
#endif
