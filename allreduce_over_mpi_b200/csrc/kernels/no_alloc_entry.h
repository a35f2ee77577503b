/* An all-reduce entry point that allocates no memory.
 *
 * This has NO counterpart in the reference project; it exists for callers of this library that
 * are not allowed to allocate device memory: plug-ins living inside a host application that has
 * handed the whole GPU to its own memory pool (a cudaMalloc from a guest would fail or starve
 * the host), latency-critical loops where a cudaMalloc (an implicit device synchronisation) is
 * unacceptable, and code running at a point of the host program where the CUDA runtime does
 * not accept allocation calls.
 *
 * ft_local_allreduce_noalloc() makes `n` buffers that all live on the CURRENT GPU hold their
 * element-wise reduction, in place - the one-shot all-reduce of the communicator, for ranks that
 * share one device.  The kernel needs staging space (every buffer is copied aside before any
 * buffer is overwritten).  The communicator takes that space from its heap; this entry point
 * takes it from a fixed array compiled into the library:
 *
 *     FT_NOALLOC_SCRATCH_BYTES = 8 MiB of device memory, per GPU that loads the library,
 *     held until the process exits.
 *
 * Limits and rules:
 *   - n * count * sizeof(dtype), with each buffer's share rounded up to 256 bytes, must fit
 *     in FT_NOALLOC_SCRATCH_BYTES; larger requests are refused with FT_ERR_TOO_LARGE and a message
 *     (ft_noalloc_last_error()).  Nothing is launched in that case.
 *   - The first call on a device does the set-up: it looks up the array's device address (a
 *     one-off, synchronous runtime query).  That first call should come before any stream
 *     capture.
 *   - Every call uses the same array and overwrites the previous call's leftovers before reading
 *     them, so nothing has to be cleared between calls; but two calls that may run on the GPU
 *     at the same time (different streams without ordering) race on it.  Order them.
 *   - No cudaMalloc / cudaFree / allocating library routine is called, on any path.
 */
#ifndef FLEXTREE_NO_ALLOC_ENTRY_H_
#define FLEXTREE_NO_ALLOC_ENTRY_H_

#include "../api/ft_types.h"

#ifdef __cplusplus
extern "C" {
#endif

#define FT_NOALLOC_SCRATCH_BYTES (8u << 20)

/* bufs[0..n): device pointers on the current device, each `count` elements of `dtype`; afterwards
 * every buffer holds the reduction (op: FT_SUM / FT_BAND) of all n, times `scale` for floating
 * types.  Asynchronous on `stream`.  Returns ft_status. */
int ft_local_allreduce_noalloc(void* const* bufs, int n, size_t count, int dtype, int op, float scale, void* stream);
const char* ft_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* FLEXTREE_NO_ALLOC_ENTRY_H_ */
