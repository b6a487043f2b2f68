/* bn_argmax_noalloc: greedy token choice for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference (artalis-io/bitnet.c); it exists for
 * users of this library.
 *
 * Who needs it.  The library's normal argmax takes its scratch (per-block partial results and a
 * ticket counter) from the caller, and the Python wrapper gets that scratch from torch's
 * allocator.  Some callers cannot do that: a host program that has handed the whole device to
 * an arena of its own and must not see cudaMalloc called behind its back (the call may fail,
 * and it synchronises the whole device even when it succeeds); a latency-bound serving loop
 * that has promised to make no allocator calls once it is running; a plain C caller that links
 * this one library and has no tensor library to borrow memory from.  For them the scratch
 * lives inside the library, in a fixed array in device memory.
 *
 * What it does.  For each of n_rows rows of float32 logits (row r starts at logits + r * ld,
 * vocab entries long) it writes the index of the largest value to out[r]; among equal values
 * the lowest index wins, as in the normal entry point.  logits and out are device pointers
 * supplied by the caller; the kernel runs on `stream`.
 *
 * Limits and rules.
 *  - At most BN_ARGMAX_NOALLOC_MAX_ROWS rows per call.  More is refused with
 *    BN_ARGMAX_NOALLOC_TOO_MANY_ROWS and nothing is launched.
 *  - The scratch is about 129 KB of device memory per GPU, held by every GPU that loads this
 *    library from the moment it is loaded until the process exits, whether or not the entry
 *    point is ever called.
 *  - The first call on a device looks up the device address of that array (once per device,
 *    with that device current).  Make this first call before any stream capture begins.
 *  - Call it with the device current on which logits, out and the stream live: the scratch used
 *    is the current device's.  Logits that live on another device are refused with
 *    BN_ARGMAX_NOALLOC_WRONG_DEVICE and nothing is launched.  Host threads may make their first
 *    calls at the same time; the set-up is done under a lock.
 *  - The entry point calls no cudaMalloc, cudaFree or other allocating routine.
 *  - All calls on a device share the one array, and it keeps what the last call left in it.
 *    The part that must start at zero (the ticket counters) is cleared on the stream at the
 *    start of every call.  Two calls whose kernels overlap on the GPU (different streams
 *    without an ordering between them) race on the scratch and give undefined results:
 *    order them.
 *
 * Returns 0 on success, 1 for bad arguments (null pointers, vocab <= 0, ld < vocab),
 * BN_ARGMAX_NOALLOC_TOO_MANY_ROWS for too many rows, BN_ARGMAX_NOALLOC_NO_DEVICE_ADDRESS if the
 * scratch's device address could not be obtained, BN_ARGMAX_NOALLOC_WRONG_DEVICE if the logits
 * live on another device than the current one, or 100 + the CUDA error code of a failed clear
 * or launch.
 */
#ifndef BN_ARGMAX_NOALLOC_H
#define BN_ARGMAX_NOALLOC_H

#include <cuda_runtime.h>

#define BN_ARGMAX_NOALLOC_MAX_ROWS 256
#define BN_ARGMAX_NOALLOC_TOO_MANY_ROWS 3
#define BN_ARGMAX_NOALLOC_NO_DEVICE_ADDRESS 4
#define BN_ARGMAX_NOALLOC_WRONG_DEVICE 5

#ifdef __cplusplus
extern "C" {
#endif

int bn_argmax_noalloc(const float* logits, int ld, int n_rows, int vocab, int* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

#endif
