/* Token picking for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference project: it exists for
 * users of this library who cannot hand the sampler a scratch buffer because
 * they cannot obtain one.  That is the case for a plain C program that links
 * the sampling library without any tensor library behind it, for a serving
 * process that gave all device memory to its own pools at start-up and wants
 * no further calls into the CUDA allocator, and for a latency-critical loop in
 * which an allocation (which may synchronise the device or fail) is not
 * acceptable once the loop runs.
 *
 * alofa_sample_noalloc does what alofa_sample does with a scratch buffer - the
 * two-stage search for the largest logit of every row, and the temperature
 * draw for rows that ask for it - but keeps its scratch in a fixed array that
 * is part of the library image: ALOFA_NOALLOC_MAX_ROWS * 32 (value, index)
 * pairs = 64 KiB of device memory on every GPU that loads the library, held
 * until the process exits.  It calls neither cudaMalloc nor cudaFree nor any
 * routine that allocates.
 *
 *   tokens       [n_rows] int32, device        (output)
 *   logits       [n_rows, vocab] float32, device
 *   temperature  [n_rows] float32, device, or NULL (all rows greedy)
 *   uniform      [n_rows] float32 in [0, 1), device, or NULL
 *   any_hot      0 promises that no temperature is positive (a row that breaks
 *                the promise gets its largest logit)
 *
 * Returns 0 on success, ALOFA_NOALLOC_TOO_MANY_ROWS when n_rows exceeds
 * ALOFA_NOALLOC_MAX_ROWS (nothing is launched), 1 for other bad arguments -
 * among them any_hot set and temperature given without uniform: a row that
 * draws needs its uniform number, and is refused rather than left unwritten -
 * and 2 when the CUDA runtime refuses (symbol lookup or launch).
 *
 * The first call on a device looks up the array's device address (with that
 * device current) and remembers it; make that first call before any stream
 * capture begins.  Host threads may make that first call at the same time:
 * each then looks the same address up and stores the same value.  All calls
 * on a device share the one array: it still holds the previous call's values
 * when the next call starts (every entry a call
 * reads is written by that call first, so nothing needs clearing), and two
 * calls that overlap on the GPU - different streams, no ordering between them
 * - race on it.  Keep calls on one stream, or order them yourself.
 */
#ifndef ALOFA_NO_ALLOC_H
#define ALOFA_NO_ALLOC_H

#include <cuda_runtime.h>

#define ALOFA_NOALLOC_MAX_ROWS 256
#define ALOFA_NOALLOC_TOO_MANY_ROWS 3

#ifdef __cplusplus
extern "C" {
#endif

int alofa_sample_noalloc(int* tokens, const float* logits, const float* temperature, const float* uniform, int n_rows, int vocab,
                         int any_hot, cudaStream_t stream);

/* The largest n_rows alofa_sample_noalloc accepts. */
int alofa_sample_noalloc_max_rows(void);

#ifdef __cplusplus
}
#endif

#endif
