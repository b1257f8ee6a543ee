/* Decode attention for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference (simonproyt/ziglm); it exists for hosts of this
 * library that are not allowed to call cudaMalloc at the time they need attention: code running while a
 * memory pool is frozen, inside a region where the allocator's lock may not be taken, or embedded in a
 * runtime that hands out all device memory itself and forbids anyone else to ask the driver for more.
 *
 * zlm_attention_decode (attention_tc.cu) needs float scratch for the partial results of its key splits and
 * the caller allocates it.  The variant below computes the same thing but keeps that scratch, and the error
 * word of its bounded waits, in file-scope device arrays of the library, so it calls no cudaMalloc, cudaFree
 * or other allocating routine.  The caller still passes every input and the output.
 *
 * Limit: T * n_heads * n_splits * (head_dim + 2) floats must not exceed
 * ZLM_NOALLOC_SCRATCH_FLOATS (2 Mi floats = 8 MiB, held by every GPU that loads the library until the
 * process exits).  A larger request is refused with ZLM_NOALLOC_ERR_TOO_LARGE and nothing is launched.
 *
 * Set-up: the first call on a device (with that device current) looks up the device address of the scratch
 * once and keeps it, and raises the kernel's shared-memory limit once per head size.  Make the first call
 * for each head size outside any stream capture.
 *
 * Sharing: every call on a device uses the same array, which keeps what the last call left.  Nothing in it
 * has to start at zero (every element the merge reads is written earlier in the same call), but two calls
 * that overlap on the GPU (different streams, or graph branches without an edge between them) race on it.
 * Calls in one stream are safe.
 */
#ifndef ZLM_ATTENTION_NOALLOC_H
#define ZLM_ATTENTION_NOALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZLM_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define ZLM_NOALLOC_ERR_TOO_LARGE (-3)

/* Same arguments and result as zlm_attention_decode without the two scratch pointers.
 * q: bf16 [T, q_row_stride] (query heads first in each row); out: bf16 [T, n_heads * head_dim];
 * k_pages, v_pages: bf16 [n_pages, n_kv_heads, 64, head_dim]; block_table: int32 rows of page numbers,
 * row seq_of_token[t] for token t; positions[t]: position of token t in its sequence.
 * Returns 0, a negative library code (-1 bad argument, -2 unsupported size, -3 scratch too small)
 * or a positive cudaError_t. */
int zlm_attention_decode_noalloc(const void* q, long q_row_stride, void* out, int T, int n_heads, int n_kv_heads,
                                 int head_dim, float scale, int window, const int* positions,
                                 const int* seq_of_token, const int* block_table, int bt_stride, const void* k_pages,
                                 const void* v_pages, long n_pages, int page_size, int n_splits,
                                 cudaStream_t stream);

/* The bounded waits of the kernels behind the function above report through an error word of their own (not
 * the one zlm_attention_tc_status reads).  This reads it into *out (0: every wait completed; 11: a cache page
 * never landed; 12: a stage never drained; 4: copies were still in flight when a block gave up) and clears it.
 * A non-zero code means the output of some call since the last check is not valid.  Allocates nothing;
 * waits for the device.  Returns 0 or a cudaError_t. */
int zlm_attention_decode_noalloc_status(int* out);

/* A sentence for a code returned by zlm_attention_decode_noalloc. */
const char* zlm_attention_decode_noalloc_error(int code);

#ifdef __cplusplus
}
#endif
#endif
