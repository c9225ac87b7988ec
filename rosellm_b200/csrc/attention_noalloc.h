/* rl_attention_decode_noalloc: paged decode attention for callers that cannot allocate.
 *
 * This entry point has no counterpart in chtho-like/rosellm; it exists for users of this
 * library.
 *
 * Who needs it.  The split decode attention (rl_attention with n_splits > 1) wants scratch
 * memory for the partial results of each split, and expects its caller to hand that memory
 * in.  Some callers cannot get device memory at call time: code running under a runtime
 * that owns the whole device heap and hands none out, a plug-in loaded into a host process
 * whose allocator it must not touch, a real-time loop in which cudaMalloc's implicit
 * synchronisation is not acceptable.  For them this variant keeps its scratch inside the
 * library, in a file-scope __device__ array, and calls no cudaMalloc, cudaFree or any other
 * allocating routine.  Inputs and outputs are still the caller's.
 *
 * Limits and rules.
 *  - The scratch holds RL_NOALLOC_SCRATCH_FLOATS floats (4 MiB).  Every GPU on which the
 *    library is loaded sets that much aside until the process exits.  A call needs
 *    n_decode * n_heads * n_splits * (head_dim + 2) floats; a call that needs more is
 *    refused with RL_NOALLOC_TOO_LARGE and launches nothing.  With n_splits == 1 the result
 *    goes straight to out and no scratch is used, so such a call is never refused for its
 *    size.  n_splits is a grid dimension: at most RL_NOALLOC_MAX_SPLITS.
 *  - status must point to an int in device memory (zero it before the first call): a block
 *    table without a page where one is read sets bit 4 there and the access is skipped.  A
 *    null status is refused with RL_NOALLOC_NO_STATUS.
 *  - The kernels are launched with programmatic dependent launch but read nothing before
 *    they wait for the work ahead of them on the stream: a cache write issued just before
 *    this call on the same stream is seen.
 *  - The first call on a device looks up the array's device address
 *    (cudaGetSymbolAddress) with that device current and remembers it.  Make that first
 *    call outside any stream capture.
 *  - All calls on a device share the one array, which keeps whatever the last call left.
 *    Nothing in it has to start at zero: every float a call reads it has written itself
 *    first.  Two calls that overlap on the GPU (different streams, no ordering between
 *    them) race on it; order them.
 *  - Only single-query (decoded) requests are served; prompt portions need no scratch and
 *    go through rl_attention.
 *
 * Arguments are those of rl_attention (see attention.cu) without the prompt-portion tiles
 * and without the scratch pointers.  Returns 0, a positive CUDA error code, or one of the
 * negative codes below; rl_attention_decode_noalloc_error gives a sentence for any of them.
 */
#pragma once
#include <cuda_runtime.h>

#define RL_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define RL_NOALLOC_BAD_HEAD_DIM (-2)
#define RL_NOALLOC_BAD_HEADS (-3)
#define RL_NOALLOC_BAD_SPLITS (-4)
#define RL_NOALLOC_TOO_LARGE (-5)
#define RL_NOALLOC_SETUP_FAILED (-6)
#define RL_NOALLOC_NO_STATUS (-7)
#define RL_NOALLOC_MAX_SPLITS 65535

#ifdef __cplusplus
extern "C" {
#endif

int rl_attention_decode_noalloc(int dtype, const void* q, long q_stride, const void* pool,
                                const int* block_table, int bt_stride, const int* q_start,
                                const int* kv_len, const int* slots, void* out, long out_stride,
                                int n_heads, int n_kv_heads, int head_dim, int page_size,
                                int window, float scale, const int* decode_reqs, int n_decode,
                                int n_splits, int* status, cudaStream_t stream);

const char* rl_attention_decode_noalloc_error(int code);

#ifdef __cplusplus
}
#endif
