/* Single-GPU token dispatch that allocates nothing.
 *
 * This entry point has no counterpart in the reference library (deepseek-ai/DeepEP).
 *
 * Who it is for. Some hosts of this library are not allowed to obtain device memory at the
 * moment they need a dispatch: a plug-in running inside an inference server whose memory
 * pool is owned and fully reserved by the server; code that runs while the process is pinned
 * to a fixed memory budget that an allocation would break; a callback in which cudaMalloc
 * would force a device-wide synchronisation and stall every other stream of the process.
 * The regular path (ElasticBuffer.dispatch) creates its heap with cudaMalloc, its status
 * words with cudaHostAlloc and its outputs through the PyTorch allocator, so those callers
 * cannot use it. This function gives them the same kernels with every byte of working
 * memory taken from one fixed device array that is part of the library image.
 *
 * What it does. For a world of ONE rank it sends every token that selects at least one valid
 * expert through the dispatch kernel and the local epilogue, and produces either
 *   - do_expand = 0: the selected tokens in token order, with their routing, or
 *   - do_expand = 1: the expert-major layout (one row per token and selected expert, expert e
 *     occupying rows [align(psum[e-1]), psum[e]) with `expert_alignment`),
 * i.e. the permutation a single-GPU MoE layer needs before its grouped GEMM. The caller
 * passes inputs AND outputs; results are bit-identical to ElasticBuffer.dispatch on a
 * one-rank group.
 *
 * Limits (fixed at build time, a call beyond them returns an error code and launches nothing):
 *   tokens <= DEEPEP_B200_NOALLOC_MAX_TOKENS, row bytes <= DEEPEP_B200_NOALLOC_MAX_ROW_BYTES
 *   (multiple of 16), top-k <= DEEPEP_B200_NOALLOC_MAX_TOPK, experts <=
 *   DEEPEP_B200_NOALLOC_MAX_EXPERTS. The scratch array is about 12 MB
 *   (deepep_b200_noalloc_scratch_bytes() gives the exact figure); every GPU that loads the
 *   library holds that much from load until the process exits, whether or not this function is
 *   ever called.
 *
 * Set-up. The first call on a device resolves the device address of the scratch array with
 * cudaGetSymbolAddress (the array's name means nothing as a pointer in host code) and reads two
 * device attributes. Make that first call with the device current and BEFORE any stream
 * capture begins on it; later calls on the same device only launch kernels.
 *
 * Sharing. All calls on a device use the same scratch array, and it keeps what the previous
 * call left there. Nothing has to be cleared by the caller: the control words are tagged with a
 * call counter, the counters the kernels use are either monotonic or reset by the kernel that
 * used them. Because of the sharing, two calls whose kernels can overlap on the GPU (different
 * streams without an ordering between them, or several host threads) race on the scratch and
 * give undefined results: keep all calls on one device ordered, e.g. on one stream. Host-side
 * bookkeeping is protected by a mutex; that does not order the kernels.
 *
 * Errors. The kernels never trap. If one of their bounded waits runs out they record a status
 * word in the scratch array; deepep_b200_noalloc_status() copies it out (0 = healthy). A
 * non-zero status is sticky: from then on every wait of later calls on that device falls
 * through at once and their outputs are not to be trusted. Once the cause is gone,
 * deepep_b200_noalloc_reset() waits for the device and clears the status and the counters.
 */
#ifndef DEEPEP_B200_DISPATCH_NOALLOC_H_
#define DEEPEP_B200_DISPATCH_NOALLOC_H_

#include <stddef.h>

#define DEEPEP_B200_NOALLOC_MAX_TOKENS 2048
#define DEEPEP_B200_NOALLOC_MAX_ROW_BYTES 4096
#define DEEPEP_B200_NOALLOC_MAX_TOPK 32
#define DEEPEP_B200_NOALLOC_MAX_EXPERTS 256

#define DEEPEP_B200_NOALLOC_OK 0
#define DEEPEP_B200_NOALLOC_ERR_TOKENS 1     /* num_tokens beyond the maximum */
#define DEEPEP_B200_NOALLOC_ERR_ROW_BYTES 2  /* row_bytes beyond the maximum or not a multiple of 16 */
#define DEEPEP_B200_NOALLOC_ERR_TOPK 3
#define DEEPEP_B200_NOALLOC_ERR_EXPERTS 4
#define DEEPEP_B200_NOALLOC_ERR_ARGUMENT 5   /* null / misaligned pointer, bad alignment value, recv_x with too few rows */
#define DEEPEP_B200_NOALLOC_ERR_CUDA 6       /* a CUDA call failed (cudaGetLastError has the reason) */

#ifdef __cplusplus
extern "C" {
#endif

/* Bytes of the fixed scratch array. */
size_t deepep_b200_noalloc_scratch_bytes(void);

/* All pointers are device pointers on the current device; the work is queued on `stream`
 * (a cudaStream_t passed as void*, NULL = default stream) and the function returns without
 * waiting for it.
 *
 * inputs
 *   x                  [num_tokens] rows of `row_bytes` bytes (any element type), 16-byte aligned,
 *                      consecutive rows `x_stride_bytes` apart (multiple of 16)
 *   topk_idx           [num_tokens, num_topk] int64 expert ids, -1 = unused lane, distinct per token
 *   topk_weights       [num_tokens, num_topk] float, or NULL
 * outputs
 *   recv_x             [num_recv_x_rows] rows of `row_bytes`; needs num_tokens rows (do_expand = 0) or
 *                      num_tokens * num_topk + num_experts * (expert_alignment - 1) rows (do_expand = 1);
 *                      fewer rows are refused with DEEPEP_B200_NOALLOC_ERR_ARGUMENT
 *   recv_topk_idx      [num_tokens, num_topk] int64 (do_expand = 0; may be NULL)
 *   recv_topk_weights  [num_tokens, num_topk] (do_expand = 0) or [num_recv_x_rows] (do_expand = 1); may be NULL
 *   recv_src_metadata  [num_tokens, num_topk + 2] int32: {source token, first used lane, row per lane or -1}
 *   psum_num_recv_per_expert  [num_experts + 1] int32, see ElasticBuffer's EPHandle; last = total rows
 *   num_recv_tokens    [1] int32, tokens that selected at least one expert
 * `num_sms` = thread blocks of the dispatch kernel (<= 0 picks 8).
 * Returns one of the DEEPEP_B200_NOALLOC_* codes. */
int deepep_b200_dispatch_local_noalloc(const void* x, long long x_stride_bytes, int row_bytes, const long long* topk_idx,
                                       const float* topk_weights, int num_tokens, int num_topk, int num_experts,
                                       int do_expand, int expert_alignment, int num_sms, void* recv_x, int num_recv_x_rows,
                                       long long* recv_topk_idx, float* recv_topk_weights, int* recv_src_metadata,
                                       int* psum_num_recv_per_expert, int* num_recv_tokens, void* stream);

/* Copies the status word of the current device to *record (0 = no wait has ever run out).
 * Synchronises with the device. */
int deepep_b200_noalloc_status(unsigned long long* record);

/* After a non-zero status: waits for the device, then clears the status word and the counters
 * in the scratch array of the current device so that later calls work again. Allocates nothing. */
int deepep_b200_noalloc_reset(void);

#ifdef __cplusplus
}
#endif

#endif /* DEEPEP_B200_DISPATCH_NOALLOC_H_ */
