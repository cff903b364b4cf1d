/* Greedy token choice without any allocation.
 *
 * This entry point has no counterpart in the reference (MarsPain/easy_gpt.cpp picks the
 * maximum on the CPU, src/sampler.cpp:13-20); it exists for hosts of this library that
 * must not allocate device memory while they run:
 *   - code that replays a captured CUDA graph or runs inside a capture, where cudaMalloc
 *     is an error;
 *   - a serving loop whose memory budget was handed out at start-up and whose allocator
 *     (the framework's or the application's) is not to be entered from the decode path;
 *   - callers that use this shared library through its C symbols alone, without torch,
 *     and have no caching allocator behind them.
 * eg_argmax (sampling.cu) splits every row over several blocks and needs scratch memory
 * for the blocks' partial results, which its caller has to provide.  Here that scratch
 * is a file-scope device array of fixed size, so the caller passes only its input and
 * its output.
 *
 * Limits and rules
 *   - at most EG_ARGMAX_NOALLOC_MAX_ROWS rows per call (more: EG_NOALLOC_TOO_MANY_ROWS,
 *     nothing is launched); any vocabulary size >= 1;
 *   - every GPU that loads the library holds the array (about 65 KB) until the process exits;
 *   - the first call on a device looks the array's device address up
 *     (cudaGetSymbolAddress, with that device current).  Make that first call outside any
 *     stream capture;
 *   - all calls on a device share the array.  Each call clears the part that must start at
 *     zero (in stream order) and relies on nothing a previous call left behind, but two
 *     calls that overlap on the GPU (different streams, no ordering between them) race on
 *     it.  Order them, or use eg_argmax with scratch of your own.
 */
#ifndef EASY_GPT_ARGMAX_NOALLOC_H
#define EASY_GPT_ARGMAX_NOALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EG_ARGMAX_NOALLOC_MAX_ROWS 256

/* return codes: 0 on success, a cudaError_t (> 0) if a CUDA call failed, or one of these */
#define EG_NOALLOC_TOO_MANY_ROWS (-1)
#define EG_NOALLOC_BAD_ARGUMENT (-2)

/* out[r] = lowest index of the maximum of logits[r * ld .. r * ld + vocab), r < rows.
 * logits: float32 on the current device; out: int32 on the current device. */
int eg_argmax_noalloc(cudaStream_t stream, const float* logits, long long ld, int rows, int vocab, int* out);

/* A sentence for a return code of eg_argmax_noalloc (static storage; never null). */
const char* eg_argmax_noalloc_message(int code);

#ifdef __cplusplus
}
#endif
#endif
