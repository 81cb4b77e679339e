// An entry point of the sampler that allocates nothing.
//
// This entry point has no counterpart in the reference (facebookresearch/fastgen),
// whose sampling goes through PyTorch and its caching allocator.
//
// Who it is for.  fg_sample() works out of a scratch buffer the caller brings, which
// in this package comes from the PyTorch allocator.  Some callers cannot obtain
// device memory at the moment they need to sample:
//   * a host program that gave all device memory to an arena of its own at start-up,
//     so that a later cudaMalloc simply fails;
//   * code that runs while a stream is being captured into a CUDA graph, where the
//     allocation calls are not allowed;
//   * a latency-critical loop that must not hit the implicit device-wide
//     synchronisation an allocation or a free can cause.
// For them fg_sample_noalloc() keeps its scratch in a fixed array inside the library
// itself.  The caller still passes the logits in and the tokens out.
//
// The price.
//   * The array is FG_SAMPLE_NOALLOC_MAX_FLOATS floats (4 MiB).  Every GPU on which
//     the library is loaded holds it until the process exits, used or not.
//   * rows * vocab must not exceed that size; larger calls are refused with an error,
//     never truncated.
//   * All calls share the one array.  Each call overwrites the part it uses before it
//     reads it, so what an earlier call left behind does no harm and nothing has to be
//     cleared; but two calls that overlap in time on the GPU (different streams) race
//     on it.  Run them on one stream, or order them yourself.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current).  Make that first call outside
//     of any stream capture; later calls do no set-up.
//   * Neither this entry point nor anything it calls uses cudaMalloc, cudaFree or an
//     allocating library routine.
#pragma once

#include <cuda_runtime.h>

#define FG_SAMPLE_NOALLOC_MAX_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and results as fg_sample() without `probs_scratch`:
// logits [rows, ld] float32; temps [rows] or null (null or <= 0: greedy); top_p in
// (0, 1]; the draw is keyed by (seed, req_keys[row], positions[row]); out_tokens
// [rows] int32; out_logprobs [rows] float32 or null.  Returns 0, or a negative code
// with the reason in fg_last_error().
int fg_sample_noalloc(const float* logits, int ld, int rows, int vocab, const float* temps, float top_p,
                      unsigned long long seed, const long long* req_keys, const int* positions,
                      int* out_tokens, float* out_logprobs, cudaStream_t stream);

// The largest rows * vocab fg_sample_noalloc() accepts.
long long fg_sample_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
