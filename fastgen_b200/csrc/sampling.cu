// Sampling on float32 logits: greedy, temperature, nucleus (top-p), logprobs.
//
// Semantics of fastgen/generate.py:887-896 and fastgen/utils/sampling.py:6-31:
//   probs = softmax(logits / temperature)
//   top-p: in descending order a token is dropped when the mass before it
//          exceeds p; a token is then drawn in proportion to what is left.
//   greedy: argmax(logits).
// The reference draws with torch.multinomial from the global generator.  Here
// the draw is a counter-based Philox4x32-10 keyed by (seed, request key,
// position), so a request's tokens do not depend on what else is in the batch.
// Ties in argmax go to the lowest index.  Equal probabilities at the nucleus
// edge are kept or dropped together.
//
// One block per row.  Reductions run in a fixed order for a given vocabulary.
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;

struct ArgMax {
  float v;
  int i;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ ArgMax block_argmax(ArgMax x, ArgMax* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = x;
  __syncthreads();
  ArgMax t = scratch[lane < (blockDim.x >> 5) ? lane : 0];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax y;
    y.v = __shfl_xor_sync(0xffffffffu, t.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, t.i, o);
    t = better(t, y);
  }
  return t;
}

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t (&k)[2]) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
  const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k[0], n1 = lo1, n2 = hi0 ^ c[3] ^ k[1], n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
  k[0] += 0x9E3779B9u;
  k[1] += 0xBB67AE85u;
}

// Uniform in [0, 1) with 24 bits, from Philox4x32-10(key = seed, counter = (req key, position)).
__device__ float philox_uniform(unsigned long long seed, unsigned long long req_key, uint32_t position) {
  uint32_t c[4] = {position, 0u, (uint32_t)req_key, (uint32_t)(req_key >> 32)};
  uint32_t k[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
#pragma unroll
  for (int r = 0; r < 10; ++r) philox_round(c, k);
  return (float)(c[0] >> 8) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temps,
              float top_p, unsigned long long seed, const long long* __restrict__ req_keys,
              const int* __restrict__ positions, int* __restrict__ out_tokens,
              float* __restrict__ out_logprobs, float* __restrict__ probs_scratch, const int* status_word) {
  __shared__ float fs[32];
  __shared__ ArgMax as[32];
  __shared__ float chunk_sums[THREADS];
  __shared__ int chosen;
  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * ld;
  const int tid = threadIdx.x;

  ArgMax am = {-INFINITY, 0x7fffffff};
  if ((((uintptr_t)x) & 15) == 0) {
    // four logits a load (the row is a stream of a few hundred kilobytes that one block reads)
    const int n4 = vocab >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
#pragma unroll 4
    for (int i = tid; i < n4; i += THREADS) {
      const float4 v = x4[i];
      am = better(am, ArgMax{v.x, 4 * i});
      am = better(am, ArgMax{v.y, 4 * i + 1});
      am = better(am, ArgMax{v.z, 4 * i + 2});
      am = better(am, ArgMax{v.w, 4 * i + 3});
    }
    for (int i = 4 * n4 + tid; i < vocab; i += THREADS) am = better(am, ArgMax{x[i], i});
  } else {
    for (int i = tid; i < vocab; i += THREADS) am = better(am, ArgMax{x[i], i});
  }
  am = block_argmax(am, as);
  const float xmax = am.v;
  const float temp = temps ? temps[row] : 0.f;
  int token = am.i;

  if (temp > 0.f) {
    float* e = probs_scratch + (size_t)row * vocab;
    const float inv_t = 1.f / temp;
    // contiguous chunk per thread so that the draw walks the vocabulary in order
    const int chunk = (vocab + THREADS - 1) / THREADS;
    const int lo = min(vocab, tid * chunk), hi = min(vocab, lo + chunk);
    float part = 0.f;
    for (int i = lo; i < hi; ++i) {
      const float v = expf((x[i] - xmax) * inv_t);
      e[i] = v;
      part += v;
    }
    const float z = block_sum(part, fs);
    float threshold = 0.f;
    if (top_p < 1.f) {
      // smallest float v with mass(e > v) <= p * z, by bisection on the bit pattern
      const float target = top_p * z;
      uint32_t blo = 0u, bhi = __float_as_uint(1.0f);
      while (blo < bhi) {
        const uint32_t mid = blo + ((bhi - blo) >> 1);
        const float v = __uint_as_float(mid);
        float s = 0.f;
        for (int i = lo; i < hi; ++i) s += e[i] > v ? e[i] : 0.f;
        s = block_sum(s, fs);
        if (s <= target) bhi = mid; else blo = mid + 1;
      }
      threshold = __uint_as_float(blo);
    }
    float kept = 0.f;
    for (int i = lo; i < hi; ++i) kept += e[i] >= threshold ? e[i] : 0.f;
    chunk_sums[tid] = kept;
    if (tid == 0) chosen = -1;
    __syncthreads();
    if (tid == 0) {
      // serial prefix over 1024 chunk sums: fixed order, negligible time
      float total = 0.f;
      for (int t = 0; t < THREADS; ++t) total += chunk_sums[t];
      const float u = philox_uniform(seed, (unsigned long long)(req_keys ? req_keys[row] : row),
                                     (uint32_t)(positions ? positions[row] : 0));
      const float goal = u * total;
      float run = 0.f, before_pick = 0.f;
      int pick = -1;
      for (int t = 0; t < THREADS; ++t) {
        if (chunk_sums[t] > 0.f) {
          // remember the last chunk with mass, should rounding overshoot the total
          pick = t;
          before_pick = run;
          if (run + chunk_sums[t] > goal) break;
        }
        run += chunk_sums[t];
      }
      chosen = pick;
      fs[0] = goal;
      fs[1] = before_pick;
    }
    __syncthreads();
    if (tid == chosen) {
      const float goal = fs[0];
      float run = fs[1];
      int pick = -1;
      for (int i = lo; i < hi; ++i) {
        if (e[i] >= threshold) {
          pick = i;
          run += e[i];
          if (run > goal) break;
        }
      }
      chosen = pick;
    }
    __syncthreads();
    if (chosen >= 0) token = chosen;
  }

  if (out_logprobs != nullptr) {
    // log softmax(logits)[token] at temperature 1 (generate.py:726-730)
    float part = 0.f;
    for (int i = tid; i < vocab; i += THREADS) part += expf(x[i] - xmax);
    const float z1 = block_sum(part, fs);
    if (tid == 0) out_logprobs[row] = x[token] - xmax - logf(z1);
  }
  if (tid == 0) out_tokens[row] = token;
  // The status word of the step's kernels rides along with the tokens: the host reads both
  // with one copy.  (Every kernel of the step is ahead of this one on the stream.)
  if (status_word != nullptr && row == 0 && tid == 0) out_tokens[gridDim.x] = *status_word;
}

__global__ void uniform_kernel(unsigned long long seed, const long long* req_keys, const int* positions,
                               float* out, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = philox_uniform(seed, (unsigned long long)req_keys[i], (uint32_t)positions[i]);
}

}  // namespace

// logits: [rows, ld] float32 (ld >= vocab).  temps: [rows] or null (null or
// temp <= 0: greedy).  req_keys/positions: what the draw is keyed by.
// probs_scratch: [rows, vocab] float32, needed when any row samples.
// out_logprobs: [rows] or null.  status_word: null, or a device int whose value is copied
// to out_tokens[rows] (out_tokens then has rows + 1 entries).
extern "C" int fg_sample(const float* logits, int ld, int rows, int vocab, const float* temps,
                         float top_p, unsigned long long seed, const long long* req_keys,
                         const int* positions, int* out_tokens, float* out_logprobs,
                         float* probs_scratch, const int* status_word, cudaStream_t stream) {
  if (rows == 0) return 0;
  FG_CHECK_ARG(vocab > 0 && ld >= vocab, "fg_sample: bad sizes vocab=%d ld=%d", vocab, ld);
  FG_CHECK_ARG(temps == nullptr || probs_scratch != nullptr, "fg_sample: sampling needs scratch");
  FG_CHECK_ARG(top_p > 0.f, "fg_sample: top_p must be positive, got %f", (double)top_p);
  sample_kernel<<<rows, THREADS, 0, stream>>>(logits, ld, vocab, temps, top_p, seed, req_keys,
                                              positions, out_tokens, out_logprobs, probs_scratch, status_word);
  FG_CHECK_LAUNCH("fg_sample");
  return 0;
}

// The uniform numbers fg_sample draws, for tests of the sampler.
extern "C" int fg_sample_uniform(unsigned long long seed, const long long* req_keys,
                                 const int* positions, float* out, int n, cudaStream_t stream) {
  if (n == 0) return 0;
  uniform_kernel<<<(n + 127) / 128, 128, 0, stream>>>(seed, req_keys, positions, out, n);
  FG_CHECK_LAUNCH("fg_sample_uniform");
  return 0;
}

// ---------------------------------------------------------------------------------
// The sampler for callers that cannot allocate (see no_alloc.h).
// ---------------------------------------------------------------------------------
#include "no_alloc.h"

// The scratch of fg_sample_noalloc: one array per GPU that loads this library, for
// the life of the process.  In host code this name only stands for the symbol; its
// device address is looked up once per device below.
static __device__ __align__(256) float g_noalloc_scratch[FG_SAMPLE_NOALLOC_MAX_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
}  // namespace

extern "C" long long fg_sample_noalloc_capacity(void) { return FG_SAMPLE_NOALLOC_MAX_FLOATS; }

extern "C" int fg_sample_noalloc(const float* logits, int ld, int rows, int vocab, const float* temps,
                                 float top_p, unsigned long long seed, const long long* req_keys,
                                 const int* positions, int* out_tokens, float* out_logprobs,
                                 cudaStream_t stream) {
  if (rows == 0) return 0;
  FG_CHECK_ARG(rows > 0 && vocab > 0 && ld >= vocab, "fg_sample_noalloc: bad sizes rows=%d vocab=%d ld=%d", rows,
               vocab, ld);
  FG_CHECK_ARG(top_p > 0.f, "fg_sample_noalloc: top_p must be positive, got %f", (double)top_p);
  FG_CHECK_ARG((long long)rows * vocab <= (long long)FG_SAMPLE_NOALLOC_MAX_FLOATS,
               "fg_sample_noalloc: rows * vocab = %lld exceeds the built-in scratch of %d floats; "
               "use fg_sample with a buffer of your own",
               (long long)rows * vocab, FG_SAMPLE_NOALLOC_MAX_FLOATS);
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  FG_CHECK_ARG(e == cudaSuccess && device >= 0 && device < kMaxDevices, "fg_sample_noalloc: no current device: %s",
               cudaGetErrorString(e));
  if (g_noalloc_ptr[device] == nullptr) {
    // first call on this device: find where the array lives there (that device is current)
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
    FG_CHECK_ARG(e == cudaSuccess && ptr != nullptr, "fg_sample_noalloc: cudaGetSymbolAddress failed: %s",
                 cudaGetErrorString(e));
    g_noalloc_ptr[device] = ptr;
  }
  sample_kernel<<<rows, THREADS, 0, stream>>>(logits, ld, vocab, temps, top_p, seed, req_keys, positions,
                                              out_tokens, out_logprobs, g_noalloc_ptr[device], nullptr);
  FG_CHECK_LAUNCH("fg_sample_noalloc");
  return 0;
}
