// SwiGLU gate: out[t, f] = silu(x[t, f]) * x[t, F + f] for x = [gate | up] of
// width 2F.  Formula of fastgen/forward.py:495 (silu(z) = z * sigmoid(z)),
// computed in float32 and rounded once.
#include "common.cuh"

template <typename T>
__global__ void silu_gate_kernel(const T* __restrict__ x, T* __restrict__ out, int ffn, size_t total) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / ffn, f = i - t * ffn;
    const float g = to_f32<T>(x[t * 2 * ffn + f]);
    const float u = to_f32<T>(x[t * 2 * ffn + ffn + f]);
    const float s = g / (1.f + expf(-g));
    out[i] = from_f32<T>(s * u);
  }
}

extern "C" int fg_silu_gate(const void* x, void* out, int dtype, int n_rows, int ffn,
                            cudaStream_t stream) {
  const size_t total = (size_t)n_rows * ffn;
  if (total == 0) return 0;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == FG_F32)
    silu_gate_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)x, (float*)out, ffn, total);
  else if (dtype == FG_BF16)
    silu_gate_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)x, (__nv_bfloat16*)out, ffn, total);
  else
    FG_CHECK_ARG(false, "fg_silu_gate: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_silu_gate");
  return 0;
}
