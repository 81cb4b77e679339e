// SwiGLU gate: out[t, f] = silu(gate[t, f]) * up[t, f] for x of width 2F that holds
// gate and up either as halves [gate | up] (interleave 0) or interleaved in blocks
// of 8 columns (interleave 8: columns 16b..16b+7 gate, 16b+8..16b+15 up of
// features 8b..8b+7, the layout of the fused gate/up weight).  Formula of fastgen/forward.py:495 (silu(z) = z * sigmoid(z)),
// computed in float32 and rounded once.
#include "common.cuh"

template <typename T>
__global__ void silu_gate_kernel(const T* __restrict__ x, T* __restrict__ out, int ffn, size_t total,
                                 int interleave) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / ffn, f = i - t * ffn;
    const size_t gi = interleave ? (f / 8) * 16 + (f % 8) : f;
    const size_t ui = interleave ? gi + 8 : ffn + f;
    const float g = to_f32<T>(x[t * 2 * ffn + gi]);
    const float u = to_f32<T>(x[t * 2 * ffn + ui]);
    const float s = g / (1.f + expf(-g));
    out[i] = from_f32<T>(s * u);
  }
}

// bfloat16 rows whose width is a multiple of 8: eight elements (16 bytes) a thread
__global__ void silu_gate_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                        int ffn, size_t total8, int interleave) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const int per_row = ffn / 8;
  for (; i < total8; i += stride) {
    const size_t t = i / per_row, f = (i - t * per_row) * 8;
    const uint4 g4 = *reinterpret_cast<const uint4*>(x + t * 2 * ffn + (interleave ? 2 * f : f));
    const uint4 u4 = *reinterpret_cast<const uint4*>(x + t * 2 * ffn + (interleave ? 2 * f + 8 : ffn + f));
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
      o2[k] = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * ffn + f) = o4;
  }
}

extern "C" int fg_silu_gate(const void* x, void* out, int dtype, int n_rows, int ffn, int interleave,
                            cudaStream_t stream) {
  FG_CHECK_ARG(interleave == 0 || (interleave == 8 && ffn % 8 == 0), "fg_silu_gate: bad interleave %d for width %d",
               interleave, ffn);
  const size_t total = (size_t)n_rows * ffn;
  if (total == 0) return 0;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == FG_BF16 && ffn % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const size_t total8 = total / 8;
    size_t b8 = (total8 + threads - 1) / threads;
    if (b8 > 148 * 16) b8 = 148 * 16;
    silu_gate_bf16x8_kernel<<<(int)b8, threads, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, ffn,
                                                             total8, interleave);
  } else if (dtype == FG_F32)
    silu_gate_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)x, (float*)out, ffn, total, interleave);
  else if (dtype == FG_BF16)
    silu_gate_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)x, (__nv_bfloat16*)out, ffn, total, interleave);
  else
    FG_CHECK_ARG(false, "fg_silu_gate: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_silu_gate");
  return 0;
}
