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

// bfloat16 rows whose width is a multiple of 8: eight elements (16 bytes) a thread.
// blockIdx.x walks a row's 16-byte pieces, blockIdx.y (and a stride loop) the rows, so no
// index needs a division; two rows are in flight a thread.
__global__ void __launch_bounds__(256)
silu_gate_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int ffn, int n_rows,
                        int interleave) {
  const int piece = blockIdx.x * blockDim.x + threadIdx.x;
  if (piece >= ffn / 8) return;
  const int f = piece * 8;
  const int g_off = interleave ? 2 * f : f, u_off = interleave ? 2 * f + 8 : ffn + f;
  auto gate = [](uint4 g4, uint4 u4) {
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
      // float32 throughout; the special-function unit's exponential and reciprocal (a few
      // units in the last place of float32, far below the bfloat16 rounding that follows):
      // with expf() and an IEEE division the kernel was bound by instruction issue
      o2[k] = __floats2bfloat162_rn(__fdividef(g.x, 1.f + __expf(-g.x)) * u.x,
                                    __fdividef(g.y, 1.f + __expf(-g.y)) * u.y);
    }
    return o4;
  };
  int t = blockIdx.y;
  for (; t + (int)gridDim.y < n_rows; t += 2 * gridDim.y) {
    const __nv_bfloat16* r0 = x + (size_t)t * 2 * ffn;
    const __nv_bfloat16* r1 = x + (size_t)(t + gridDim.y) * 2 * ffn;
    const uint4 g0 = *reinterpret_cast<const uint4*>(r0 + g_off), u0 = *reinterpret_cast<const uint4*>(r0 + u_off);
    const uint4 g1 = *reinterpret_cast<const uint4*>(r1 + g_off), u1 = *reinterpret_cast<const uint4*>(r1 + u_off);
    *reinterpret_cast<uint4*>(out + (size_t)t * ffn + f) = gate(g0, u0);
    *reinterpret_cast<uint4*>(out + (size_t)(t + gridDim.y) * ffn + f) = gate(g1, u1);
  }
  if (t < n_rows) {
    const __nv_bfloat16* r0 = x + (size_t)t * 2 * ffn;
    *reinterpret_cast<uint4*>(out + (size_t)t * ffn + f) =
        gate(*reinterpret_cast<const uint4*>(r0 + g_off), *reinterpret_cast<const uint4*>(r0 + u_off));
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
    const int bx = (ffn / 8 + threads - 1) / threads;
    int by = n_rows < 65535 ? n_rows : 65535;
    while (by > 1 && (long long)bx * by > 148 * 32) by = (by + 1) / 2;  // rows beyond the grid: the stride loop
    silu_gate_bf16x8_kernel<<<dim3(bx, by), threads, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, ffn,
                                                                  n_rows, interleave);
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
