// RMSNorm, optionally fused with the residual sum that precedes it:
//   if delta: h[t,:] += delta[t,:]      (float32 sum, h stored back)
//   out[t,:] = h[t,:] * rsqrt(mean(h^2) + eps) * w[:]
// Formula of fastgen/kernels/rmsnorm.py:33-60 (float32 throughout, the product
// rounded once to the output type); the fused sum replaces h.add_ of
// fastgen/forward.py:472,499.  One block per row; the order of the row's
// reduction depends only on dim and the block size.
#include "common.cuh"

template <typename TH, typename TD, typename TO>
__global__ void rmsnorm_kernel(TH* __restrict__ h, const TD* __restrict__ delta,
                               const void* __restrict__ w, int w_dtype, TO* __restrict__ out,
                               const int* __restrict__ rows, int dim, float eps) {
  __shared__ float scratch[32];
  // With `rows`, output row i is computed from input row rows[i] and the sum
  // is not stored back (the same input row may be gathered twice).
  const size_t base = (size_t)(rows ? rows[blockIdx.x] : blockIdx.x) * dim;
  const size_t obase = (size_t)blockIdx.x * dim;
  const bool store_h = delta != nullptr && rows == nullptr;
  float ss = 0.f;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float v = to_f32<TH>(h[base + d]);
    if (delta != nullptr) {
      v += to_f32<TD>(delta[base + d]);
      v = to_f32<TH>(from_f32<TH>(v));
      if (store_h) h[base + d] = from_f32<TH>(v);
    }
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)dim + eps);
  if (out == nullptr) return;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    // when the sum was stored, each thread re-reads exactly what it wrote
    float v = to_f32<TH>(h[base + d]);
    if (delta != nullptr && !store_h) v = to_f32<TH>(from_f32<TH>(v + to_f32<TD>(delta[base + d])));
    out[obase + d] = from_f32<TO>(v * rstd * load_as_f32(w, w_dtype, d));
  }
}

// h: [T, dim] (h_dtype), delta: [T, dim] or null, w: [dim], out: [n_rows, dim] or
// null (null: only the sum is done).  rows: null, or n_rows indices into h and
// delta to gather (then h is left untouched).
extern "C" int fg_rmsnorm(void* h, int h_dtype, const void* delta, int delta_dtype, const void* w,
                          int w_dtype, void* out, int out_dtype, const int* rows, int n_rows, int dim,
                          float eps, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  FG_CHECK_ARG(dim > 0, "fg_rmsnorm: bad dim %d", dim);
  const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
#define LAUNCH(TH, TD, TO)                                                       \
  rmsnorm_kernel<TH, TD, TO><<<n_rows, threads, 0, stream>>>(                    \
      (TH*)h, (const TD*)delta, w, w_dtype, (TO*)out, rows, dim, eps)
  const int key = h_dtype * 4 + (delta ? delta_dtype : h_dtype) * 2 + out_dtype;
  switch (key) {
    case 0: LAUNCH(float, float, float); break;
    case 1: LAUNCH(float, float, __nv_bfloat16); break;
    case 2: LAUNCH(float, __nv_bfloat16, float); break;
    case 3: LAUNCH(float, __nv_bfloat16, __nv_bfloat16); break;
    case 4: LAUNCH(__nv_bfloat16, float, float); break;
    case 5: LAUNCH(__nv_bfloat16, float, __nv_bfloat16); break;
    case 6: LAUNCH(__nv_bfloat16, __nv_bfloat16, float); break;
    case 7: LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16); break;
    default: FG_CHECK_ARG(false, "fg_rmsnorm: bad dtypes");
  }
#undef LAUNCH
  FG_CHECK_LAUNCH("fg_rmsnorm");
  return 0;
}
