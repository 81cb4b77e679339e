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

// Vectorised variant for dim % 4 == 0 and dim <= 1024 * ITEMS: a thread keeps its
// ITEMS x 4 elements in registers between the reduction and the scaling, so the
// row is read once.  Same arithmetic, same result type; the order of the row's
// sum again depends only on dim.
template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <typename T>
__device__ __forceinline__ void store4(T* p, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* p, float4 v) {
  *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}
__device__ __forceinline__ float4 load4_any(const void* p, int dtype, int i) {
  return dtype == FG_F32 ? load4<float>(static_cast<const float*>(p) + i)
                         : load4<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p) + i);
}

constexpr int VEC_THREADS = 256;

template <typename TH, typename TD, typename TO, int ITEMS>
__global__ void __launch_bounds__(VEC_THREADS)
rmsnorm_vec_kernel(TH* h, const TD* delta, const void* __restrict__ w, int w_dtype, TO* __restrict__ out,
                   const int* __restrict__ rows, int dim, float eps) {
  // h and delta come from earlier kernels of the step: no __restrict__, so that their
  // loads stay below the wait
  __shared__ float scratch[32];
  pdl_trigger();
  // the norm's weight and the row indices do not depend on the kernels before this one: they are
  // on their way while those finish, instead of being a second round trip behind the reduction
  float4 ww[ITEMS];
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    const int d = (it * VEC_THREADS + threadIdx.x) * 4;
    ww[it] = (out != nullptr && d < dim) ? load4_any(w, w_dtype, d) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const size_t base = (size_t)(rows ? rows[blockIdx.x] : blockIdx.x) * dim;
  const size_t obase = (size_t)blockIdx.x * dim;
  const bool store_h = delta != nullptr && rows == nullptr;
  pdl_wait();
  float4 v[ITEMS];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    const int d = (it * VEC_THREADS + threadIdx.x) * 4;
    v[it] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (d < dim) {
      v[it] = load4<TH>(h + base + d);
      if (delta != nullptr) {
        const float4 e = load4<TD>(delta + base + d);
        v[it].x += e.x; v[it].y += e.y; v[it].z += e.z; v[it].w += e.w;
        // the stored sum is what is normed
        v[it].x = to_f32<TH>(from_f32<TH>(v[it].x)); v[it].y = to_f32<TH>(from_f32<TH>(v[it].y));
        v[it].z = to_f32<TH>(from_f32<TH>(v[it].z)); v[it].w = to_f32<TH>(from_f32<TH>(v[it].w));
        if (store_h) store4<TH>(h + base + d, v[it]);
      }
      ss += v[it].x * v[it].x + v[it].y * v[it].y + v[it].z * v[it].z + v[it].w * v[it].w;
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)dim + eps);
  if (out == nullptr) return;
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    const int d = (it * VEC_THREADS + threadIdx.x) * 4;
    if (d < dim)
      store4<TO>(out + obase + d, make_float4(v[it].x * rstd * ww[it].x, v[it].y * rstd * ww[it].y,
                                              v[it].z * rstd * ww[it].z, v[it].w * rstd * ww[it].w));
  }
}

template <typename TH, typename TD, typename TO>
static void launch_vec(int items, int n_rows, cudaStream_t stream, TH* h, const TD* delta, const void* w,
                       int w_dtype, TO* out, const int* rows, int dim, float eps) {
  switch (items) {
    case 1: fg_launch_pdl(rmsnorm_vec_kernel<TH, TD, TO, 1>, dim3(n_rows), dim3(VEC_THREADS), 0, stream, h, delta, w, w_dtype, out, rows, dim, eps); break;
    case 2: fg_launch_pdl(rmsnorm_vec_kernel<TH, TD, TO, 2>, dim3(n_rows), dim3(VEC_THREADS), 0, stream, h, delta, w, w_dtype, out, rows, dim, eps); break;
    case 4: fg_launch_pdl(rmsnorm_vec_kernel<TH, TD, TO, 4>, dim3(n_rows), dim3(VEC_THREADS), 0, stream, h, delta, w, w_dtype, out, rows, dim, eps); break;
    default: fg_launch_pdl(rmsnorm_vec_kernel<TH, TD, TO, 8>, dim3(n_rows), dim3(VEC_THREADS), 0, stream, h, delta, w, w_dtype, out, rows, dim, eps); break;
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
  const auto aligned = [](const void* p) { return p == nullptr || ((uintptr_t)p & 15) == 0; };
  const bool vec = dim % 4 == 0 && dim <= VEC_THREADS * 4 * 8 && aligned(h) && aligned(delta) && aligned(w) &&
                   aligned(out);
  int items = 1;
  while (items * VEC_THREADS * 4 < dim) items *= 2;
#define LAUNCH(TH, TD, TO)                                                                       \
  do {                                                                                           \
    if (vec)                                                                                     \
      launch_vec<TH, TD, TO>(items, n_rows, stream, (TH*)h, (const TD*)delta, w, w_dtype, (TO*)out, \
                             rows, dim, eps);                                                    \
    else                                                                                         \
      rmsnorm_kernel<TH, TD, TO><<<n_rows, threads, 0, stream>>>((TH*)h, (const TD*)delta, w,    \
                                                                 w_dtype, (TO*)out, rows, dim, eps); \
  } while (0)
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
