// Shared helpers of the fastgen_b200 kernels (sm_100a).
//
// Conventions of the C interface:
//  * every entry point is `extern "C"`, takes raw device pointers and the
//    stream to launch on, and returns 0 or a negative error code after storing
//    a message that `fg_last_error()` returns;
//  * `dtype` arguments are FG_F32 or FG_BF16;
//  * no entry point allocates device memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FG_F32 0
#define FG_BF16 1

// Status bits that kernels OR into the engine's device status word instead of
// trapping; the host reads the word at its next synchronisation point.
#define FG_STATUS_BAD_PAGE 1      // a block-table entry was negative or too large
#define FG_STATUS_BAD_TOKEN 2     // a token id outside the vocabulary
#define FG_STATUS_WAIT_TIMEOUT 4  // a bounded wait on a barrier gave up
#define FG_STATUS_BAD_SPLITS 8    // decode attention was launched with too few splits

void fg_set_error(const char* fmt, ...);

#define FG_CHECK_ARG(cond, ...)  \
  do {                           \
    if (!(cond)) {               \
      fg_set_error(__VA_ARGS__); \
      return -1;                 \
    }                            \
  } while (0)

#define FG_CHECK_LAUNCH(name)                                         \
  do {                                                                \
    cudaError_t e_ = cudaGetLastError();                              \
    if (e_ != cudaSuccess) {                                          \
      fg_set_error("%s: launch failed: %s", name, cudaGetErrorString(e_)); \
      return -2;                                                      \
    }                                                                 \
  } while (0)

// ---------------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched through fg_launch_pdl may start
// while the kernel before it on the stream is still running: pdl_trigger() (first
// statement) lets the next kernel start early in turn, and pdl_wait() blocks until
// the previous kernel has completed and its writes are visible.  Before pdl_wait() a
// kernel may only touch what no earlier kernel of the step writes (weights, block
// tables, positions) and must not write global memory.  What an earlier kernel of the
// step wrote must not be read through a `const __restrict__` pointer: the compiler may
// move such a load above the wait (it takes the data for constant), and the kernel then
// sees the previous step's values.  Such data is read through plain pointers or with
// ld_global_16 / ld_global_4 below.  Both calls are no-ops for a kernel launched the
// ordinary way.  FG_NO_PDL=1 in the environment turns the attribute off.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// Loads that stay where they are written (never hoisted above a wait, never through the
// read-only cache).
__device__ __forceinline__ uint4 ld_global_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_global_4(const void* p) {
  uint32_t v;
  asm volatile("ld.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}

bool fg_pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t fg_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = fg_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Load element i of an array whose element type is only known at run time.
__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
  return dtype == FG_F32 ? static_cast<const float*>(p)[i]
                         : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ void store_from_f32(void* p, int dtype, size_t i, float v) {
  if (dtype == FG_F32)
    static_cast<float*>(p)[i] = v;
  else
    static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block; `scratch` holds one float per warp (<= 32).  The order of
// the additions depends only on the block size, never on the data's position.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}
