// Tensor maps (TMA descriptors) for the paged key/value pools.
//
// A pool is one dense tensor [layers, n_pages, kv_heads, page, head_dim]; the map
// describes it with a box of [box_rows, 64 elements] (128 bytes a row, swizzled
// by 128 bytes in shared memory), so one TMA instruction brings the rows of one
// page for one head and one half of the head size.
//
// The driver's encoder is looked up at run time, so the library does not link
// against libcuda.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace {
PFN_cuTensorMapEncodeTiled_v12000 encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}
}  // namespace

// out_map: 128 bytes on the host (64-byte aligned).  base: the pool on the device.
extern "C" int fg_make_kv_tensor_map(void* out_map, const void* base, int n_layers, int n_pages,
                                     int n_kv_heads, int page_size, int head_dim, int box_rows) {
  FG_CHECK_ARG(((uintptr_t)out_map & 63) == 0, "fg_make_kv_tensor_map: the map must be 64-byte aligned");
  FG_CHECK_ARG(head_dim % 64 == 0, "fg_make_kv_tensor_map: head size %d is not a multiple of 64", head_dim);
  FG_CHECK_ARG(box_rows > 0 && box_rows <= 256 && box_rows <= page_size,
               "fg_make_kv_tensor_map: bad box of %d rows for pages of %d", box_rows, page_size);
  auto encode = encoder();
  FG_CHECK_ARG(encode != nullptr, "fg_make_kv_tensor_map: the driver has no cuTensorMapEncodeTiled");
  const cuuint64_t dims[5] = {(cuuint64_t)head_dim, (cuuint64_t)page_size, (cuuint64_t)n_kv_heads,
                              (cuuint64_t)n_pages, (cuuint64_t)n_layers};
  const cuuint64_t row = (cuuint64_t)head_dim * 2;
  const cuuint64_t strides[4] = {row, row * page_size, row * page_size * n_kv_heads,
                                 row * page_size * n_kv_heads * n_pages};
  const cuuint32_t box[5] = {64, (cuuint32_t)box_rows, 1, 1, 1};
  const cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
  CUresult r = encode(reinterpret_cast<CUtensorMap*>(out_map), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5,
                      const_cast<void*>(base), dims, strides, box, elem_strides,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FG_CHECK_ARG(r == CUDA_SUCCESS, "fg_make_kv_tensor_map: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}
