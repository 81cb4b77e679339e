// Attention entry points for one head size, fixed at compile time by
// -DFG_HEAD_DIM=<multiple of 16>.  The builder compiles one library per head
// size a model needs.
#include "attention_simt.cuh"

#ifndef FG_HEAD_DIM
#error "compile with -DFG_HEAD_DIM=<head size>"
#endif
static_assert(FG_HEAD_DIM % 16 == 0 && FG_HEAD_DIM >= 16 && FG_HEAD_DIM <= 256,
              "head sizes are multiples of 16 from 16 to 256");

extern "C" int fg_attention_head_dim() { return FG_HEAD_DIM; }

// Tiling contract with the host: a tile holds tokens_per_tile = max(1, 16 / hpb)
// consecutive tokens of one request, where hpb = min(group, 16) heads share a
// block; grid.z covers the group in slices of hpb heads.
extern "C" int fg_attention_rows_per_block() { return fg_attn::ROWS; }

extern "C" int fg_attention_simt(const void* q, int q_stride, void* out, int out_stride, int dtype,
                                 const void* k_pages, const void* v_pages, const int* block_table,
                                 int table_width, int page_size, int n_pages, const int* pos,
                                 const int* tile_req, const int* tile_tok0, const int* tile_ntok,
                                 int n_tiles, int n_heads, int n_kv_heads, int head_dim, int window,
                                 float scale, int* status, cudaStream_t stream) {
  using namespace fg_attn;
  if (n_tiles == 0) return 0;
  FG_CHECK_ARG(head_dim == FG_HEAD_DIM, "fg_attention_simt: library built for head size %d, got %d",
               FG_HEAD_DIM, head_dim);
  FG_CHECK_ARG(n_kv_heads > 0 && n_heads % n_kv_heads == 0, "fg_attention_simt: %d heads over %d kv heads",
               n_heads, n_kv_heads);
  FG_CHECK_ARG(n_kv_heads <= 65535, "fg_attention_simt: too many kv heads");
  const int group = n_heads / n_kv_heads;
  const int hpb = group < ROWS ? group : ROWS;
  dim3 grid(n_tiles, n_kv_heads, (group + hpb - 1) / hpb);
  constexpr size_t smem = simt_smem_bytes<FG_HEAD_DIM>();
  cudaError_t e;
  if (dtype == FG_F32) {
    auto kern = attention_simt_kernel<float, FG_HEAD_DIM>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FG_CHECK_ARG(e == cudaSuccess, "fg_attention_simt: shared memory: %s", cudaGetErrorString(e));
    kern<<<grid, THREADS, smem, stream>>>((const float*)q, q_stride, (float*)out, out_stride,
                                          (const float*)k_pages, (const float*)v_pages, block_table,
                                          table_width, page_size, n_pages, pos, tile_req, tile_tok0,
                                          tile_ntok, n_kv_heads, group, hpb, window, scale, status);
  } else if (dtype == FG_BF16) {
    auto kern = attention_simt_kernel<__nv_bfloat16, FG_HEAD_DIM>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FG_CHECK_ARG(e == cudaSuccess, "fg_attention_simt: shared memory: %s", cudaGetErrorString(e));
    kern<<<grid, THREADS, smem, stream>>>(
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride,
        (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table, table_width,
        page_size, n_pages, pos, tile_req, tile_tok0, tile_ntok, n_kv_heads, group, hpb, window, scale,
        status);
  } else {
    FG_CHECK_ARG(false, "fg_attention_simt: bad dtype %d", dtype);
  }
  FG_CHECK_LAUNCH("fg_attention_simt");
  return 0;
}
