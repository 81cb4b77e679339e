// Attention entry points for one head size, fixed at compile time by
// -DFG_HEAD_DIM=<multiple of 16>.  The builder compiles one library per head
// size a model needs.
#include <string.h>

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

// ---------------------------------------------------------------------------------
// bfloat16 on the tensor cores
// ---------------------------------------------------------------------------------
#include "attention_mma.cuh"

extern "C" int fg_attention_prefill_rows() { return fg_mma::PREFILL_ROWS; }
extern "C" int fg_attention_decode_split() { return fg_mma::DECODE_SPLIT; }

// Floats of scratch that fg_attention_decode_bf16 needs.
// The scratch opens with FIRST_PAIR_INTS ints (for every request the number of (request,
// split) pairs before it, written by the persistent kernel for the merge of the splits), then
// the partials.  max_pairs bounds the pairs of a step (0: n_seqs * max_splits).
constexpr int FIRST_PAIR_INTS = 1024;

extern "C" long long fg_attention_decode_scratch_floats(int n_seqs, int max_splits, int n_heads, long long max_pairs) {
  const long long all = (long long)n_seqs * max_splits;
  if (max_pairs <= 0 || max_pairs > all) max_pairs = all;
  return FIRST_PAIR_INTS + max_pairs * n_heads * fg_mma::part_stride<FG_HEAD_DIM>();
}

[[maybe_unused]] static int sm_count() {
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return n_sms;
}

// Whether single tokens of these shapes go to the persistent kernel (whose launch does not
// depend on the requests' lengths and whose partials are numbered by pairs).
extern "C" int fg_attention_decode_is_persistent(int n_seqs, int n_heads, int n_kv_heads, int page_size);

// Prompt portions.  Tiles hold max(1, 64 / hpb) consecutive tokens of one request,
// hpb = min(group, 64); grid.z walks the group in slices of hpb heads.
extern "C" int fg_attention_prefill_bf16(const void* q, int q_stride, void* out, int out_stride,
                                         const void* k_pages, const void* v_pages, const int* block_table,
                                         int table_width, int page_size, int n_pages, const int* pos,
                                         const int* tile_req, const int* tile_tok0, const int* tile_ntok,
                                         int n_tiles, int n_heads, int n_kv_heads, int head_dim, int window,
                                         float scale, int* status, cudaStream_t stream) {
  using namespace fg_mma;
  if (n_tiles == 0) return 0;
  FG_CHECK_ARG(head_dim == FG_HEAD_DIM, "fg_attention_prefill_bf16: library built for head size %d, got %d",
               FG_HEAD_DIM, head_dim);
  FG_CHECK_ARG(n_kv_heads > 0 && n_heads % n_kv_heads == 0 && n_kv_heads <= 65535,
               "fg_attention_prefill_bf16: %d heads over %d kv heads", n_heads, n_kv_heads);
  FG_CHECK_ARG(q_stride % 8 == 0 && ((uintptr_t)q & 15) == 0,
               "fg_attention_prefill_bf16: queries must be 16-byte aligned with a row stride multiple of 8");
  const int group = n_heads / n_kv_heads;
  const int hpb = group < PREFILL_ROWS ? group : PREFILL_ROWS;
  dim3 grid(n_tiles, n_kv_heads, (group + hpb - 1) / hpb);
  constexpr size_t smem = prefill_smem_bytes<FG_HEAD_DIM>();
  auto kern = attention_prefill_kernel<FG_HEAD_DIM>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FG_CHECK_ARG(e == cudaSuccess, "fg_attention_prefill_bf16: shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  kern<<<grid, THREADS, smem, stream>>>(
      (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pages,
      (const __nv_bfloat16*)v_pages, block_table, table_width, page_size, n_pages, pos, tile_req, tile_tok0,
      tile_ntok, n_kv_heads, group, hpb, window, scale * 1.4426950408889634f, status);
  FG_CHECK_LAUNCH("fg_attention_prefill_bf16");
  return 0;
}

// Single tokens: sequence i of the list is token seq_tok[i] of request seq_req[i]
// (negative: padding).  max_splits >= ceil((largest position + 1) / 128).
extern "C" int fg_attention_decode_bf16(const void* q, int q_stride, void* out, int out_stride,
                                        const void* k_pages, const void* v_pages, const int* block_table,
                                        int table_width, int page_size, int n_pages, const int* pos,
                                        const int* seq_req, const int* seq_tok, int n_seqs, int n_heads,
                                        int n_kv_heads, int head_dim, int window, float scale, float* scratch,
                                        long long scratch_floats, int max_splits, int* status,
                                        cudaStream_t stream) {
  using namespace fg_mma;
  if (n_seqs == 0) return 0;
  FG_CHECK_ARG(head_dim == FG_HEAD_DIM, "fg_attention_decode_bf16: library built for head size %d, got %d",
               FG_HEAD_DIM, head_dim);
  FG_CHECK_ARG(n_kv_heads > 0 && n_heads % n_kv_heads == 0 && n_kv_heads <= 65535 && n_seqs <= 65535,
               "fg_attention_decode_bf16: %d heads over %d kv heads, %d sequences", n_heads, n_kv_heads, n_seqs);
  FG_CHECK_ARG(max_splits > 0, "fg_attention_decode_bf16: max_splits must be positive");
  FG_CHECK_ARG(scratch != nullptr &&
                   scratch_floats >= fg_attention_decode_scratch_floats(n_seqs, max_splits, n_heads, 0),
               "fg_attention_decode_bf16: scratch of %lld floats is too small (%lld needed)", scratch_floats,
               fg_attention_decode_scratch_floats(n_seqs, max_splits, n_heads, 0));
  FG_CHECK_ARG(q_stride % 8 == 0 && ((uintptr_t)q & 15) == 0,
               "fg_attention_decode_bf16: queries must be 16-byte aligned with a row stride multiple of 8");
  const int group = n_heads / n_kv_heads;
  constexpr size_t smem = decode_smem_bytes<FG_HEAD_DIM>();
  auto kern = attention_decode_kernel<FG_HEAD_DIM>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FG_CHECK_ARG(e == cudaSuccess, "fg_attention_decode_bf16: shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  const float scale_log2 = scale * 1.4426950408889634f;
  scratch += FIRST_PAIR_INTS;
  dim3 grid(max_splits, n_kv_heads, n_seqs);
  kern<<<grid, THREADS, smem, stream>>>((const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_pages,
                                        (const __nv_bfloat16*)v_pages, block_table, table_width, page_size,
                                        n_pages, pos, seq_req, seq_tok, n_heads, n_kv_heads, group, window,
                                        scale_log2, scratch, max_splits, status);
  FG_CHECK_LAUNCH("fg_attention_decode_bf16");
  dim3 cgrid(n_heads, n_seqs);
  attention_combine_kernel<FG_HEAD_DIM><<<cgrid, COMBINE_THREADS, 0, stream>>>(
      scratch, (__nv_bfloat16*)out, out_stride, pos, seq_req, seq_tok, n_heads, window, max_splits, nullptr, status);
  FG_CHECK_LAUNCH("fg_attention_combine");
  return 0;
}

// ---------------------------------------------------------------------------------
// single tokens with tiled TMA loads (head sizes that are multiples of 64)
// ---------------------------------------------------------------------------------
#if FG_HEAD_DIM % 64 == 0
#include "attention_tma.cuh"

extern "C" int fg_attention_decode_tma_supported() { return 1; }

// As fg_attention_decode_bf16, with the pools given as tensor maps (128 bytes each,
// on the host, made by fg_make_kv_tensor_map) and the layer's index in the pool.
extern "C" int fg_attention_decode_tma_bf16(const void* q, int q_stride, void* out, int out_stride,
                                            const void* k_map, const void* v_map, int layer,
                                            const int* block_table, int table_width, int page_size,
                                            int n_pages, const int* pos, const int* seq_req,
                                            const int* seq_tok, int n_seqs, int n_heads, int n_kv_heads,
                                            int head_dim, int window, float scale, float* scratch,
                                            long long scratch_floats, int max_splits, long long max_pairs,
                                            int* status, cudaStream_t stream) {
  using namespace fg_tma;
  if (n_seqs == 0) return 0;
  FG_CHECK_ARG(head_dim == FG_HEAD_DIM, "fg_attention_decode_tma_bf16: library built for head size %d, got %d",
               FG_HEAD_DIM, head_dim);
  FG_CHECK_ARG(n_kv_heads > 0 && n_heads % n_kv_heads == 0 && n_kv_heads <= 65535 && n_seqs <= 65535,
               "fg_attention_decode_tma_bf16: %d heads over %d kv heads, %d sequences", n_heads, n_kv_heads, n_seqs);
  const int group = n_heads / n_kv_heads;
  FG_CHECK_ARG(group <= DECODE_ROWS, "fg_attention_decode_tma_bf16: groups of %d heads are not supported", group);
  FG_CHECK_ARG(page_size >= 8 && (page_size & (page_size - 1)) == 0,
               "fg_attention_decode_tma_bf16: pages of %d slots are not supported", page_size);
  FG_CHECK_ARG(max_splits > 0 && scratch != nullptr, "fg_attention_decode_tma_bf16: no scratch");
  FG_CHECK_ARG(q_stride % 8 == 0 && ((uintptr_t)q & 15) == 0,
               "fg_attention_decode_tma_bf16: queries must be 16-byte aligned with a row stride multiple of 8");
  CUtensorMap km, vm;
  memcpy(&km, k_map, sizeof(CUtensorMap));
  memcpy(&vm, v_map, sizeof(CUtensorMap));
  int* first_pair = reinterpret_cast<int*>(scratch);
  float* partials = scratch + FIRST_PAIR_INTS;
  const int* combine_pairs = nullptr;
  if (fg_attention_decode_is_persistent(n_seqs, n_heads, n_kv_heads, page_size)) {
    // Blocks that stay on their SM (a producer warp ahead of four consumer warps) walk the
    // (request, split, kv head) items that exist; the launch does not depend on the lengths.
    const long long all = (long long)n_seqs * max_splits;
    if (max_pairs <= 0 || max_pairs > all) max_pairs = all;
    FG_CHECK_ARG(scratch_floats >= fg_attention_decode_scratch_floats(n_seqs, max_splits, n_heads, max_pairs),
                 "fg_attention_decode_tma_bf16: scratch of %lld floats is too small", scratch_floats);
    const size_t psmem = decode_persistent_smem_bytes<FG_HEAD_DIM>(group);
    auto pkern = attention_decode_persistent_kernel<FG_HEAD_DIM>;
    static size_t pattr_set = 0;
    if (pattr_set < psmem) {
      cudaError_t e = cudaFuncSetAttribute(pkern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)psmem);
      FG_CHECK_ARG(e == cudaSuccess, "fg_attention_decode_tma_bf16: shared memory: %s", cudaGetErrorString(e));
      pattr_set = psmem;
    }
    fg_launch_pdl(pkern, dim3(ps_blocks_per_sm<FG_HEAD_DIM>() * sm_count()), dim3(PS_THREADS), psmem, stream, km, vm,
                  layer, (const __nv_bfloat16*)q, q_stride, block_table, table_width, page_size, n_pages, pos,
                  seq_req, seq_tok, n_seqs, n_heads, n_kv_heads, group, window, scale * 1.4426950408889634f,
                  partials, first_pair, max_pairs, max_splits, status);
    combine_pairs = first_pair;
  } else {
    // one block per (request, kv head, split): larger groups of heads, very many requests
    FG_CHECK_ARG(scratch_floats >= fg_attention_decode_scratch_floats(n_seqs, max_splits, n_heads, 0),
                 "fg_attention_decode_tma_bf16: scratch of %lld floats is too small", scratch_floats);
    constexpr size_t smem = decode_tma_smem_bytes<FG_HEAD_DIM>();
    auto kern = attention_decode_tma_kernel<FG_HEAD_DIM>;
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      FG_CHECK_ARG(e == cudaSuccess, "fg_attention_decode_tma_bf16: shared memory: %s", cudaGetErrorString(e));
      attr_set = true;
    }
    dim3 grid(max_splits, n_kv_heads, n_seqs);
    fg_launch_pdl(kern, grid, dim3(THREADS), smem, stream, km, vm, layer, (const __nv_bfloat16*)q, q_stride,
                  block_table, table_width, page_size, n_pages, pos, seq_req, seq_tok, n_heads, group, window,
                  scale * 1.4426950408889634f, partials, max_splits, status);
  }
  FG_CHECK_LAUNCH("fg_attention_decode_tma_bf16");
  dim3 cgrid(n_heads, n_seqs);
  fg_launch_pdl(fg_mma::attention_combine_kernel<FG_HEAD_DIM>, cgrid, dim3(fg_mma::COMBINE_THREADS), 0, stream,
                (const float*)partials, (__nv_bfloat16*)out, out_stride, pos, seq_req, seq_tok, n_heads, window,
                max_splits, combine_pairs, status);
  FG_CHECK_LAUNCH("fg_attention_combine");
  return 0;
}

extern "C" int fg_attention_decode_is_persistent(int n_seqs, int n_heads, int n_kv_heads, int page_size) {
  (void)page_size;
  const int group = n_kv_heads > 0 ? n_heads / n_kv_heads : 0;
  return group >= 1 && group <= fg_tma::PS_MAX_GROUP && n_seqs <= fg_tma::PS_MAX_SEQS &&
         fg_tma::decode_persistent_smem_bytes<FG_HEAD_DIM>(group) <= 227 * 1024 - 4352 - 256;
}

extern "C" int fg_attention_prefill_tma_rows() { return fg_tma::PF_ROWS; }

// As fg_attention_prefill_bf16 with the pools given as tensor maps.  Tiles hold
// max(1, 128 / hpb) consecutive tokens of one request, hpb = min(group, 128).
extern "C" int fg_attention_prefill_tma_bf16(const void* q, int q_stride, void* out, int out_stride,
                                             const void* k_map, const void* v_map, int layer,
                                             const int* block_table, int table_width, int page_size,
                                             int n_pages, const int* pos, const int* tile_req,
                                             const int* tile_tok0, const int* tile_ntok, int n_tiles,
                                             int n_heads, int n_kv_heads, int head_dim, int window, float scale,
                                             int* status, cudaStream_t stream) {
  using namespace fg_tma;
  if (n_tiles == 0) return 0;
  FG_CHECK_ARG(head_dim == FG_HEAD_DIM, "fg_attention_prefill_tma_bf16: library built for head size %d, got %d",
               FG_HEAD_DIM, head_dim);
  FG_CHECK_ARG(n_kv_heads > 0 && n_heads % n_kv_heads == 0 && n_kv_heads <= 65535,
               "fg_attention_prefill_tma_bf16: %d heads over %d kv heads", n_heads, n_kv_heads);
  FG_CHECK_ARG(n_tiles <= 65535, "fg_attention_prefill_tma_bf16: %d tiles in one call (at most 65535)", n_tiles);
  FG_CHECK_ARG(page_size >= 8 && (page_size & (page_size - 1)) == 0,
               "fg_attention_prefill_tma_bf16: pages of %d slots are not supported", page_size);
  FG_CHECK_ARG(q_stride % 8 == 0 && ((uintptr_t)q & 15) == 0,
               "fg_attention_prefill_tma_bf16: queries must be 16-byte aligned with a row stride multiple of 8");
  const int group = n_heads / n_kv_heads;
  const int hpb = group < PF_ROWS ? group : PF_ROWS;
  CUtensorMap km, vm;
  memcpy(&km, k_map, sizeof(CUtensorMap));
  memcpy(&vm, v_map, sizeof(CUtensorMap));
  constexpr size_t smem = prefill_tma_smem_bytes<FG_HEAD_DIM>();
  auto kern = attention_prefill_tma_kernel<FG_HEAD_DIM>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FG_CHECK_ARG(e == cudaSuccess, "fg_attention_prefill_tma_bf16: shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  dim3 grid(n_kv_heads, n_tiles, (group + hpb - 1) / hpb);
  kern<<<grid, PF_THREADS, smem, stream>>>(km, vm, layer, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out,
                                           out_stride, block_table, table_width, page_size, n_pages, pos,
                                           tile_req, tile_tok0, tile_ntok, n_tiles, group, hpb, window,
                                           scale * 1.4426950408889634f, status);
  FG_CHECK_LAUNCH("fg_attention_prefill_tma_bf16");
  return 0;
}

#if FG_HEAD_DIM == 64 || FG_HEAD_DIM == 128
#include "attention_tcgen05.cuh"

extern "C" int fg_attention_prefill_tc5_supported() { return 1; }

// Prompt portions on tcgen05 / TMEM.  Arguments and tiling (128 rows an item) as for
// fg_attention_prefill_tma_bf16, plus `work_counter`: one unsigned int on the device that is
// zero between launches (the kernel leaves it so) and is not shared by launches that can
// run at the same time; the tensor maps must have boxes of min(page, 64) rows.
//
// A launch of fewer items than resident blocks works on its long items in several parts (see
// the kernel).  That needs, for every (item, part), fg_tc5::ROWS * (head size + 2) floats of
// `split_scratch`, and two ints of `split_flags` for every item, zero before the first launch
// (the kernel leaves the counter so).
// fg_attention_prefill_tc5_split_slots says how many (item, part) pairs a launch wants room
// for, or 0 if it would not split: too many items, or, where the host knows the most keys an
// item reads (`max_keys`, else -1), too few keys for a second part.  With null pointers or
// less room (`split_slots`) the launch does not split either.
//
// `real_tiles` (may be null) points at the number of tiles at the end of the list that are
// real, for a launch that is captured in a graph whose list has padding in front
// (`nominal_tiles` in fg_attention_prefill_tc5_split_slots: the tiles of a step of the graph's
// token count that holds prompt tokens only; 0 without such a list): the kernel then hands out
// the real tiles only and chooses the number of parts itself, which asks for room for one pair
// a block.
static long long tc5_items(int n_tiles, int n_heads, int n_kv_heads) {
  const int group = n_heads / n_kv_heads;
  const int hpb = group < fg_tc5::ROWS ? group : fg_tc5::ROWS;
  return (long long)n_tiles * n_kv_heads * ((group + hpb - 1) / hpb);
}

static int tc5_parts(long long items) {
  const long long parts = 2ll * sm_count() / (items > 0 ? items : 1);
  return (int)(parts < 1 ? 1 : parts > fg_tc5::MAX_PARTS ? fg_tc5::MAX_PARTS : parts);
}

extern "C" int fg_attention_prefill_tc5_split_slots(int n_tiles, int n_heads, int n_kv_heads, int max_keys,
                                                    int nominal_tiles) {
  if (n_tiles <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return 0;
  // an item is split from 2 * SPLIT_MIN_TILES key tiles on
  if (max_keys >= 0 && max_keys <= (2 * fg_tc5::SPLIT_MIN_TILES - 1) * fg_tc5::KEYS) return 0;
  // (with padding in the list: the instantiation that can split, unless a step whose tokens
  // are all prompt tokens, `nominal_tiles` tiles, would fill the launch's blocks anyway)
  if (nominal_tiles > 0) return tc5_items(nominal_tiles, n_heads, n_kv_heads) < 2ll * sm_count() ? 2 * sm_count() : 0;
  const long long items = tc5_items(n_tiles, n_heads, n_kv_heads);
  const int parts = tc5_parts(items);
  return parts > 1 ? (int)(items * parts) : 0;
}

extern "C" int fg_attention_prefill_tc5_bf16(const void* q, int q_stride, void* out, int out_stride,
                                             const void* k_map, const void* v_map, int layer,
                                             const int* block_table, int table_width, int page_size,
                                             int n_pages, const int* pos, const int* tile_req,
                                             const int* tile_tok0, const int* tile_ntok, int n_tiles,
                                             int n_heads, int n_kv_heads, int head_dim, int window, float scale,
                                             unsigned int* work_counter, float* split_scratch, int* split_flags,
                                             int split_slots, int max_keys, const int* real_tiles, int nominal_tiles,
                                             int* status, cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  FG_CHECK_ARG(work_counter != nullptr, "fg_attention_prefill_tc5_bf16: no work counter");
  FG_CHECK_ARG(head_dim == FG_HEAD_DIM, "fg_attention_prefill_tc5_bf16: library built for head size %d, got %d",
               FG_HEAD_DIM, head_dim);
  FG_CHECK_ARG(n_kv_heads > 0 && n_heads % n_kv_heads == 0 && n_kv_heads <= 65535,
               "fg_attention_prefill_tc5_bf16: %d heads over %d kv heads", n_heads, n_kv_heads);
  FG_CHECK_ARG(page_size >= 8 && (page_size & (page_size - 1)) == 0,
               "fg_attention_prefill_tc5_bf16: pages of %d slots are not supported", page_size);
  FG_CHECK_ARG(q_stride % 8 == 0 && ((uintptr_t)q & 15) == 0 && out_stride % 8 == 0 && ((uintptr_t)out & 15) == 0,
               "fg_attention_prefill_tc5_bf16: queries and outputs must be 16-byte aligned with strides multiple of 8");
  const int group = n_heads / n_kv_heads;
  const int hpb = group < fg_tc5::ROWS ? group : fg_tc5::ROWS;
  CUtensorMap km, vm;
  memcpy(&km, k_map, sizeof(CUtensorMap));
  memcpy(&vm, v_map, sizeof(CUtensorMap));
  constexpr size_t smem = fg_tc5::smem_bytes<FG_HEAD_DIM>();
  auto kern_whole = fg_tc5::attention_prefill_tc5_kernel<FG_HEAD_DIM, false>;
  auto kern_parts = fg_tc5::attention_prefill_tc5_kernel<FG_HEAD_DIM, true>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern_whole, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kern_parts, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FG_CHECK_ARG(e == cudaSuccess, "fg_attention_prefill_tc5_bf16: shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  // two blocks an SM take the (tile, kv head, slice of the group) items from a counter
  const long long items = tc5_items(n_tiles, n_heads, n_kv_heads);
  FG_CHECK_ARG(items < (1ll << 30), "fg_attention_prefill_tc5_bf16: %lld work items in one call", items);
  const int want = fg_attention_prefill_tc5_split_slots(n_tiles, n_heads, n_kv_heads, max_keys,
                                                        real_tiles ? (nominal_tiles > 0 ? nominal_tiles : 1) : 0);
  const long long resident = 2ll * sm_count();
  const bool split = want > 0 && split_scratch && split_flags && want <= split_slots;
  const int parts = split && !real_tiles ? tc5_parts(items) : 1;
  const long long total = items * parts;
  // (a launch that chooses its parts itself has all its blocks)
  const int grid = (int)(split && real_tiles ? resident : total < resident ? total : resident);
  (split ? kern_parts : kern_whole)<<<grid, fg_tc5::THREADS, smem, stream>>>(
      km, vm, layer, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, block_table, table_width,
      page_size, n_pages, pos, tile_req, tile_tok0, tile_ntok, n_tiles, n_kv_heads, group, hpb, window,
      scale * 1.4426950408889634f, work_counter, parts, split_scratch, split_flags, split_slots, real_tiles, status);
  FG_CHECK_LAUNCH("fg_attention_prefill_tc5_bf16");
  return 0;
}
#else
extern "C" int fg_attention_prefill_tc5_supported() { return 0; }
extern "C" int fg_attention_prefill_tc5_split_slots(int, int, int, int, int) { return 0; }
#endif
#else
extern "C" int fg_attention_decode_tma_supported() { return 0; }
extern "C" int fg_attention_prefill_tc5_supported() { return 0; }
extern "C" int fg_attention_prefill_tc5_split_slots(int, int, int, int, int) { return 0; }
extern "C" int fg_attention_decode_is_persistent(int, int, int, int) { return 0; }
#endif
