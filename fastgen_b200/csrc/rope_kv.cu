// Rotary position encoding of queries and keys fused with the write of keys
// and values into their cache pages.
//
// Replaces apply_rope x2 (fastgen/kernels/rope.py:57-89) and paged_memcpy x2
// (fastgen/kernels/paged_memcpy.py:57-76) of fastgen/forward.py:449-460.
//   angle = float(pos) * freqs[j]                      (float32 product)
//   x[2j]   = re * cos(angle) - im * sin(angle)
//   x[2j+1] = im * cos(angle) + re * sin(angle)        (precise sinf/cosf)
// Queries are rotated in place.  Keys are rotated and stored, values copied, to
//   slot = block_table[req, pos / page] * page + pos % page
// of a pool laid out [n_pages, n_kv_heads, page, head_dim], so that the
// [page, head_dim] tile of one head is contiguous.
// Tokens whose request index is negative are padding: nothing is written.
#include "common.cuh"

constexpr int ROPE_THREADS = 128;

// One thread per adjacent pair: blockIdx.x is the token, blockIdx.y a slab of
// 128 pairs out of [query pairs | key pairs | value pairs].
template <typename T>
__global__ void __launch_bounds__(ROPE_THREADS)
rope_kv_kernel(T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride,
               const T* __restrict__ v, int v_stride, const int* __restrict__ pos,
               const int* __restrict__ req, const float* __restrict__ freqs, T* __restrict__ k_pages,
               T* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
               int page_size, int n_pages, int n_heads, int n_kv_heads, int head_dim, int* status) {
  const int t = blockIdx.x;
  const int r = req[t];
  if (r < 0) return;
  const int half = head_dim >> 1;
  const int n_q = n_heads * half, n_kv = (k != nullptr) ? n_kv_heads * half : 0;
  const int item = blockIdx.y * ROPE_THREADS + threadIdx.x;
  if (item >= n_q + 2 * n_kv) return;
  const int p = pos[t];
  if (item < n_q) {
    const int j = item % half;
    T* x = q + (size_t)t * q_stride + (item / half) * head_dim + 2 * j;
    const float re = to_f32<T>(x[0]), im = to_f32<T>(x[1]);
    float s = 0.f, c = 1.f;
    if (freqs != nullptr) sincosf((float)p * freqs[j], &s, &c);
    x[0] = from_f32<T>(re * c - im * s);
    x[1] = from_f32<T>(im * c + re * s);
    return;
  }
  const bool is_v = item >= n_q + n_kv;
  const int kv_item = item - n_q - (is_v ? n_kv : 0);
  const int g = kv_item / half, j = kv_item - g * half;
  const int logical = p / page_size;
  const int page = (logical < table_width) ? block_table[(size_t)r * table_width + logical] : -1;
  if (page < 0 || page >= n_pages) {
    if (status) atomicOr(status, FG_STATUS_BAD_PAGE);
    return;
  }
  const size_t dst = (((size_t)page * n_kv_heads + g) * page_size + (p - logical * page_size)) * head_dim + 2 * j;
  if (is_v) {
    const T* x = v + (size_t)t * v_stride + g * head_dim + 2 * j;
    v_pages[dst] = x[0];
    v_pages[dst + 1] = x[1];
  } else {
    const T* x = k + (size_t)t * k_stride + g * head_dim + 2 * j;
    const float re = to_f32<T>(x[0]), im = to_f32<T>(x[1]);
    float s = 0.f, c = 1.f;
    if (freqs != nullptr) sincosf((float)p * freqs[j], &s, &c);
    k_pages[dst] = from_f32<T>(re * c - im * s);
    k_pages[dst + 1] = from_f32<T>(im * c + re * s);
  }
}

// q: [T, n_heads*head_dim] with row stride q_stride (elements), rotated in place.
// k, v: [T, n_kv_heads*head_dim] with their strides, or both null (queries only).
// freqs: float32 [head_dim/2] or null for no rotation.
extern "C" int fg_rope_kv_write(void* q, int q_stride, const void* k, int k_stride, const void* v,
                                int v_stride, int dtype, const int* pos, const int* req,
                                const float* freqs, void* k_pages, void* v_pages,
                                const int* block_table, int table_width, int page_size, int n_pages,
                                int n_tokens, int n_heads, int n_kv_heads, int head_dim, int* status,
                                cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  FG_CHECK_ARG(head_dim > 0 && head_dim % 2 == 0, "fg_rope_kv_write: head_dim %d must be even", head_dim);
  FG_CHECK_ARG((k == nullptr) == (v == nullptr), "fg_rope_kv_write: k and v must both be given or both null");
  FG_CHECK_ARG(k == nullptr || (k_pages && v_pages && block_table && page_size > 0),
               "fg_rope_kv_write: cache arguments missing");
  const int items = (n_heads + (k ? 2 * n_kv_heads : 0)) * head_dim / 2;
  const dim3 grid(n_tokens, (items + ROPE_THREADS - 1) / ROPE_THREADS);
  const int threads = ROPE_THREADS;
  FG_CHECK_ARG(grid.y <= 65535, "fg_rope_kv_write: too many heads");
  if (dtype == FG_F32)
    rope_kv_kernel<float><<<grid, threads, 0, stream>>>(
        (float*)q, q_stride, (const float*)k, k_stride, (const float*)v, v_stride, pos, req, freqs,
        (float*)k_pages, (float*)v_pages, block_table, table_width, page_size, n_pages, n_heads,
        n_kv_heads, head_dim, status);
  else if (dtype == FG_BF16)
    rope_kv_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        (__nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v,
        v_stride, pos, req, freqs, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, block_table,
        table_width, page_size, n_pages, n_heads, n_kv_heads, head_dim, status);
  else
    FG_CHECK_ARG(false, "fg_rope_kv_write: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_rope_kv_write");
  return 0;
}
