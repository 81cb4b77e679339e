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

// An adjacent pair as one access (4 bytes of bfloat16, 8 of float32) when the
// launch found every pair aligned, else as two.
template <typename T>
__device__ __forceinline__ float2 load_pair(const T* p, bool vec);
template <>
__device__ __forceinline__ float2 load_pair<float>(const float* p, bool vec) {
  if (vec) return *reinterpret_cast<const float2*>(p);
  return make_float2(p[0], p[1]);
}
template <>
__device__ __forceinline__ float2 load_pair<__nv_bfloat16>(const __nv_bfloat16* p, bool vec) {
  if (vec) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  return make_float2(__bfloat162float(p[0]), __bfloat162float(p[1]));
}
template <typename T>
__device__ __forceinline__ void store_pair(T* p, float2 v, bool vec);
template <>
__device__ __forceinline__ void store_pair<float>(float* p, float2 v, bool vec) {
  if (vec) *reinterpret_cast<float2*>(p) = v;
  else { p[0] = v.x; p[1] = v.y; }
}
template <>
__device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16* p, float2 v, bool vec) {
  if (vec) *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y);
  else { p[0] = __float2bfloat16_rn(v.x); p[1] = __float2bfloat16_rn(v.y); }
}

// One thread per adjacent pair: blockIdx.x is the token, blockIdx.y a slab of
// 128 pairs out of [query pairs | key pairs | value pairs].
template <typename T>
__global__ void __launch_bounds__(ROPE_THREADS)
rope_kv_kernel(T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride,
               const T* __restrict__ v, int v_stride, const int* __restrict__ pos,
               const int* __restrict__ req, const float* __restrict__ freqs, T* __restrict__ k_pages,
               T* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
               int page_size, int n_pages, int n_heads, int n_kv_heads, int head_dim, int* status,
               bool vec, int items_per_thread) {
  const int t = blockIdx.x;
  const int r = req[t];
  if (r < 0) return;
  const int half = head_dim >> 1;
  const int n_q = n_heads * half, n_kv = (k != nullptr) ? n_kv_heads * half : 0;
  const int p = pos[t];
  for (int it = 0; it < items_per_thread; ++it) {
  const int item = (blockIdx.y * items_per_thread + it) * ROPE_THREADS + threadIdx.x;
  if (item >= n_q + 2 * n_kv) return;
  if (item < n_q) {
    const int j = item % half;
    T* x = q + (size_t)t * q_stride + (item / half) * head_dim + 2 * j;
    const float2 v = load_pair<T>(x, vec);
    float s = 0.f, c = 1.f;
    if (freqs != nullptr) sincosf((float)p * freqs[j], &s, &c);
    store_pair<T>(x, make_float2(v.x * c - v.y * s, v.y * c + v.x * s), vec);
    continue;
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
    if (vec) {
      // a plain copy: move the pair's bits
      if (sizeof(T) == 2) *reinterpret_cast<uint32_t*>(v_pages + dst) = *reinterpret_cast<const uint32_t*>(x);
      else *reinterpret_cast<uint2*>(v_pages + dst) = *reinterpret_cast<const uint2*>(x);
    } else {
      v_pages[dst] = x[0];
      v_pages[dst + 1] = x[1];
    }
  } else {
    const T* x = k + (size_t)t * k_stride + g * head_dim + 2 * j;
    const float2 kv = load_pair<T>(x, vec);
    float s = 0.f, c = 1.f;
    if (freqs != nullptr) sincosf((float)p * freqs[j], &s, &c);
    store_pair<T>(k_pages + dst, make_float2(kv.x * c - kv.y * s, kv.y * c + kv.x * s), vec);
  }
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
  // few tokens: one pair a thread, many small blocks; many tokens: several pairs a
  // thread, so that the number of blocks stays in the low thousands
  int ipt = 1;
  while (ipt < 16 && (long long)n_tokens * ((items + ROPE_THREADS * ipt - 1) / (ROPE_THREADS * ipt)) > 4096) ipt *= 2;
  const dim3 grid(n_tokens, (items + ROPE_THREADS * ipt - 1) / (ROPE_THREADS * ipt));
  const int threads = ROPE_THREADS;
  FG_CHECK_ARG(grid.y <= 65535, "fg_rope_kv_write: too many heads");
  const size_t pair = dtype == FG_F32 ? 8 : 4;
  const auto ok = [&](const void* p, int stride) { return p == nullptr || (((uintptr_t)p % pair) == 0 && stride % 2 == 0); };
  const bool vec = ok(q, q_stride) && ok(k, k_stride) && ok(v, v_stride) && ok(k_pages, 0) && ok(v_pages, 0);
  if (dtype == FG_F32)
    rope_kv_kernel<float><<<grid, threads, 0, stream>>>(
        (float*)q, q_stride, (const float*)k, k_stride, (const float*)v, v_stride, pos, req, freqs,
        (float*)k_pages, (float*)v_pages, block_table, table_width, page_size, n_pages, n_heads,
        n_kv_heads, head_dim, status, vec, ipt);
  else if (dtype == FG_BF16)
    rope_kv_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        (__nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v,
        v_stride, pos, req, freqs, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, block_table,
        table_width, page_size, n_pages, n_heads, n_kv_heads, head_dim, status, vec, ipt);
  else
    FG_CHECK_ARG(false, "fg_rope_kv_write: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_rope_kv_write");
  return 0;
}
