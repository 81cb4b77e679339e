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

// A thread owns one pair index j of one token: it computes sin and cos of the
// token's angle for j once and walks the heads (queries, then keys, then values)
// that its block is given: blockIdx.x is the token, blockIdx.y a slice of the
// heads (few tokens get more slices, so that the GPU is still filled).
template <typename T>
__global__ void __launch_bounds__(ROPE_THREADS)
rope_kv_kernel(T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride,
               const T* __restrict__ v, int v_stride, const int* __restrict__ pos,
               const int* __restrict__ req, const float* __restrict__ freqs, T* __restrict__ k_pages,
               T* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
               int page_size, int n_pages, int n_heads, int n_kv_heads, int head_dim, int* status,
               bool vec, int heads_per_block) {
  const int t = blockIdx.x;
  const int r = req[t];
  if (r < 0) return;
  const int half = head_dim >> 1;
  const int lanes = ROPE_THREADS / half > 0 ? ROPE_THREADS / half : 1;  // heads walked side by side
  const int j = threadIdx.x % half, lane_head = threadIdx.x / half;
  if (lane_head >= lanes) return;
  const int p = pos[t];
  const int n_kv = (k != nullptr) ? n_kv_heads : 0;
  const int total = n_heads + 2 * n_kv;  // heads in the order q..., k..., v...
  const int h_end = min(total, (int)(blockIdx.y + 1) * heads_per_block);
  float s = 0.f, c = 1.f;
  if (freqs != nullptr) sincosf((float)p * freqs[j], &s, &c);
  size_t slot = 0;
  bool have_slot = false;
  for (int h = blockIdx.y * heads_per_block + lane_head; h < h_end; h += lanes) {
    if (h < n_heads) {
      T* x = q + (size_t)t * q_stride + h * head_dim + 2 * j;
      const float2 val = load_pair<T>(x, vec);
      store_pair<T>(x, make_float2(val.x * c - val.y * s, val.y * c + val.x * s), vec);
      continue;
    }
    if (!have_slot) {
      const int logical = p / page_size;
      const int page = (logical < table_width) ? block_table[(size_t)r * table_width + logical] : -1;
      if (page < 0 || page >= n_pages) {
        if (status) atomicOr(status, FG_STATUS_BAD_PAGE);
        return;
      }
      slot = (size_t)page * n_kv_heads * page_size + (p - logical * page_size);
      have_slot = true;
    }
    const bool is_v = h >= n_heads + n_kv;
    const int g = h - n_heads - (is_v ? n_kv : 0);
    const size_t dst = (slot + (size_t)g * page_size) * head_dim + 2 * j;
    if (is_v) {
      const T* x = v + (size_t)t * v_stride + g * head_dim + 2 * j;
      store_pair<T>(v_pages + dst, load_pair<T>(x, vec), vec);
    } else {
      const T* x = k + (size_t)t * k_stride + g * head_dim + 2 * j;
      const float2 val = load_pair<T>(x, vec);
      store_pair<T>(k_pages + dst, make_float2(val.x * c - val.y * s, val.y * c + val.x * s), vec);
    }
  }
}

// bfloat16 with 16-byte accesses: a thread owns four adjacent pairs (8 elements) of one
// token, computes their four angles once and walks the heads, several heads in flight.
// Needs head_dim % 8 == 0 and 16-byte aligned rows.
constexpr int ROPE_UNROLL = 4;

__global__ void __launch_bounds__(ROPE_THREADS)
rope_kv_bf16x8_kernel(__nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k, int k_stride,
                      const __nv_bfloat16* __restrict__ v, int v_stride, const int* __restrict__ pos,
                      const int* __restrict__ req, const float* __restrict__ freqs,
                      __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                      const int* __restrict__ block_table, int table_width, int page_size, int n_pages,
                      int n_heads, int n_kv_heads, int head_dim, int* status, int heads_per_block) {
  const int t = blockIdx.x;
  const int r = req[t];
  if (r < 0) return;
  const int pieces = head_dim >> 3;                 // 16-byte pieces a head
  const int lanes = ROPE_THREADS / pieces;          // heads walked side by side
  const int piece = threadIdx.x % pieces, lane_head = threadIdx.x / pieces;
  if (lane_head >= lanes) return;
  const int p = pos[t];
  const int n_kv = (k != nullptr) ? n_kv_heads : 0;
  const int total = n_heads + 2 * n_kv;  // heads in the order q..., k..., v...
  const int h_end = min(total, (int)(blockIdx.y + 1) * heads_per_block);
  float sn[4], cs[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    sn[i] = 0.f;
    cs[i] = 1.f;
    if (freqs != nullptr) sincosf((float)p * freqs[piece * 4 + i], &sn[i], &cs[i]);
  }
  size_t slot = 0;
  if (n_kv > 0) {
    const int logical = p / page_size;
    const int page = (logical < table_width) ? block_table[(size_t)r * table_width + logical] : -1;
    if (page < 0 || page >= n_pages) {
      if (status) atomicOr(status, FG_STATUS_BAD_PAGE);
      return;
    }
    slot = (size_t)page * n_kv_heads * page_size + (p - logical * page_size);
  }
  auto rotate = [&](uint4 raw) {
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 val = __bfloat1622float2(h2[i]);
      h2[i] = __floats2bfloat162_rn(val.x * cs[i] - val.y * sn[i], val.y * cs[i] + val.x * sn[i]);
    }
    return raw;
  };
  for (int h0 = blockIdx.y * heads_per_block + lane_head; h0 < h_end; h0 += lanes * ROPE_UNROLL) {
    uint4 raw[ROPE_UNROLL];
    // the loads of several heads first, then their rotations and stores
#pragma unroll
    for (int u = 0; u < ROPE_UNROLL; ++u) {
      const int h = h0 + u * lanes;
      if (h >= h_end) continue;
      const __nv_bfloat16* src;
      if (h < n_heads) src = q + (size_t)t * q_stride + h * head_dim;
      else if (h < n_heads + n_kv) src = k + (size_t)t * k_stride + (h - n_heads) * head_dim;
      else src = v + (size_t)t * v_stride + (h - n_heads - n_kv) * head_dim;
      raw[u] = *reinterpret_cast<const uint4*>(src + piece * 8);
    }
#pragma unroll
    for (int u = 0; u < ROPE_UNROLL; ++u) {
      const int h = h0 + u * lanes;
      if (h >= h_end) continue;
      if (h < n_heads) {
        *reinterpret_cast<uint4*>(q + (size_t)t * q_stride + h * head_dim + piece * 8) = rotate(raw[u]);
        continue;
      }
      const bool is_v = h >= n_heads + n_kv;
      const int g = h - n_heads - (is_v ? n_kv : 0);
      const size_t dst = (slot + (size_t)g * page_size) * head_dim + piece * 8;
      *reinterpret_cast<uint4*>((is_v ? v_pages : k_pages) + dst) = is_v ? raw[u] : rotate(raw[u]);
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
  FG_CHECK_ARG(head_dim / 2 <= ROPE_THREADS, "fg_rope_kv_write: head size %d is too large", head_dim);
  const int total_heads = n_heads + (k ? 2 * n_kv_heads : 0);
  // many tokens: one block a token; few tokens: slices of heads, so that there are enough blocks
  int slices = n_tokens >= 1024 ? 1 : (n_tokens >= 128 ? 4 : 16);
  if (slices > total_heads) slices = total_heads;
  const int ipt = (total_heads + slices - 1) / slices;  // heads per block
  const dim3 grid(n_tokens, (total_heads + ipt - 1) / ipt);
  const int threads = ROPE_THREADS;
  FG_CHECK_ARG(grid.y <= 65535, "fg_rope_kv_write: too many heads");
  const size_t pair = dtype == FG_F32 ? 8 : 4;
  const auto ok = [&](const void* p, int stride) { return p == nullptr || (((uintptr_t)p % pair) == 0 && stride % 2 == 0); };
  const bool vec = ok(q, q_stride) && ok(k, k_stride) && ok(v, v_stride) && ok(k_pages, 0) && ok(v_pages, 0);
  const auto ok16 = [&](const void* p, int stride) { return p == nullptr || (((uintptr_t)p & 15) == 0 && stride % 8 == 0); };
  if (dtype == FG_BF16 && head_dim % 8 == 0 && head_dim / 8 <= ROPE_THREADS && ok16(q, q_stride) && ok16(k, k_stride) &&
      ok16(v, v_stride) && ok16(k_pages, 0) && ok16(v_pages, 0)) {
    rope_kv_bf16x8_kernel<<<grid, threads, 0, stream>>>(
        (__nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, pos, req,
        freqs, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, block_table, table_width, page_size, n_pages,
        n_heads, n_kv_heads, head_dim, status, ipt);
    FG_CHECK_LAUNCH("fg_rope_kv_write");
    return 0;
  }
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
