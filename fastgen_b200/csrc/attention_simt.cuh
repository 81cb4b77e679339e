// Paged causal attention on the CUDA cores, float32 arithmetic throughout.
//
// One kernel serves prompt portions and single decoded tokens alike: the host
// cuts the step's query tokens into tiles (request, first token, token count)
// and each thread block handles one tile for one group of query heads that
// share a key/value head.  Keys and values come only from the cache pages
// (the step's own keys were written before), in tiles of 32 positions that
// always start at multiples of 32 from position 0, so that the order of every
// sum depends only on the query's own position -- not on how the prompt was
// cut, what else is in the batch, or which pages hold the keys.
//
// Semantics of fastgen/forward.py:176-258: softmax(q.k * scale) v over the
// positions j <= pos(query) of the query's own request (and j > pos - window
// when a window is given), grouped-query heads h -> h / (Hq/Hkv).
// Running maximum, sum and output accumulator are float32; exp is expf.
//
// Storage type T (float or bf16) only affects loads and the final store.
#pragma once

#include "common.cuh"

namespace fg_attn {

constexpr int ROWS = 16;      // query rows (token x head-of-group) per block
constexpr int KEYS = 32;      // key positions per tile
constexpr int THREADS = 128;

template <typename T, int HD>
__global__ void __launch_bounds__(THREADS)
attention_simt_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                      const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                      const int* __restrict__ block_table, int table_width, int page_size,
                      int n_pages, const int* __restrict__ pos, const int* __restrict__ tile_req,
                      const int* __restrict__ tile_tok0, const int* __restrict__ tile_ntok,
                      int n_kv_heads, int group, int heads_per_block, int window, float scale,
                      int* status) {
  constexpr int HP = HD + 1;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float(*Qs)[HP] = reinterpret_cast<float(*)[HP]>(smem_raw);
  float(*Ks)[HP] = reinterpret_cast<float(*)[HP]>(Qs + ROWS);
  float(*Vs)[HP] = reinterpret_cast<float(*)[HP]>(Ks + KEYS);
  float(*Ps)[KEYS + 1] = reinterpret_cast<float(*)[KEYS + 1]>(Vs + KEYS);
  __shared__ float alpha_s[ROWS];
  __shared__ float l_s[ROWS];
  __shared__ long long key_base[KEYS];
  __shared__ int row_pos[ROWS];

  const int tile = blockIdx.x;
  const int g = blockIdx.y;        // key/value head
  const int sub = blockIdx.z;      // which slice of the group's heads
  const int b = tile_req[tile];
  const int tok0 = tile_tok0[tile];
  const int ntok = tile_ntok[tile];
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;

  // row r -> (token r / heads_per_block, head-of-group sub*hpb + r % hpb)
  auto row_token = [&](int r) { return r / heads_per_block; };
  auto row_head = [&](int r) { return sub * heads_per_block + (r % heads_per_block); };
  auto row_valid = [&](int r) { return row_token(r) < ntok && row_head(r) < group; };

  if (b < 0) {
    // padding of a fixed-size batch: no request, the output rows are zeroed
    for (int i = tid; i < ROWS * HD; i += THREADS) {
      const int r = i / HD, d = i - r * HD;
      if (row_valid(r))
        out[(size_t)(tok0 + row_token(r)) * out_stride + (g * group + row_head(r)) * HD + d] = from_f32<T>(0.f);
    }
    return;
  }
  if (tid < ROWS) row_pos[tid] = row_valid(tid) ? pos[tok0 + row_token(tid)] : -1;
  for (int i = tid; i < ROWS * HD; i += THREADS) {
    const int r = i / HD, d = i - r * HD;
    float v = 0.f;
    if (row_valid(r))
      v = to_f32<T>(q[(size_t)(tok0 + row_token(r)) * q_stride + (g * group + row_head(r)) * HD + d]);
    Qs[r][d] = v;
  }
  __syncthreads();

  int max_pos = -1, min_pos = 0x7fffffff;
  for (int r = 0; r < ROWS; ++r) {
    const int p = row_pos[r];
    if (p >= 0) {
      max_pos = max(max_pos, p);
      min_pos = min(min_pos, p);
    }
  }
  if (max_pos < 0) return;
  int k_lo = 0;
  if (window > 0) k_lo = max(0, min_pos - window + 1) / KEYS * KEYS;

  // this thread's 4 score rows: warp, warp+4, warp+8, warp+12; column = lane
  float m_run[4], l_run[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m_run[i] = -INFINITY;
    l_run[i] = 0.f;
  }
  // this thread's output elements: row tid/8, columns tid%8 + 8*i
  constexpr int OD = HD / 8;
  float o_acc[OD];
#pragma unroll
  for (int i = 0; i < OD; ++i) o_acc[i] = 0.f;
  const int o_row = tid >> 3, o_col = tid & 7;

  for (int k0 = k_lo; k0 <= max_pos; k0 += KEYS) {
    if (tid < KEYS) {
      const int j = k0 + tid;
      long long base = -1;
      if (j <= max_pos) {
        const int logical = j / page_size;
        const int page = logical < table_width ? block_table[(size_t)b * table_width + logical] : -1;
        if (page >= 0 && page < n_pages) {
          base = (((long long)page * n_kv_heads + g) * page_size + (j - logical * page_size)) * HD;
        } else if (window <= 0 || j > min_pos - window) {
          // a key some row must see has no page
          if (status) atomicOr(status, FG_STATUS_BAD_PAGE);
        }
      }
      key_base[tid] = base;
    }
    __syncthreads();
    for (int i = tid; i < KEYS * HD; i += THREADS) {
      const int c = i / HD, d = i - c * HD;
      const long long base = key_base[c];
      float kv = 0.f, vv = 0.f;
      if (base >= 0) {
        kv = to_f32<T>(k_pages[base + d]);
        vv = to_f32<T>(v_pages[base + d]);
      }
      Ks[c][d] = kv;
      Vs[c][d] = vv;
    }
    __syncthreads();

    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
    for (int d = 0; d < HD; ++d) {
      const float kv = Ks[lane][d];
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i] = fmaf(Qs[warp + 4 * i][d], kv, s[i]);
    }
    const int j = k0 + lane;
    const bool has_key = key_base[lane] >= 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = warp + 4 * i;
      const int p = row_pos[r];
      const bool visible = has_key && p >= 0 && j <= p && (window <= 0 || j > p - window);
      const float sv = visible ? s[i] * scale : -INFINITY;
      const float m_tile = warp_max(sv);
      const float m_new = fmaxf(m_run[i], m_tile);
      float pr = 0.f, al = 1.f;
      if (m_new != -INFINITY) {
        pr = visible ? expf(sv - m_new) : 0.f;
        al = (m_run[i] == -INFINITY) ? 0.f : expf(m_run[i] - m_new);
      }
      const float psum = warp_sum(pr);
      l_run[i] = l_run[i] * al + psum;
      m_run[i] = m_new;
      Ps[r][lane] = pr;
      if (lane == 0) alpha_s[r] = al;
    }
    __syncthreads();

    {
      const float al = alpha_s[o_row];
#pragma unroll
      for (int i = 0; i < OD; ++i) o_acc[i] *= al;
#pragma unroll 4
      for (int c = 0; c < KEYS; ++c) {
        const float pr = Ps[o_row][c];
#pragma unroll
        for (int i = 0; i < OD; ++i) o_acc[i] = fmaf(pr, Vs[c][o_col + 8 * i], o_acc[i]);
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (lane == 0) l_s[warp + 4 * i] = l_run[i];
  __syncthreads();
  if (row_valid(o_row)) {
    const float l = l_s[o_row];
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* o = out + (size_t)(tok0 + row_token(o_row)) * out_stride + (g * group + row_head(o_row)) * HD;
#pragma unroll
    for (int i = 0; i < OD; ++i) o[o_col + 8 * i] = from_f32<T>(o_acc[i] * inv);
  }
}

template <int HD>
constexpr size_t simt_smem_bytes() {
  return sizeof(float) * ((ROWS + 2 * KEYS) * (HD + 1) + ROWS * (KEYS + 1));
}

}  // namespace fg_attn
