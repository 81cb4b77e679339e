// Single-token (decode) attention for bfloat16 with tiled TMA loads.
//
// Same split / merge / combine scheme and the same arithmetic as
// attention_decode_kernel (attention_mma.cuh); what changes is how the split's
// 128 key and value rows reach shared memory: one elected thread issues one
// cp.async.bulk.tensor instruction per (page, 64-element half of the head size),
// the copies are tracked by two mbarriers (keys, values), and the rows land
// 128-byte swizzled, which ldmatrix then reads without bank conflicts.  The
// pool is described by a 5-d tensor map [layer, page, kv head, slot, element].
//
// Needs head sizes that are multiples of 64, pages of a power of two >= 8 slots
// and groups of at most 16 query heads; other shapes use the cp.async kernel.
#pragma once

#include <cuda.h>

#include "attention_mma.cuh"

namespace fg_tma {

using namespace fg_mma;

constexpr int SPLIT = DECODE_SPLIT;          // 128 key positions
constexpr int HALF_BYTES = SPLIT * 128;      // one 64-element half of all rows

__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            int c4, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, "
      "%4, %5, %6}], [%7];\n" ::"r"(smem_u32(dst)),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(smem_u32(bar))
      : "memory");
}

// byte offset of the 16-byte piece `chunk` (0..7) of `row` inside a swizzled half
__device__ __forceinline__ int swz(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

template <int HD, int NT>
__device__ __forceinline__ void qk_product_swz(float (&s)[NT][4], const uint32_t (&qf)[HD / 16][4],
                                               const unsigned char* ks, int row0, int lane) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
    const unsigned char* half = ks + (kk / 4) * HALF_BYTES;
    const int chunk = (kk % 4) * 2 + ((lane >> 3) & 1);
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      const int row = row0 + np * 16 + (lane & 7) + ((lane >> 4) << 3);
      ldmatrix_x4(b, half + swz(row, chunk));
      mma_16816(s[2 * np], qf[kk], b[0], b[1]);
      mma_16816(s[2 * np + 1], qf[kk], b[2], b[3]);
    }
  }
}

template <int HD, int NT>
__device__ __forceinline__ void pv_product_swz(float (&o)[HD / 8][4], const float (&p)[NT][4],
                                               const unsigned char* vs, int row0, int lane) {
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
    a[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
    a[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
    a[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
    const int row = row0 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
    for (int np = 0; np < HD / 16; ++np) {
      uint32_t b[4];
      const unsigned char* half = vs + (np / 4) * HALF_BYTES;
      const int chunk = (np % 4) * 2 + (lane >> 4);
      ldmatrix_x4_trans(b, half + swz(row, chunk));
      mma_16816(o[2 * np], a, b[0], b[1]);
      mma_16816(o[2 * np + 1], a, b[2], b[3]);
    }
  }
}

template <int HD>
constexpr size_t decode_tma_smem_bytes() {
  // keys, values (unpadded, swizzled), padded queries, and slack to align to 1024
  return (size_t)2 * SPLIT * HD * 2 + sizeof(__nv_bfloat16) * Tile<HD>::LD * DECODE_ROWS + 1024;
}

template <int HD>
__global__ void __launch_bounds__(THREADS)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                            int layer, const __nv_bfloat16* __restrict__ q, int q_stride,
                            const int* __restrict__ block_table, int table_width, int page_size, int n_pages,
                            const int* __restrict__ pos, const int* __restrict__ seq_req,
                            const int* __restrict__ seq_tok, int n_heads, int group, int window,
                            float scale_log2, float* __restrict__ scratch, int max_splits, int* status) {
  static_assert(HD % 64 == 0, "tiled loads take 64-element halves");
  constexpr int LD = Tile<HD>::LD;
  constexpr int NT = 4;
  constexpr int HALVES = HD / 64;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  unsigned char* Ks = smem;                       // [HALVES][SPLIT rows][128 B]
  unsigned char* Vs = Ks + HALVES * HALF_BYTES;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(Vs + HALVES * HALF_BYTES);
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ int box_page[SPLIT / 8];  // page of each box, -1: nothing to load

  const int split = blockIdx.x, g = blockIdx.y, seq = blockIdx.z;
  const int b = seq_req[seq];
  if (b < 0) return;
  const int tok = seq_tok[seq];
  const int p = pos[tok];
  const int k0 = split * SPLIT;
  if (k0 > p) return;
  const int k_begin = window > 0 ? max(0, p - window + 1) : 0;
  if (k0 + SPLIT <= k_begin) return;
  const int k_end = p + 1;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int box_rows = min(page_size, SPLIT);
  const int n_boxes = SPLIT / box_rows;

  if (tid < n_boxes) {
    const int j0 = k0 + tid * box_rows;
    int page = -1;
    if (j0 < k_end && j0 + box_rows > k_begin) {
      const int logical = j0 / page_size;
      page = logical < table_width ? block_table[(size_t)b * table_width + logical] : -1;
      if (page < 0 || page >= n_pages) {
        page = -1;
        if (status) atomicOr(status, FG_STATUS_BAD_PAGE);
      }
    }
    box_page[tid] = page;
  }
  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_fence_init();
  }
  __syncthreads();

  if (tid == 0) {
    int n_valid = 0;
    for (int i = 0; i < n_boxes; ++i) n_valid += box_page[i] >= 0;
    const int bytes = n_valid * box_rows * HD * 2;
    const int slot0 = k0 % page_size;  // 0 unless pages are longer than a split
    mbar_arrive_expect(&bars[0], bytes);
    for (int i = 0; i < n_boxes; ++i)
      if (box_page[i] >= 0)
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
          tma_load_5d(Ks + h * HALF_BYTES + i * box_rows * 128, &k_map, h * 64, slot0, g, box_page[i], layer,
                      &bars[0]);
    mbar_arrive_expect(&bars[1], bytes);
    for (int i = 0; i < n_boxes; ++i)
      if (box_page[i] >= 0)
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
          tma_load_5d(Vs + h * HALF_BYTES + i * box_rows * 128, &v_map, h * 64, slot0, g, box_page[i], layer,
                      &bars[1]);
  }
  // boxes with nothing to load hold zeros (a masked probability times garbage could be NaN)
  for (int i = 0; i < n_boxes; ++i) {
    if (box_page[i] >= 0) continue;
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int h = 0; h < HALVES; ++h)
      for (int c = tid; c < box_rows * 8; c += THREADS) {
        *reinterpret_cast<uint4*>(Ks + h * HALF_BYTES + i * box_rows * 128 + c * 16) = z;
        *reinterpret_cast<uint4*>(Vs + h * HALF_BYTES + i * box_rows * 128 + c * 16) = z;
      }
  }
  constexpr int CH = HD / 8;
  for (int i = tid; i < DECODE_ROWS * CH; i += THREADS) {
    const int r = i / CH, c = i - r * CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < group) v = *reinterpret_cast<const uint4*>(q + (size_t)tok * q_stride + (g * group + r) * HD + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * LD + c * 8) = v;
  }
  __syncthreads();
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk)
    ldmatrix_x4(qf[kk], Qs + (lane & 15) * LD + kk * 16 + ((lane >> 4) << 3));

  mbar_wait(&bars[0], 0, status);
  float s[NT][4];
  qk_product_swz<HD, NT>(s, qf, Ks, warp * 32, lane);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int j = k0 + warp * 32 + nt * 8 + 2 * (lane & 3) + (e & 1);
      const bool vis = j >= k_begin && j < k_end;
      s[nt][e] = vis ? s[nt][e] * scale_log2 : -INFINITY;
    }
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  softmax_step<HD, NT>(s, o, m, l);
  mbar_wait(&bars[1], 0, status);
  pv_product_swz<HD, NT>(o, s, Vs, warp * 32, lane);

  // merge the 4 warps through shared memory (the keys' space is free now)
  float* wm = reinterpret_cast<float*>(Qs);
  float* wl = wm + 4 * DECODE_ROWS;
  __syncthreads();
  float* wo = reinterpret_cast<float*>(Ks);  // [4][16][HD]
  const int r0 = lane >> 2;
  if ((lane & 3) == 0) {
    wm[warp * DECODE_ROWS + r0] = m[0];
    wm[warp * DECODE_ROWS + r0 + 8] = m[1];
    wl[warp * DECODE_ROWS + r0] = l[0];
    wl[warp * DECODE_ROWS + r0 + 8] = l[1];
  }
#pragma unroll
  for (int nt = 0; nt < HD / 8; ++nt) {
    const int d = nt * 8 + 2 * (lane & 3);
    if (r0 < group)
      *reinterpret_cast<float2*>(wo + (warp * DECODE_ROWS + r0) * HD + d) = make_float2(o[nt][0], o[nt][1]);
    if (r0 + 8 < group)
      *reinterpret_cast<float2*>(wo + (warp * DECODE_ROWS + r0 + 8) * HD + d) = make_float2(o[nt][2], o[nt][3]);
  }
  __syncthreads();
  for (int i = tid; i < group * HD; i += THREADS) {
    const int r = i / HD, d = i - r * HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, wm[w * DECODE_ROWS + r]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = wm[w * DECODE_ROWS + r];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
      acc += f * wo[(w * DECODE_ROWS + r) * HD + d];
      ll += f * wl[w * DECODE_ROWS + r];
    }
    float* dst = scratch + (((size_t)seq * n_heads + g * group + r) * max_splits + split) * part_stride<HD>();
    dst[d] = acc;
    if (d == 0) {
      dst[HD] = mm;
      dst[HD + 1] = ll;
    }
  }
}

}  // namespace fg_tma
