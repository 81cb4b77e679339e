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
// Two kernels for single tokens: attention_decode_tma_kernel, one block per (request,
// kv head, split), for steps with few such items; and
// attention_decode_persistent_kernel, whose blocks stay on their SM and walk the items
// that exist (a producer warp streams keys and values through a ring of slots ahead of
// four consumer warps), for steps with many.  Both leave partials per split in scratch
// for attention_combine_kernel.  The file also holds the mma.sync prompt kernel on the
// same TMA tiles (attention_prefill_tma_kernel), used where tcgen05 is not.
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

template <int HD, int NT, int HALF = HALF_BYTES>
__device__ __forceinline__ void qk_product_swz(float (&s)[NT][4], const uint32_t (&qf)[HD / 16][4],
                                               const unsigned char* ks, int row0, int lane) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
    const unsigned char* half = ks + (kk / 4) * HALF;
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

template <int HD, int NT, int HALF = HALF_BYTES>
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
      const unsigned char* half = vs + (np / 4) * HALF;
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
                            int layer, const __nv_bfloat16* q, int q_stride,
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
  __shared__ int gave_up;              // set by a wait that ran out (see mbar_wait)

  // positions, slots and block tables are inputs of the step (no kernel of the step
  // writes them), so the page look-ups and the barrier set-up run while the kernel
  // before this one finishes; keys, values and queries are touched after the wait
  pdl_trigger();
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
    gave_up = 0;
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_fence_init();
  }
  __syncthreads();
  // The step's own kernels write keys and values at the tokens' positions only, so a
  // split that ends before this token's position is loaded without waiting for them.
  const bool early = k0 + SPLIT <= p;
  if (!early) pdl_wait();

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
  if (early) pdl_wait();  // the queries come from the kernel before
  constexpr int CH = HD / 8;
  for (int i = tid; i < DECODE_ROWS * CH; i += THREADS) {
    const int r = i / CH, c = i - r * CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < group) v = ld_global_16(q + (size_t)tok * q_stride + (g * group + r) * HD + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * LD + c * 8) = v;
  }
  __syncthreads();
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk)
    ldmatrix_x4(qf[kk], Qs + (lane & 15) * LD + kk * 16 + ((lane >> 4) << 3));

  mbar_wait(&bars[0], 0, status, &gave_up);
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
  mbar_wait(&bars[1], 0, status, &gave_up);
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


// ---------------------------------------------------------------------------------
// single tokens, persistent: blocks stay on their SM and walk a list of (request, kv
// head, split) items.  A producer warp streams the items' keys and values through a ring
// of shared-memory slots (keys and values of a split take a slot each) while four
// consumer warps work on the slots before, so page look-ups, launch ramps and the merge
// of the warps hide behind the loads.  The products are taken transposed: keys (or value
// columns) are the 16-row operand and the group's heads the 8-column one, so a group of
// up to 8 heads wastes half of a tile instead of three quarters.
// ---------------------------------------------------------------------------------
constexpr int PS_THREADS = 160;  // 4 consumer warps + 1 producer warp
constexpr int PS_CONSUMERS = 128;
constexpr int PS_SLOTS = 3;
constexpr int PS_MAX_GROUP = 8;
constexpr int PS_MAX_SEQS = 512;   // requests whose positions a block keeps in shared memory

template <int HD>
__host__ __device__ constexpr int ps_merge_ld() { return HD + 4; }  // rows of the merge buffer fall on different banks

template <int HD>
inline size_t decode_persistent_smem_bytes(int group) {
  // the ring, the merge buffer of the four warps (values, maxima, sums), alignment slack
  return (size_t)PS_SLOTS * SPLIT * HD * 2 + (size_t)4 * group * ps_merge_ld<HD>() * 4 + 2 * 4 * PS_MAX_GROUP * 4 +
         1024;
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}

// blocks an SM: the ring of a head size of 64 is half as large, and its items are half as
// long for the same work around them, so a third block pays
template <int HD>
constexpr int ps_blocks_per_sm() { return HD <= 64 ? 3 : 2; }

template <int HD>
__global__ void __launch_bounds__(PS_THREADS, ps_blocks_per_sm<HD>())
attention_decode_persistent_kernel(const __grid_constant__ CUtensorMap k_map,
                                   const __grid_constant__ CUtensorMap v_map, int layer,
                                   const __nv_bfloat16* q, int q_stride,
                                   const int* __restrict__ block_table, int table_width, int page_size,
                                   int n_pages, const int* __restrict__ pos, const int* __restrict__ seq_req,
                                   const int* __restrict__ seq_tok, int n_seqs, int n_heads, int n_kv_heads,
                                   int group, int window, float scale_log2, float* __restrict__ scratch,
                                   int* __restrict__ first_pair_out, long long max_pairs, int max_splits,
                                   int* status) {
  static_assert(HD % 64 == 0, "tiled loads take 64-element halves");
  constexpr int HALVES = HD / 64;
  constexpr int SLOT_BYTES = HALVES * HALF_BYTES;  // keys (or values) of one split
  constexpr int MLD = ps_merge_ld<HD>();
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  unsigned char* ring = smem;                                              // [PS_SLOTS][HALVES][SPLIT rows][128 B]
  float* wo = reinterpret_cast<float*>(ring + PS_SLOTS * SLOT_BYTES);      // [4 warps][group][MLD]
  float* wm = wo + 4 * group * MLD;                                        // [4][8] maxima
  float* wl = wm + 4 * PS_MAX_GROUP;                                       // [4][8] sums
  __shared__ __align__(8) uint64_t full[PS_SLOTS], empty[PS_SLOTS];
  // per request: the token's position (-1: padding lane) and the number of (request, split)
  // pairs before it
  __shared__ int s_pos[PS_MAX_SEQS], s_cum[PS_MAX_SEQS + 1];
  __shared__ int gave_up;  // set by a wait that ran out: the waits after it return at once (see mbar_wait)

  pdl_trigger();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    gave_up = 0;
    for (int i = 0; i < PS_SLOTS; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 4);  // one arrival a consumer warp
    }
    mbar_fence_init();
  }
  // Requests differ in length, and a request only has the splits its keys reach: the items
  // are the (request, split, kv head) triples that exist, numbered request by request, so
  // that block b takes items b, b + G, ... and every block gets the same number of them.
  // Positions are inputs of the step (no kernel of the step writes them).
  auto first_split = [&](int p) { return window > 0 ? max(0, p - window + 1) / SPLIT : 0; };
  for (int sq = tid; sq < n_seqs; sq += PS_THREADS) s_pos[sq] = seq_req[sq] < 0 ? -1 : pos[seq_tok[sq]];
  __syncthreads();
  if (warp == 0) {
    // an exclusive scan of the split counts: each lane sums a stretch, the warp scans the sums
    const int per_lane = (n_seqs + 31) / 32;
    const int lo = lane * per_lane, hi = min(n_seqs, lo + per_lane);
    int sum = 0;
    for (int sq = lo; sq < hi; ++sq) {
      const int p = s_pos[sq];
      sum += p < 0 ? 0 : min(p / SPLIT, max_splits - 1) - first_split(p) + 1;
    }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - sum;
    for (int sq = lo; sq < hi; ++sq) {
      s_cum[sq] = run;
      const int p = s_pos[sq];
      run += p < 0 ? 0 : min(p / SPLIT, max_splits - 1) - first_split(p) + 1;
    }
    if (lane == 31) s_cum[n_seqs] = incl;
  }
  __syncthreads();
  // The step's own kernels write keys and values at the tokens' positions only: the
  // producer loads splits that end before the token's position without waiting for the
  // kernel before this one, and waits once it meets a split that holds the position.
  // The consumers wait before they read the queries.

  const int box_rows = min(page_size, SPLIT);
  const int n_boxes = SPLIT / box_rows;
  // the (request, split) pairs also number the partials, [pair][head]: what the merge of the
  // splits needs to find them goes to global memory
  if (blockIdx.x == 0)
    for (int sq = tid; sq <= n_seqs; sq += PS_THREADS) first_pair_out[sq] = s_cum[sq];
  int n_pairs = s_cum[n_seqs];
  if (n_pairs > max_pairs) {
    // the scratch was sized for fewer: report instead of writing past it
    if (tid == 0 && blockIdx.x == 0 && status) atomicOr(status, FG_STATUS_BAD_SPLITS);
    n_pairs = (int)max_pairs;
  }
  const int total = n_pairs * n_kv_heads;
  // Both kinds of warps walk the same list.
  auto item_of = [&](int item, int& seq, int& g, int& split, int& p, int& k_begin) -> bool {
    g = item % n_kv_heads;
    const int r = item / n_kv_heads;
    int lo = 0, hi = n_seqs;  // the last request whose first pair is <= r
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_cum[mid] <= r) lo = mid; else hi = mid;
    }
    seq = lo;
    p = s_pos[seq];
    split = first_split(p) + (r - s_cum[seq]);
    k_begin = window > 0 ? max(0, p - window + 1) : 0;
    return true;
  };

  if (warp == 4) {
    // ================================ producer ================================
    int n_fill = 0;  // fills so far: item i's keys are fill 2i, its values fill 2i + 1
    bool waited = false;
    for (int item = blockIdx.x; item < total; item += gridDim.x) {
      int seq, g, split, p, k_begin;
      if (!item_of(item, seq, g, split, p, k_begin)) continue;
      const int k0 = split * SPLIT, k_end = p + 1;
      if (!waited && k0 + SPLIT > p) {
        pdl_wait();
        waited = true;
      }
      const int b = seq_req[seq];
      // pages of the split's boxes: lane i looks up box i
      int page = -1;
      if (lane < n_boxes) {
        const int j0 = k0 + lane * box_rows;
        if (j0 < k_end && j0 + box_rows > k_begin) {
          const int logical = j0 / page_size;
          page = logical < table_width ? block_table[(size_t)b * table_width + logical] : -1;
          if (page < 0 || page >= n_pages) {
            page = -1;
            if (status) atomicOr(status, FG_STATUS_BAD_PAGE);
          }
        }
      }
      const unsigned valid = __ballot_sync(0xffffffffu, page >= 0);
      const int bytes = __popc(valid) * box_rows * HD * 2;
      const int slot0 = k0 % page_size;  // 0 unless pages are longer than a split
#pragma unroll
      for (int kv = 0; kv < 2; ++kv) {
        const int slot = n_fill % PS_SLOTS;
        if (n_fill >= PS_SLOTS) mbar_wait(&empty[slot], (n_fill / PS_SLOTS - 1) & 1, status, &gave_up);
        unsigned char* dst = ring + slot * SLOT_BYTES;
        // boxes with nothing to load hold zeros (a masked probability times garbage could be NaN)
        if (valid != (n_boxes >= 32 ? 0xffffffffu : (1u << n_boxes) - 1u)) {
          for (int i = 0; i < n_boxes; ++i) {
            if (valid & (1u << i)) continue;
            const uint4 z = make_uint4(0, 0, 0, 0);
            for (int h = 0; h < HALVES; ++h)
              for (int c = lane; c < box_rows * 8; c += 32)
                *reinterpret_cast<uint4*>(dst + h * HALF_BYTES + i * box_rows * 128 + c * 16) = z;
          }
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_expect(&full[slot], bytes);
        __syncwarp();
        if (page >= 0) {  // lane i issues box i's copies
#pragma unroll
          for (int h = 0; h < HALVES; ++h)
            tma_load_5d(dst + h * HALF_BYTES + lane * box_rows * 128, kv ? &v_map : &k_map, h * 64, slot0, g, page,
                        layer, &full[slot]);
        }
        ++n_fill;
      }
    }
    if (!waited) pdl_wait();
  } else {
    // ================================ consumers ================================
    pdl_wait();
    int n_item = 0;
    const int hq = lane >> 2, qd = (lane & 3) * 2;
    for (int item = blockIdx.x; item < total; item += gridDim.x) {
      int seq, g, split, p, k_begin;
      if (!item_of(item, seq, g, split, p, k_begin)) continue;
      const int k0 = split * SPLIT, k_end = p + 1;
      const int tok = seq_tok[seq];
      // the queries as the 8-column operand, straight from global memory: column lane/4 is
      // a head of the group (zero beyond it), rows 2*(lane%4), +1 and +8, +9 of each 16 dims
      uint32_t qb[HD / 16][2];
      {
        const __nv_bfloat16* qrow = q + (size_t)tok * q_stride + (g * group + hq) * HD + qd;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          qb[kk][0] = hq < group ? ld_global_4(qrow + kk * 16) : 0u;
          qb[kk][1] = hq < group ? ld_global_4(qrow + kk * 16 + 8) : 0u;
        }
      }
      const int fk = 2 * n_item, fv = fk + 1;
      const int slot_k = fk % PS_SLOTS, slot_v = fv % PS_SLOTS;
      const unsigned char* Ks = ring + slot_k * SLOT_BYTES;
      const unsigned char* Vs = ring + slot_v * SLOT_BYTES;

      // S^T[keys, heads] = K Q^T for this warp's 32 keys
      mbar_wait(&full[slot_k], (fk / PS_SLOTS) & 1, status, &gave_up);
      float s[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        s[mt][0] = s[mt][1] = s[mt][2] = s[mt][3] = 0.f;
        const int row = warp * 32 + mt * 16 + (lane & 15);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          uint32_t a[4];
          ldmatrix_x4(a, Ks + (kk >> 2) * HALF_BYTES + swz(row, (kk & 3) * 2 + (lane >> 4)));
          mma_16816(s[mt], a, qb[kk][0], qb[kk][1]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[slot_k]);  // this warp is done with the keys

      // softmax over the warp's keys, per head: this thread holds heads qd and qd + 1
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = k0 + warp * 32 + mt * 16 + hq + ((e & 2) ? 8 : 0);
          const bool vis = j >= k_begin && j < k_end;
          s[mt][e] = vis ? s[mt][e] * scale_log2 : -INFINITY;
          mx[e & 1] = fmaxf(mx[e & 1], s[mt][e]);
        }
      float sum[2] = {0.f, 0.f};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          // the probabilities are rounded to bfloat16 for the product; sum what is used
          const float pr = mx[e & 1] == -INFINITY
                               ? 0.f
                               : __bfloat162float(__float2bfloat16_rn(exp2f(s[mt][e] - mx[e & 1])));
          s[mt][e] = pr;
          sum[e & 1] += pr;
        }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 4);
        sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 8);
        sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 16);
      }
      // P^T as the 8-column operand: an 8x8 transpose in registers for each half tile
      uint32_t pb[2][2];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        pb[mt][0] = movmatrix_trans(pack_bf16(s[mt][0], s[mt][1]));
        pb[mt][1] = movmatrix_trans(pack_bf16(s[mt][2], s[mt][3]));
      }

      // O^T[dims, heads] = V^T P^T
      mbar_wait(&full[slot_v], (fv / PS_SLOTS) & 1, status, &gave_up);
      float o[HD / 16][4];
#pragma unroll
      for (int dt = 0; dt < HD / 16; ++dt) {
        o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          const int key = warp * 32 + ks * 16 + ((lane >> 4) << 3) + (lane & 7);
          uint32_t a[4];
          ldmatrix_x4_trans(a, Vs + (dt >> 2) * HALF_BYTES + swz(key, (dt & 3) * 2 + ((lane >> 3) & 1)));
          mma_16816(o[dt], a, pb[ks][0], pb[ks][1]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[slot_v]);  // ... and with the values

      // merge the four warps (heads of the group only)
      if (hq == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          wm[warp * PS_MAX_GROUP + qd + h] = mx[h];
          wl[warp * PS_MAX_GROUP + qd + h] = sum[h];
        }
      }
#pragma unroll
      for (int dt = 0; dt < HD / 16; ++dt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int head = qd + (e & 1), d = dt * 16 + hq + ((e & 2) ? 8 : 0);
          if (head < group) wo[(warp * group + head) * MLD + d] = o[dt][e];
        }
      asm volatile("bar.sync 1, %0;\n" ::"n"(PS_CONSUMERS) : "memory");
      for (int i = tid; i < group * HD; i += PS_CONSUMERS) {
        const int r = i / HD, d = i - r * HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, wm[w * PS_MAX_GROUP + r]);
        float acc = 0.f, ll = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const float mw = wm[w * PS_MAX_GROUP + r];
          const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
          acc += f * wo[(w * group + r) * MLD + d];
          ll += f * wl[w * PS_MAX_GROUP + r];
        }
        float* dst = scratch + ((size_t)(item / n_kv_heads) * n_heads + g * group + r) * part_stride<HD>();
        dst[d] = acc;
        if (d == 0) {
          dst[HD] = mm;
          dst[HD + 1] = ll;
        }
      }
      asm volatile("bar.sync 1, %0;\n" ::"n"(PS_CONSUMERS) : "memory");  // the merge buffer is free again
      ++n_item;
    }
  }
}

// ---------------------------------------------------------------------------------
// prompt portions with tiled TMA loads
// ---------------------------------------------------------------------------------
constexpr int PF_ROWS = 128;   // query rows per block (8 warps x 16)
constexpr int PF_KEYS = 64;    // key positions per tile
constexpr int PF_THREADS = 256;
constexpr int PF_HALF = PF_KEYS * 128;  // bytes of one 64-element half of a tile

// Online softmax on raw scores: the scale is folded into the exponent,
// p = 2^((s - m) * c) with c = scale * log2(e); m is kept in raw units.
template <int HD, int NT>
__device__ __forceinline__ void softmax_step_raw(float (&s)[NT][4], float (&o)[HD / 8][4], float (&m)[2],
                                                 float (&l)[2], float c) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float mx = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * h], s[nt][2 * h + 1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m[h], mx);
    float alpha = 1.f, sum = 0.f;
    if (m_new == -INFINITY) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) s[nt][2 * h] = s[nt][2 * h + 1] = 0.f;
    } else {
      alpha = (m[h] == -INFINITY) ? 0.f : exp2f((m[h] - m_new) * c);
      const float mc = m_new * c;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const float p0 = exp2f(fmaf(s[nt][2 * h], c, -mc));
        const float p1 = exp2f(fmaf(s[nt][2 * h + 1], c, -mc));
        s[nt][2 * h] = p0;
        s[nt][2 * h + 1] = p1;
        sum += p0 + p1;
      }
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    l[h] = l[h] * alpha + sum;
    m[h] = m_new;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
      o[nt][2 * h] *= alpha;
      o[nt][2 * h + 1] *= alpha;
    }
  }
}

template <int HD>
constexpr size_t prefill_tma_smem_bytes() {
  // two stages of keys and values (unpadded, swizzled), padded queries, alignment slack
  return (size_t)2 * 2 * PF_KEYS * HD * 2 + sizeof(__nv_bfloat16) * Tile<HD>::LD * PF_ROWS + 1024;
}

template <int HD>
__global__ void __launch_bounds__(PF_THREADS)
attention_prefill_tma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                             int layer, const __nv_bfloat16* __restrict__ q, int q_stride,
                             __nv_bfloat16* __restrict__ out, int out_stride, const int* __restrict__ block_table,
                             int table_width, int page_size, int n_pages, const int* __restrict__ pos,
                             const int* __restrict__ tile_req, const int* __restrict__ tile_tok0,
                             const int* __restrict__ tile_ntok, int n_tiles_total, int group,
                             int heads_per_block, int window, float scale_log2, int* status) {
  static_assert(HD % 64 == 0, "tiled loads take 64-element halves");
  constexpr int LD = Tile<HD>::LD;
  constexpr int NT = PF_KEYS / 8;
  constexpr int HALVES = HD / 64;
  constexpr int STAGE_BYTES = HALVES * PF_HALF;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  unsigned char* Ks = smem;                     // [2 stages][HALVES][64 rows][128 B]
  unsigned char* Vs = Ks + 2 * STAGE_BYTES;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(Vs + 2 * STAGE_BYTES);
  __shared__ __align__(8) uint64_t full[2];
  __shared__ int row_pos[PF_ROWS];
  constexpr int PAGE_STAGE = 512;             // box page ids kept in shared memory at a time
  __shared__ int box_pages[PAGE_STAGE];
  __shared__ int gave_up;  // set by a wait that ran out (see mbar_wait)

  // the tile list is in ascending order of work and blockIdx.x runs fastest: all key/value
  // heads of the heaviest tile start first
  const int tile = n_tiles_total - 1 - blockIdx.y;
  const int g = blockIdx.x, sub = blockIdx.z;
  const int b = tile_req[tile];
  const int tok0 = tile_tok0[tile], ntok = tile_ntok[tile];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (b < 0) return;

  auto row_token = [&](int r) { return r / heads_per_block; };
  auto row_head = [&](int r) { return sub * heads_per_block + (r % heads_per_block); };
  auto row_valid = [&](int r) { return row_token(r) < ntok && row_head(r) < group; };

  if (tid < PF_ROWS) row_pos[tid] = row_valid(tid) ? pos[tok0 + row_token(tid)] : -1;
  constexpr int CH = HD / 8;
  for (int i = tid; i < PF_ROWS * CH; i += PF_THREADS) {
    const int r = i / CH, c = i - r * CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row_valid(r))
      v = *reinterpret_cast<const uint4*>(q + (size_t)(tok0 + row_token(r)) * q_stride +
                                          (g * group + row_head(r)) * HD + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * LD + c * 8) = v;
  }
  if (tid == 0) {
    gave_up = 0;
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    mbar_fence_init();
  }
  __syncthreads();

  // tokens of a tile are consecutive positions: the extremes are at its ends
  const int min_pos = row_pos[0];
  const int max_pos = min_pos + ntok - 1;
  const int k_begin = window > 0 ? max(0, min_pos - window + 1) : 0;
  const int k_lo = k_begin / PF_KEYS * PF_KEYS;
  const int k_end = max_pos + 1;
  const int n_tiles = (k_end - k_lo + PF_KEYS - 1) / PF_KEYS;
  const int* table_row = block_table + (size_t)b * table_width;
  const int box_rows = min(page_size, PF_KEYS);
  const int n_boxes = PF_KEYS / box_rows;

  // page of box x (counted over all key tiles), or -1 when the box holds no position in
  // [k_begin, k_end); looked up for a stretch of tiles at a time so that the block-table
  // reads are off the critical path of every tile
  const int tiles_per_fill = PAGE_STAGE / n_boxes;
  auto fill_pages = [&](int t_first) {
    const int n = min(tiles_per_fill, n_tiles - t_first) * n_boxes;
    for (int x = tid; x < n; x += PF_THREADS) {
      const int j0 = k_lo + t_first * PF_KEYS + x * box_rows;
      int page = -1;
      if (j0 < k_end && j0 + box_rows > k_begin) {
        const int logical = j0 / page_size;
        page = logical < table_width ? table_row[logical] : -1;
        if (page < 0 || page >= n_pages) {
          if (status) atomicOr(status, FG_STATUS_BAD_PAGE);
          page = -1;
        }
      }
      box_pages[x] = page;
    }
  };
  auto box_page = [&](int t, int i) { return box_pages[(t % tiles_per_fill) * n_boxes + i]; };
  fill_pages(0);
  __syncthreads();
  auto issue = [&](int t) {  // thread 0 only
    const int stage = t & 1;
    int n_valid = 0;
    for (int i = 0; i < n_boxes; ++i) n_valid += box_page(t, i) >= 0;
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    mbar_arrive_expect(&full[stage], 2 * n_valid * box_rows * HD * 2);
    const int slot0 = (k_lo + t * PF_KEYS) % page_size;
    for (int i = 0; i < n_boxes; ++i) {
      const int page = box_page(t, i);
      if (page < 0) continue;
      const int slot = page_size > PF_KEYS ? slot0 : 0;
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        tma_load_5d(Ks + stage * STAGE_BYTES + h * PF_HALF + i * box_rows * 128, &k_map, h * 64, slot, g, page,
                    layer, &full[stage]);
        tma_load_5d(Vs + stage * STAGE_BYTES + h * PF_HALF + i * box_rows * 128, &v_map, h * 64, slot, g, page,
                    layer, &full[stage]);
      }
    }
  };
  // boxes that are not loaded must hold zeros (only at the ends of a request with small pages)
  auto zero_missing = [&](int t) -> bool {
    bool any = false;
    for (int i = 0; i < n_boxes; ++i) {
      if (box_page(t, i) >= 0) continue;
      any = true;
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int h = 0; h < HALVES; ++h)
        for (int c = tid; c < box_rows * 8; c += PF_THREADS) {
          *reinterpret_cast<uint4*>(Ks + (t & 1) * STAGE_BYTES + h * PF_HALF + i * box_rows * 128 + c * 16) = z;
          *reinterpret_cast<uint4*>(Vs + (t & 1) * STAGE_BYTES + h * PF_HALF + i * box_rows * 128 + c * 16) = z;
        }
    }
    return any;
  };
  if (tid == 0) issue(0);

  const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
  const int p0 = row_pos[r0], p1 = row_pos[r1];
  int warp_max = -1, warp_min = 0x7fffffff;
  bool warp_full = true;  // all 16 rows of the warp hold a query
  for (int r = warp * 16; r < warp * 16 + 16; ++r) {
    const int p = row_pos[r];
    warp_max = max(warp_max, p);
    if (p >= 0) warp_min = min(warp_min, p); else warp_full = false;
  }
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk)
    ldmatrix_x4(qf[kk], Qs + (warp * 16 + (lane & 15)) * LD + kk * 16 + ((lane >> 4) << 3));

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  for (int t = 0; t < n_tiles; ++t) {
    // the copy of tile t+1 is issued one tile ahead; where t+1 starts a new stretch of
    // page ids, the stretch is looked up first (tile t's ids are not needed any more:
    // its copy is in flight and its missing boxes are zeroed before the look-up)
    const bool missing = zero_missing(t);
    if ((t + 1) % tiles_per_fill == 0 && t + 1 < n_tiles) {
      __syncthreads();
      fill_pages(t + 1);
      __syncthreads();
    } else if (missing) {
      __syncthreads();
    }
    if (t + 1 < n_tiles && tid == 0) issue(t + 1);  // its stage was released by the barrier below
    mbar_wait(&full[t & 1], (t >> 1) & 1, status, &gave_up);
    const int k0 = k_lo + t * PF_KEYS;
    if (k0 <= warp_max) {
      const unsigned char* ks = Ks + (t & 1) * STAGE_BYTES;
      const unsigned char* vs = Vs + (t & 1) * STAGE_BYTES;
      float s[NT][4];
      qk_product_swz<HD, NT, PF_HALF>(s, qf, ks, 0, lane);
      // only tiles that touch the diagonal, the window's edge or an unused row need the mask
      const bool need_mask = !warp_full || k0 + PF_KEYS - 1 > warp_min ||
                             (window > 0 && k0 <= warp_max - window);
      if (need_mask) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = k0 + nt * 8 + 2 * (lane & 3) + (e & 1);
            const int p = (e < 2) ? p0 : p1;
            const bool vis = p >= 0 && j <= p && (window <= 0 || j > p - window);
            if (!vis) s[nt][e] = -INFINITY;
          }
      }
      softmax_step_raw<HD, NT>(s, o, m, l, scale_log2);
      pv_product_swz<HD, NT, PF_HALF>(o, s, vs, 0, lane);
    }
    __syncthreads();  // everyone is done with this stage before it is refilled
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = h ? r1 : r0;
    if (!row_valid(r)) continue;
    const float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
    __nv_bfloat16* dst = out + (size_t)(tok0 + row_token(r)) * out_stride + (g * group + row_head(r)) * HD;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
      const int d = nt * 8 + 2 * (lane & 3);
      *reinterpret_cast<__nv_bfloat162*>(dst + d) =
          __floats2bfloat162_rn(o[nt][2 * h] * inv, o[nt][2 * h + 1] * inv);
    }
  }
}

}  // namespace fg_tma
