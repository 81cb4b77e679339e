// Paged causal attention for bfloat16 on the tensor cores (mma.sync m16n8k16,
// float32 accumulate), in two kernels that share their building blocks:
//
//  * attention_prefill_kernel: prompt portions.  A block owns 64 query rows
//    (consecutive tokens of one request x the query heads that share one
//    key/value head) and walks the request's keys in tiles of 64 positions,
//    double-buffered with cp.async, with the online softmax of the flash
//    attention scheme.
//  * attention_decode_kernel: single tokens.  A block owns one (request,
//    key/value head, split of 128 key positions); its 4 warps take 32 positions
//    each and merge; partial (max, sum, output) go to scratch and
//    attention_combine_kernel merges the splits.  A split always covers
//    positions [128 s, 128 s + 128), whatever else is in the batch.
//
// Semantics as in attention_simt.cuh (fastgen/forward.py:176-258): scores
// q.k * scale over positions j <= pos (and j > pos - window), softmax and the
// running maximum / sum / output in float32 (exp2f on log2e-scaled scores),
// probabilities rounded to bfloat16 for the second product, as the tensor core
// needs.  Keys and values are read from pages laid out [page, kv_head, slot, HD].
#pragma once

#include "common.cuh"

namespace fg_mma {

constexpr int THREADS = 128;
constexpr int PREFILL_ROWS = 64;
constexpr int PREFILL_KEYS = 64;
constexpr int DECODE_SPLIT = 128;  // key positions per split
constexpr int DECODE_ROWS = 16;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool pred) {
  const int bytes = pred ? 16 : 0;  // 0: the 16 bytes are zero-filled, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Shared-memory tiles have rows of HD + 8 bf16: the 16-byte pad makes the
// 8 rows of an ldmatrix fall into distinct banks for every HD multiple of 16.
template <int HD>
struct Tile {
  static constexpr int LD = HD + 8;
};

// Offsets (in elements, -1 = no such row) of the key/value rows k0 .. k0+rows-1 of
// a request in its pools: one page look-up (a division) per row, done by `rows`
// threads.  Rows outside [k_begin, k_end) or without a page get -1.
template <int HD>
__device__ __forceinline__ void kv_row_offsets(long long* row_off, const int* __restrict__ table_row,
                                               int table_width, int page_size, int n_pages, int n_kv_heads,
                                               int g, int k0, int rows, int k_begin, int k_end, int tid,
                                               int* status) {
  if (tid < rows) {
    const int j = k0 + tid;
    long long off = -1;
    if (j >= k_begin && j < k_end) {
      const int logical = j / page_size;
      const int page = logical < table_width ? table_row[logical] : -1;
      if (page >= 0 && page < n_pages)
        off = (((long long)page * n_kv_heads + g) * page_size + (j - logical * page_size)) * HD;
      else if (status)
        atomicOr(status, FG_STATUS_BAD_PAGE);
    }
    row_off[tid] = off;
  }
}

// Bring `rows` rows into shared memory with 16-byte asynchronous copies;
// consecutive threads take consecutive pieces of a row.  Rows with offset -1 are
// zero-filled.
template <int HD>
__device__ __forceinline__ void load_kv_rows(__nv_bfloat16* dst, const __nv_bfloat16* __restrict__ pages,
                                             const long long* row_off, int rows, int tid, int nthreads) {
  constexpr int CH = HD / 8;  // 16-byte pieces per row
  for (int i = tid; i < rows * CH; i += nthreads) {
    const int r = i / CH, c = i - r * CH;
    const long long off = row_off[r];
    cp_async_16(dst + r * Tile<HD>::LD + c * 8, off >= 0 ? pages + off + c * 8 : pages, off >= 0);
  }
}

// S[16 x NK*8] += Q[16 x HD] K^T for one warp; K rows start at `ks`.
template <int HD, int NT>
__device__ __forceinline__ void qk_product(float (&s)[NT][4], const uint32_t (&qf)[HD / 16][4],
                                           const __nv_bfloat16* ks, int lane) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      const int key = np * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int dim = kk * 16 + (((lane >> 3) & 1) << 3);
      ldmatrix_x4(b, ks + key * Tile<HD>::LD + dim);
      mma_16816(s[2 * np], qf[kk], b[0], b[1]);
      mma_16816(s[2 * np + 1], qf[kk], b[2], b[3]);
    }
  }
}

// O[16 x HD] += P[16 x NT*8] V for one warp; V rows start at `vs`.
template <int HD, int NT>
__device__ __forceinline__ void pv_product(float (&o)[HD / 8][4], const float (&p)[NT][4],
                                           const __nv_bfloat16* vs, int lane) {
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
    a[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
    a[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
    a[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
    for (int np = 0; np < HD / 16; ++np) {
      uint32_t b[4];
      const int key = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int dim = np * 16 + ((lane >> 4) << 3);
      ldmatrix_x4_trans(b, vs + key * Tile<HD>::LD + dim);
      mma_16816(o[2 * np], a, b[0], b[1]);
      mma_16816(o[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// One online-softmax step on a warp's S tile.  s holds scores already multiplied
// by scale*log2(e) and masked with -inf; m/l are the running max and sum of the
// thread's two rows (lane/4 and lane/4+8).  On return s holds the probabilities.
template <int HD, int NT>
__device__ __forceinline__ void softmax_step(float (&s)[NT][4], float (&o)[HD / 8][4], float (&m)[2],
                                             float (&l)[2]) {
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
      alpha = (m[h] == -INFINITY) ? 0.f : exp2f(m[h] - m_new);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        // the probabilities are rounded to bfloat16 for the product; sum what is used
        const float p0 = __bfloat162float(__float2bfloat16_rn(exp2f(s[nt][2 * h] - m_new)));
        const float p1 = __bfloat162float(__float2bfloat16_rn(exp2f(s[nt][2 * h + 1] - m_new)));
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

// ---------------------------------------------------------------------------------
// prefill
// ---------------------------------------------------------------------------------
template <int HD>
constexpr size_t prefill_smem_bytes() {
  return sizeof(__nv_bfloat16) * Tile<HD>::LD * (PREFILL_ROWS + 4 * PREFILL_KEYS);
}

template <int HD>
__global__ void __launch_bounds__(THREADS)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                         int out_stride, const __nv_bfloat16* __restrict__ k_pages,
                         const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_table,
                         int table_width, int page_size, int n_pages, const int* __restrict__ pos,
                         const int* __restrict__ tile_req, const int* __restrict__ tile_tok0,
                         const int* __restrict__ tile_ntok, int n_kv_heads, int group, int heads_per_block,
                         int window, float scale_log2, int* status) {
  constexpr int LD = Tile<HD>::LD;
  constexpr int NT = PREFILL_KEYS / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Ks = Qs + PREFILL_ROWS * LD;            // 2 stages
  __nv_bfloat16* Vs = Ks + 2 * PREFILL_KEYS * LD;        // 2 stages
  __shared__ int row_pos[PREFILL_ROWS];
  __shared__ long long row_off[2][PREFILL_KEYS];

  const int tile = blockIdx.x, g = blockIdx.y, sub = blockIdx.z;
  const int b = tile_req[tile];
  const int tok0 = tile_tok0[tile], ntok = tile_ntok[tile];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  auto row_token = [&](int r) { return r / heads_per_block; };
  auto row_head = [&](int r) { return sub * heads_per_block + (r % heads_per_block); };
  auto row_valid = [&](int r) { return row_token(r) < ntok && row_head(r) < group; };

  if (b < 0) return;  // prompt portions are never padding
  if (tid < PREFILL_ROWS) row_pos[tid] = row_valid(tid) ? pos[tok0 + row_token(tid)] : -1;
  // queries -> shared memory (zero rows where the tile is not full)
  constexpr int CH = HD / 8;
  for (int i = tid; i < PREFILL_ROWS * CH; i += THREADS) {
    const int r = i / CH, c = i - r * CH;
    const bool ok = row_valid(r);
    const __nv_bfloat16* src =
        ok ? q + (size_t)(tok0 + row_token(r)) * q_stride + (g * group + row_head(r)) * HD + c * 8 : q;
    cp_async_16(Qs + r * LD + c * 8, src, ok);
  }
  cp_async_commit();
  __syncthreads();
  int max_pos = -1, min_pos = 0x7fffffff;
  {
    // rows are ordered by token, so the extremes sit at the ends of the valid rows
    for (int r = 0; r < PREFILL_ROWS; r += heads_per_block) {
      const int p = row_pos[r];
      if (p >= 0) {
        max_pos = max(max_pos, p);
        min_pos = min(min_pos, p);
      }
    }
  }
  if (max_pos < 0) {
    cp_async_wait<0>();
    return;
  }
  const int k_lo = window > 0 ? max(0, min_pos - window + 1) / PREFILL_KEYS * PREFILL_KEYS : 0;
  const int k_begin = window > 0 ? max(0, min_pos - window + 1) : 0;
  const int k_end = max_pos + 1;
  const int* table_row = block_table + (size_t)b * table_width;
  const int n_tiles = (k_end - k_lo + PREFILL_KEYS - 1) / PREFILL_KEYS;

  // offsets of tile t's rows are computed one tile ahead of its copies
  auto offsets = [&](int t) {
    kv_row_offsets<HD>(row_off[t & 1], table_row, table_width, page_size, n_pages, n_kv_heads, g,
                       k_lo + t * PREFILL_KEYS, PREFILL_KEYS, k_begin, k_end, tid, status);
  };
  auto issue = [&](int t) {
    const int stage = t & 1;
    load_kv_rows<HD>(Ks + stage * PREFILL_KEYS * LD, k_pages, row_off[stage], PREFILL_KEYS, tid, THREADS);
    load_kv_rows<HD>(Vs + stage * PREFILL_KEYS * LD, v_pages, row_off[stage], PREFILL_KEYS, tid, THREADS);
    cp_async_commit();
  };
  offsets(0);
  __syncthreads();
  issue(0);
  if (n_tiles > 1) offsets(1);

  // the warp's 16 rows; this thread's two rows
  const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
  const int p0 = row_pos[r0], p1 = row_pos[r1];
  int warp_max = -1;
  for (int r = warp * 16; r < warp * 16 + 16; ++r) warp_max = max(warp_max, row_pos[r]);

  cp_async_wait<1>();  // queries have landed
  __syncthreads();
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk)
    ldmatrix_x4(qf[kk], Qs + (warp * 16 + (lane & 15)) * LD + kk * 16 + ((lane >> 4) << 3));

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  for (int t = 0; t < n_tiles; ++t) {
    if (t + 1 < n_tiles) {
      issue(t + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // tile t's rows have landed and its offsets are no longer needed
    if (t + 2 < n_tiles) offsets(t + 2);
    const int k0 = k_lo + t * PREFILL_KEYS;
    if (k0 <= warp_max) {
      const __nv_bfloat16* ks = Ks + (t & 1) * PREFILL_KEYS * LD;
      const __nv_bfloat16* vs = Vs + (t & 1) * PREFILL_KEYS * LD;
      float s[NT][4];
      qk_product<HD, NT>(s, qf, ks, lane);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = k0 + nt * 8 + 2 * (lane & 3) + (e & 1);
          const int p = (e < 2) ? p0 : p1;
          const bool vis = p >= 0 && j <= p && (window <= 0 || j > p - window);
          s[nt][e] = vis ? s[nt][e] * scale_log2 : -INFINITY;
        }
      }
      softmax_step<HD, NT>(s, o, m, l);
      pv_product<HD, NT>(o, s, vs, lane);
    }
    __syncthreads();  // everyone is done with this stage before it is refilled
  }

  // O / l -> out
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

// ---------------------------------------------------------------------------------
// decode: split over key positions, then combine
// ---------------------------------------------------------------------------------
// Bulk asynchronous copies (the TMA engine, untiled form) tracked by an mbarrier.
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::);
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect(uint64_t* bar, int bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// 16-byte aligned source and destination, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, int bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// Bounded wait.  It gives up after `limit` polls, ORs FG_STATUS_WAIT_TIMEOUT into the status
// word and sets `*gave_up`, a flag in the block's shared memory (zero at the block's start).
// Once the flag is set every other wait of the block that is given the flag returns false
// at its next poll instead of counting to the limit itself: a block whose copies or
// products never arrive loses the time of one wait, runs through the rest of its loops on
// whatever its buffers hold (the status word tells the host that the step's results are void),
// and returns.  No control flow depends on the flag, so named barriers stay matched.
//
// A parity wait can only tell "this phase is over" from "not yet" while the waiter is less
// than two completions behind the barrier: a barrier must not complete a second time before
// a waiter of the first completion has looked (give every stage a barrier of its own).
constexpr int MBAR_WAIT_POLLS = 1 << 22;

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, int parity) {
  uint32_t done;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, int parity, int* status, int* gave_up = nullptr,
                                          int limit = MBAR_WAIT_POLLS) {
  if (mbar_try_wait(bar, parity)) return true;  // the usual case costs what it did without the flag
  for (int it = 1; it < limit; ++it) {
    if (gave_up != nullptr && *reinterpret_cast<volatile int*>(gave_up) != 0) return false;
    if (mbar_try_wait(bar, parity)) return true;
  }
  if (gave_up != nullptr) *reinterpret_cast<volatile int*>(gave_up) = 1;
  if (status) atomicOr(status, FG_STATUS_WAIT_TIMEOUT);
  return false;
}

template <int HD>
constexpr size_t decode_smem_bytes() {
  // K and V of the split and the padded queries; the merge buffers reuse K's space
  return sizeof(__nv_bfloat16) * Tile<HD>::LD * (2 * DECODE_SPLIT + DECODE_ROWS);
}

// scratch layout per (token, head, split): HD floats of output, then (max, sum)
template <int HD>
__host__ __device__ constexpr int part_stride() { return HD + 2; }

template <int HD>
__global__ void __launch_bounds__(THREADS)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                        const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                        const int* __restrict__ block_table, int table_width, int page_size, int n_pages,
                        const int* __restrict__ pos, const int* __restrict__ seq_req,
                        const int* __restrict__ seq_tok, int n_heads, int n_kv_heads, int group,
                        int window, float scale_log2, float* __restrict__ scratch, int max_splits,
                        int* status) {
  static_assert(THREADS >= DECODE_SPLIT, "one thread per key position computes its row offset");
  constexpr int LD = Tile<HD>::LD;
  constexpr int NT = 4;  // 32 key positions per warp
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Vs = Ks + DECODE_SPLIT * LD;
  __nv_bfloat16* Qs = Vs + DECODE_SPLIT * LD;
  __shared__ long long row_off[DECODE_SPLIT];

  const int split = blockIdx.x, g = blockIdx.y, seq = blockIdx.z;
  const int b = seq_req[seq];
  if (b < 0) return;  // padding lane of a fixed-size batch
  const int tok = seq_tok[seq];
  const int p = pos[tok];
  const int k0 = split * DECODE_SPLIT;
  if (k0 > p) return;  // this split lies beyond the request's keys
  const int k_begin = window > 0 ? max(0, p - window + 1) : 0;
  if (k0 + DECODE_SPLIT <= k_begin) return;  // wholly before the window
  const int k_end = p + 1;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  kv_row_offsets<HD>(row_off, block_table + (size_t)b * table_width, table_width, page_size, n_pages,
                     n_kv_heads, g, k0, DECODE_SPLIT, k_begin, k_end, tid, status);
  __syncthreads();
  load_kv_rows<HD>(Ks, k_pages, row_off, DECODE_SPLIT, tid, THREADS);
  cp_async_commit();
  load_kv_rows<HD>(Vs, v_pages, row_off, DECODE_SPLIT, tid, THREADS);
  cp_async_commit();

  constexpr int CH = HD / 8;
  for (int sub = 0; sub * DECODE_ROWS < group; ++sub) {
    // groups wider than 16 heads are walked in slices of 16; K and V stay in place
    const int rows_here = min(DECODE_ROWS, group - sub * DECODE_ROWS);
    if (sub > 0) __syncthreads();
    for (int i = tid; i < DECODE_ROWS * CH; i += THREADS) {
      const int r = i / CH, c = i - r * CH;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < rows_here)
        v = *reinterpret_cast<const uint4*>(q + (size_t)tok * q_stride +
                                            (g * group + sub * DECODE_ROWS + r) * HD + c * 8);
      *reinterpret_cast<uint4*>(Qs + r * LD + c * 8) = v;
    }
    __syncthreads();
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk)
      ldmatrix_x4(qf[kk], Qs + (lane & 15) * LD + kk * 16 + ((lane >> 4) << 3));

    if (sub == 0) {
      cp_async_wait<1>();  // keys
      __syncthreads();
    }
    float s[NT][4];
    qk_product<HD, NT>(s, qf, Ks + warp * 32 * LD, lane);
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
    if (sub == 0) {
      cp_async_wait<0>();  // values
      __syncthreads();
    }
    pv_product<HD, NT>(o, s, Vs + warp * 32 * LD, lane);

    // merge the 4 warps through shared memory (only the rows that hold heads)
    float* wm = reinterpret_cast<float*>(Qs);           // [4][16] max, then [4][16] sum: fits the Q tile
    float* wl = wm + 4 * DECODE_ROWS;
    __syncthreads();                                    // all warps are done with Q and K
    float* wo = reinterpret_cast<float*>(Ks);           // [4][rows][HD]
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
      if (r0 < rows_here)
        *reinterpret_cast<float2*>(wo + (warp * DECODE_ROWS + r0) * HD + d) = make_float2(o[nt][0], o[nt][1]);
      if (r0 + 8 < rows_here)
        *reinterpret_cast<float2*>(wo + (warp * DECODE_ROWS + r0 + 8) * HD + d) = make_float2(o[nt][2], o[nt][3]);
    }
    __syncthreads();
    for (int i = tid; i < rows_here * HD; i += THREADS) {
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
      const int head = g * group + sub * DECODE_ROWS + r;
      float* dst = scratch + (((size_t)seq * n_heads + head) * max_splits + split) * part_stride<HD>();
      dst[d] = acc;
      if (d == 0) {
        dst[HD] = mm;
        dst[HD + 1] = ll;
      }
    }
    if ((sub + 1) * DECODE_ROWS < group) {
      // K's space was used for the merge: bring the keys back for the next slice of heads
      __syncthreads();
      load_kv_rows<HD>(Ks, k_pages, row_off, DECODE_SPLIT, tid, THREADS);
      cp_async_commit();
      cp_async_wait<0>();
    }
  }
}

// out[token, head, :] = sum_s o_s * 2^(m_s - m) / sum_s l_s * 2^(m_s - m) over the
// request's splits.  One block of COMBINE_THREADS per (head, token): warp w sums the splits
// s_lo + w, s_lo + w + W, ... (a lane holds two neighbouring dimensions of every 64), then the
// warps' sums are added in ascending warp order.  The order of the additions depends on the
// request's own splits only, never on the batch.
constexpr int COMBINE_THREADS = 256;

template <int HD>
__global__ void __launch_bounds__(COMBINE_THREADS)
attention_combine_kernel(const float* scratch, __nv_bfloat16* __restrict__ out, int out_stride,
                         const int* __restrict__ pos, const int* __restrict__ seq_req,
                         const int* __restrict__ seq_tok, int n_heads, int window, int max_splits,
                         const int* first_pair, int* status) {
  // first_pair (written by the kernel before, so no __restrict__): null, or for every
  // request the number of (request, split) pairs before it; the partials are then
  // numbered [pair][head] (only the splits that exist), else [request][head][split].
  constexpr int WARPS = COMBINE_THREADS / 32;
  constexpr int NV = (HD + 63) / 64;  // float2 pieces a lane holds
  constexpr int PS = part_stride<HD>();
  static_assert(PS % 2 == 0, "partials are read as float2");
  __shared__ float red[WARPS];
  __shared__ float acc_s[WARPS][NV * 64];
  __shared__ float ll_s[WARPS];
  pdl_trigger();
  // the lists of sequences and positions are inputs of the step: read while the kernel before
  // this one finishes; its partials (and first_pair) are touched after the wait
  const int seq = blockIdx.y, head = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tok = seq_tok[seq];
  const int request = seq_req[seq];
  const int p = request < 0 ? 0 : pos[tok];
  pdl_wait();
  __nv_bfloat16* dst = out + (size_t)tok * out_stride + head * HD;
  // a padding lane has no request: nothing is written for it (its token index may be any row,
  // also one that belongs to a request of the step)
  if (request < 0) return;
  const int s_lo = window > 0 ? max(0, p - window + 1) / DECODE_SPLIT : 0;
  int s_hi = p / DECODE_SPLIT;  // inclusive
  if (s_hi >= max_splits) {
    // the launch was sized for shorter requests: report instead of reading past the scratch
    if (tid == 0 && status) atomicOr(status, FG_STATUS_BAD_SPLITS);
    s_hi = max_splits - 1;
  }
  // base[s * step]: the partial of split s
  const size_t step = first_pair != nullptr ? (size_t)n_heads * PS : PS;
  const float* base = first_pair != nullptr
                          ? scratch + ((size_t)(first_pair[seq] - s_lo) * n_heads + head) * PS
                          : scratch + ((size_t)seq * n_heads + head) * max_splits * PS;
  // the overall maximum
  float mm = -INFINITY;
  for (int s = s_lo + tid; s <= s_hi; s += COMBINE_THREADS) mm = fmaxf(mm, base[(size_t)s * step + HD]);
  mm = warp_max(mm);
  if (lane == 0) red[warp] = mm;
  __syncthreads();
  mm = red[0];
#pragma unroll
  for (int w = 1; w < WARPS; ++w) mm = fmaxf(mm, red[w]);
  // this warp's splits
  float2 acc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) acc[i] = make_float2(0.f, 0.f);
  float ll = 0.f;
#pragma unroll 4
  for (int s = s_lo + warp; s <= s_hi; s += WARPS) {
    const float* part = base + (size_t)s * step;
    const float ms = part[HD];
    const float wgt = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
    ll += wgt * part[HD + 1];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = i * 64 + lane * 2;
      if (d < HD) {
        const float2 v = *reinterpret_cast<const float2*>(part + d);
        acc[i].x += wgt * v.x;
        acc[i].y += wgt * v.y;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    acc_s[warp][i * 64 + lane * 2] = acc[i].x;
    acc_s[warp][i * 64 + lane * 2 + 1] = acc[i].y;
  }
  if (lane == 0) ll_s[warp] = ll;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) total += ll_s[w];
  const float inv = total > 0.f ? 1.f / total : 0.f;
  for (int d = tid; d < HD; d += COMBINE_THREADS) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) a += acc_s[w][d];
    dst[d] = __float2bfloat16_rn(a * inv);
  }
}

}  // namespace fg_mma
