// Prompt attention for bfloat16 on the 5th-generation tensor cores:
// tcgen05.mma issued by one thread, operands in 128-byte-swizzled shared memory
// (keys and values brought by TMA straight into the operand layout), the scores
// S and the output O accumulated in tensor memory (TMEM).
//
// A block owns 128 query rows (consecutive tokens of one request x the query
// heads of one key/value head) and walks the request's keys in tiles of 64:
//
//   load warp:      TMA(K_t, V_t) into stage t & 1 as soon as S_{t-2} / O_{t-2} are done
//   MMA warp:       S_{t+1} = Q K_{t+1}^T  (tcgen05.mma, M128 N64 K16 x HD/16, one thread)
//   4 softmax warps: S_t from TMEM (one row a thread: no shuffles for max and sum),
//                    p = 2^((s - m) c),  P_t (bf16) back into TMEM over S_t's columns
//   MMA warp:       O += P_t V_t      (tcgen05.mma with A from TMEM, M128 N=HD K16 x 4)
//
// The warps only meet at mbarriers (scores ready, probabilities ready, output
// done), so the tensor core computes S_{t+1} and O_t while the softmax warps are
// busy with the exponentials, and two blocks share an SM.  The running maximum is only raised when a row's maximum grew by
// more than 2^8 (the accumulated O is then rescaled in TMEM), which is exact:
// m is just the reference point of the exponent.
//
// Semantics as in the other attention kernels (fastgen/forward.py:176-258):
// float32 scores, maximum, sum and output; probabilities rounded to bfloat16 for
// the second product.  Waits on mbarriers are bounded.
//
// Needs head size 64 or 128, pages of a power of two >= 8 slots.
#pragma once

#include <cuda.h>

#include "attention_tma.cuh"
#include "tc5_primitives.cuh"

namespace fg_tc5 {

using namespace fg_mma;
using fg_tma::tma_load_5d;

constexpr int ROWS = 128;     // query rows a block
constexpr int KEYS = 64;      // key positions a tile
constexpr int SOFTMAX_THREADS = 128;
constexpr int THREADS = 192;  // 4 softmax warps, a load warp, an MMA warp
constexpr int LOAD_WARP = 4, MMA_WARP = 5;
constexpr int KV_HALF = KEYS * 128;   // bytes of one 64-element half of a K or V tile
constexpr int Q_HALF = ROWS * 128;    // ... of the Q tile
constexpr float RESCALE_THRESHOLD = 8.f;  // in units of log2
constexpr int SPLIT_MIN_TILES = 8;        // fewest key tiles of a part of a split item
constexpr int MAX_PARTS = 16;             // most parts of an item (one block adds them up)

// 2^x as the special-function unit gives it (relative error about 2^-22, results below
// 2^-126 flushed to zero): the probabilities are rounded to bfloat16 right after, and
// exp2f()'s extra range handling would cost three more instructions an element.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// maximum of three in one instruction (sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// ---- two float32 values in one 64-bit register: the packed arithmetic of sm_100 ----
__device__ __forceinline__ uint64_t f32x2(float lo, float hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void f32x2_split(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

template <int HD>
constexpr size_t smem_bytes() {
  // Q and two stages of K and V; plus alignment slack
  return (size_t)ROWS * HD * 2 + 2 * 2 * (size_t)KEYS * HD * 2 + 1024;
}
constexpr int TMEM_COLS = 256;  // S0, S1 (64 columns each; P overwrites its S) + O (HD <= 128)

// How a launch hands its work out.  `real_tiles` (null: all of them) points at the number of
// tiles at the end of the tile list that are real; a captured graph's list has padding entries
// in front of them, their number changes from replay to replay, and the host cannot choose the
// number of parts a launch ahead.  The kernel then chooses it: as many as the launch's blocks
// allow, given the real items, and the partials have room for.
struct HandOut {
  int n_real;  // tiles that are handed out, the last ones of the list
  int parts;   // draws an item
};
__device__ __forceinline__ HandOut hand_out(const int* real_tiles, int n_tiles_total, int n_kv_heads, int n_subs,
                                            int parts_given, int main_grid, int split_slots, bool split) {
  HandOut h;
  h.n_real = n_tiles_total;
  h.parts = split ? parts_given : 1;
  if (real_tiles) {
    h.n_real = min(max((int)ld_global_4(real_tiles), 0), n_tiles_total);
    if (split) {
      const long long items = (long long)h.n_real * n_kv_heads * n_subs;
      h.parts = items > 0 ? (int)min((long long)MAX_PARTS, max(1ll, main_grid / items)) : 1;
      if (items * h.parts > split_slots) h.parts = 1;
    }
  }
  return h;
}

// The partial of one part of a split item: this thread's row of O (tensor memory, unnormalised),
// its reference maximum (in units of log2) and its row sum, to [column][row] in `slot` (which
// already points at the row), so that a warp's rows are neighbours.  Not inlined: the kernel's
// main loop is sensitive to what the compiler makes of the code around it.
template <int HD>
__device__ __noinline__ void write_partial(uint32_t o_addr, float* slot, float m, float l) {
#pragma unroll
  for (int cc = 0; cc < HD / 32; ++cc) {
    float o[32];
    tmem_ld32(o_addr + cc * 32, o);
#pragma unroll
    for (int i = 0; i < 32; ++i) __stcg(slot + (size_t)(cc * 32 + i) * ROWS, o[i]);
  }
  __stcg(slot + (size_t)HD * ROWS, m);
  __stcg(slot + (size_t)(HD + 1) * ROWS, l);
}

// This thread's row of a split item: the parts' partials, weighed by their reference maxima
// and summed in the order of the parts, normalised, to `dst` (the row's output).  `slots`
// points at the row in the first part's partial.
template <int HD>
__device__ __noinline__ void merge_parts(const float* slots, int n_parts, __nv_bfloat16* dst, bool valid) {
  constexpr size_t SLOT = (size_t)ROWS * (HD + 2);
  float m_all = -INFINITY;
  for (int p = 0; p < n_parts; ++p) m_all = fmaxf(m_all, __ldcg(slots + p * SLOT + (size_t)HD * ROWS));
  // the weight of part p (a part that saw no key has -inf and weighs nothing)
  auto weight = [&](int p) {
    const float m_p = __ldcg(slots + p * SLOT + (size_t)HD * ROWS);
    return m_p == -INFINITY ? 0.f : exp2f(m_p - m_all);
  };
  float l_all = 0.f;
  for (int p = 0; p < n_parts; ++p) l_all += __ldcg(slots + p * SLOT + (size_t)(HD + 1) * ROWS) * weight(p);
  const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
#pragma unroll 1
  for (int cc = 0; cc < HD / 16; ++cc) {
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
#pragma unroll 2
    for (int p = 0; p < n_parts; ++p) {
      const float w = weight(p) * inv;
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] += __ldcg(slots + p * SLOT + (size_t)(cc * 16 + i) * ROWS) * w;
    }
    if (valid) {
#pragma unroll
      for (int i = 0; i < 16; i += 8) {
        uint4 v;
        v.x = pack_bf16(acc[i], acc[i + 1]);
        v.y = pack_bf16(acc[i + 2], acc[i + 3]);
        v.z = pack_bf16(acc[i + 4], acc[i + 5]);
        v.w = pack_bf16(acc[i + 6], acc[i + 7]);
        *reinterpret_cast<uint4*>(dst + cc * 16 + i) = v;
      }
    }
  }
}

// SPLIT: the instantiation for launches that work on long items in parts (`parts` > 1); the
// other one has none of that code (its main loop proved sensitive to it: head size 64 ran 5 %
// slower with it).
template <int HD, bool SPLIT>
__global__ void __launch_bounds__(THREADS, 2)
attention_prefill_tc5_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                             int layer, const __nv_bfloat16* __restrict__ q, int q_stride,
                             __nv_bfloat16* __restrict__ out, int out_stride, const int* __restrict__ block_table,
                             int table_width, int page_size, int n_pages, const int* __restrict__ pos,
                             const int* __restrict__ tile_req, const int* __restrict__ tile_tok0,
                             const int* __restrict__ tile_ntok, int n_tiles_total, int n_kv_heads, int group,
                             int heads_per_block, int window, float scale_log2, unsigned int* work_counter,
                             int parts, float* split_scratch, int* split_flags, int split_slots,
                             const int* real_tiles, int* status) {
  static_assert(HD == 64 || HD == 128, "head sizes 64 and 128");
  constexpr int HALVES = HD / 64;
  constexpr int STAGE_BYTES = HALVES * KV_HALF;
  constexpr uint32_t IDESC_S = instr_desc(KEYS, false);
  constexpr uint32_t IDESC_O = instr_desc(HD, true);
  constexpr int COL_S0 = 0, COL_O = 2 * KEYS;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  unsigned char* Qs = smem;                         // [HALVES][128 rows][128 B]
  unsigned char* Ks = Qs + HALVES * Q_HALF;         // [2][HALVES][64 rows][128 B]
  unsigned char* Vs = Ks + 2 * STAGE_BYTES;
  // full_k/full_v: a tile's keys/values have landed; s_done: its scores are in TMEM;
  // p_ready: all 128 softmax threads stored its probabilities; o_done: its P V is done.
  // Every barrier completes once a key tile, and the block counts its key tiles through
  // all the work it takes (`base` below): stage and parity follow that running number.
  // drained: used once, at the end of a block one of whose waits ran out.
  __shared__ __align__(8) uint64_t full_k[2], full_v[2], s_done[2], p_ready[2], o_done[2], drained;
  __shared__ uint32_t tmem_base_s;
  __shared__ unsigned int work_s;
  __shared__ int gave_up;  // set by a wait that ran out: the waits after it return at once (see mbar_wait)
  __shared__ int first_pos_s;
  __shared__ int split_order_s;  // of a split item: how many of its parts were through before this one
  constexpr int PAGE_STAGE = 256;
  __shared__ int box_pages[PAGE_STAGE];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool softmax_thread = tid < SOFTMAX_THREADS;

  // Tensor memory first: while a block holds the allocation permit no other block of the
  // kernel starts on its SM.
  if (warp == LOAD_WARP) {
    tmem_alloc(&tmem_base_s, TMEM_COLS);
    tmem_relinquish();
  }
  if (tid == SOFTMAX_THREADS) {
    gave_up = 0;
    mbar_init(&full_k[0], 1);
    mbar_init(&full_k[1], 1);
    mbar_init(&full_v[0], 1);
    mbar_init(&full_v[1], 1);
    mbar_init(&s_done[0], 1);
    mbar_init(&s_done[1], 1);
    // two of them: a softmax warp may be one tile ahead of another
    mbar_init(&p_ready[0], SOFTMAX_THREADS);
    mbar_init(&p_ready[1], SOFTMAX_THREADS);
    // one for the tiles of each parity: a waiter of O_t's completion can then never be two
    // completions behind (the next one, O_{t+2}'s, needs that waiter's own work)
    mbar_init(&o_done[0], 1);
    mbar_init(&o_done[1], 1);
    mbar_init(&drained, 1);
    mbar_fence_init();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;

  // Work = (query tile, key/value head, slice of the group's heads).  The blocks of the
  // launch (two an SM) take the first items by their index and draw the rest from a
  // counter: a block that started a new tile list entry only when another block of the
  // launch had ended would wait for its SM to drain.  The list is in ascending order of
  // work and is handed out from its end with the heads running fastest, so the longest
  // items start first and the short ones fill the tail.
  //
  // A launch of fewer items than resident blocks would leave SMs idle and be bound by its
  // longest item.  With `parts` > 1 every item is `parts` draws that follow each other in the
  // hand-out: an item of many key tiles is worked on in up to `parts` stretches of at least
  // SPLIT_MIN_TILES tiles (the draws beyond that do nothing).  Every part of such an item
  // leaves its unnormalised O, its reference maximum and its row sums in `split_scratch`,
  // and counts itself in `split_flags` (two ints an item: the parts that are through, zero
  // between launches, and the number of parts of the item in the last launch that split, for
  // tests to read); the part that counts last adds the partials up.
  const unsigned int n_subs = (group + heads_per_block - 1) / heads_per_block;
  const HandOut ho = hand_out(real_tiles, n_tiles_total, n_kv_heads, n_subs, parts, gridDim.x, split_slots, SPLIT);
  const int n_real = ho.n_real;
  parts = ho.parts;
  const unsigned int total_work = (unsigned int)n_real * n_kv_heads * n_subs * parts;
  const unsigned int last_draw = (total_work > gridDim.x ? total_work - gridDim.x : 0u) + gridDim.x - 1;
  int base = 0;  // key tiles this block has been through before the current item
  bool dead = false;  // a wait of this block ran out during an earlier item

  for (unsigned int work = blockIdx.x; work < total_work;) {
    const int part = SPLIT ? work % parts : 0;
    const unsigned int item = SPLIT ? work / parts : work;
    const int g = item % n_kv_heads;
    const int tile = n_tiles_total - 1 - (int)((item / n_kv_heads) % n_real);
    const int sub = item / n_kv_heads / n_real;
    const int b = tile_req[tile];
    const int tok0 = tile_tok0[tile], ntok = tile_ntok[tile];
    int n_tiles = 0;

    // (uniform over the block; after a wait ran out the block only draws its items, so that
    // the counter still returns to zero)
    if (b >= 0 && !dead) {
      auto row_token = [&](int r) { return r / heads_per_block; };
      auto row_head = [&](int r) { return sub * heads_per_block + (r % heads_per_block); };
      auto row_valid = [&](int r) { return row_token(r) < ntok && row_head(r) < group; };

      bool my_valid = false;
      int my_pos = -1;
      // the softmax threads' rows: their positions, and the queries -> shared memory in the
      // K-major operand layout (16-byte pieces, swizzled)
      auto stage_queries = [&]() {
        if (softmax_thread) {
          my_valid = row_valid(tid);
          my_pos = my_valid ? pos[tok0 + row_token(tid)] : -1;
          if (tid == 0) first_pos_s = my_pos;
          const __nv_bfloat16* src =
              q + (size_t)(tok0 + row_token(tid)) * q_stride + (g * group + row_head(tid)) * HD;
#pragma unroll
          for (int c = 0; c < HD / 8; ++c) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (my_valid) v = *reinterpret_cast<const uint4*>(src + c * 8);
            *reinterpret_cast<uint4*>(Qs + (c / 8) * Q_HALF + fg_tma::swz(tid, c % 8)) = v;
          }
          fence_async_smem();  // written by ordinary stores, read by the tensor core
        }
        __syncthreads();
      };
      // a draw of a launch in parts first sees whether it has key tiles at all
      if (!SPLIT) stage_queries();
      const int min_pos = SPLIT ? pos[tok0] : first_pos_s;  // tokens of a tile are consecutive positions
      const int max_pos = min_pos + ntok - 1;
      const int k_begin = window > 0 ? max(0, min_pos - window + 1) : 0;
      const int k_end = max_pos + 1;
      const int item_tiles = (k_end - k_begin / KEYS * KEYS + KEYS - 1) / KEYS;
      // this part's key tiles: the item's are cut into stretches of equal length, at most `parts`
      // of them (fewer where the rounded-up length leaves nothing for the last ones)
      const int most_parts = SPLIT ? max(1, min(parts, item_tiles / SPLIT_MIN_TILES)) : 1;
      const int tiles_per_part = (item_tiles + most_parts - 1) / most_parts;
      const int n_parts = SPLIT ? (item_tiles + tiles_per_part - 1) / tiles_per_part : 1;
      const int first_tile = part * tiles_per_part;
      n_tiles = SPLIT ? max(0, min(tiles_per_part, item_tiles - first_tile)) : item_tiles;
      const bool split = SPLIT && n_parts > 1;
      const int k_lo = k_begin / KEYS * KEYS + first_tile * KEYS;
      if (SPLIT && parts > 1 && part == 0 && tid == 0) split_flags[2 * item + 1] = split ? n_parts : 0;
      if (SPLIT && n_tiles > 0) stage_queries();  // (uniform over the block)

      if (n_tiles == 0) {
        // (nothing: the item has fewer parts than the launch gives every item)
      } else if (warp == LOAD_WARP) {
        // ================================ load warp ================================
        // Keys and values of tile t go to the stage of its running number as soon as that
        // stage is free: the keys' once the S two tiles back is done, the values' once
        // that tile's O is.
        const int* table_row = block_table + (size_t)b * table_width;
        const int box_rows = min(page_size, KEYS);
        const int n_boxes = KEYS / box_rows;
        const int tiles_per_fill = PAGE_STAGE / n_boxes;
        // page ids of a stretch of key tiles, looked up by the warp's 32 lanes
        auto fill_pages = [&](int t_first) {
          const int n = min(tiles_per_fill, n_tiles - t_first) * n_boxes;
          for (int x = lane; x < n; x += 32) {
            const int j0 = k_lo + t_first * KEYS + x * box_rows;
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
          __syncwarp();
        };
        // bring tile t's keys (or values) into its stage; boxes that hold no position of
        // the request are zero-filled instead (a masked probability times garbage could be NaN)
        auto load_tile = [&](int t, const int* pages, bool values) {
          const int stage = (base + t) & 1;
          unsigned char* dst = (values ? Vs : Ks) + stage * STAGE_BYTES;
          uint64_t* bar = values ? &full_v[stage] : &full_k[stage];
          int n_valid = 0;
          for (int i = 0; i < n_boxes; ++i) n_valid += pages[i] >= 0;
          if (n_valid < n_boxes) {
            for (int i = 0; i < n_boxes; ++i) {
              if (pages[i] >= 0) continue;
              const uint4 z = make_uint4(0, 0, 0, 0);
              for (int h = 0; h < HALVES; ++h)
                for (int c = lane; c < box_rows * 8; c += 32)
                  *reinterpret_cast<uint4*>(dst + h * KV_HALF + i * box_rows * 128 + c * 16) = z;
            }
            fence_async_smem();
            __syncwarp();
          }
          if (lane == 0) {
            mbar_arrive_expect(bar, n_valid * box_rows * HD * 2);
            const int slot = (k_lo + t * KEYS) & (page_size - 1) & ~(KEYS - 1);  // 0 unless pages are longer than a tile
            for (int i = 0; i < n_boxes; ++i) {
              const int page = pages[i];
              if (page < 0) continue;
#pragma unroll
              for (int h = 0; h < HALVES; ++h)
                tma_load_5d(dst + h * KV_HALF + i * box_rows * 128, values ? &v_map : &k_map, h * 64, slot, g,
                            page, layer, bar);
            }
          }
          __syncwarp();
        };
        int staged = 0;  // tiles of the staged stretch that were loaded
        if (n_boxes == 1) {
          // pages at least as long as a tile: one box a tile, and one lane does everything
          // between the page look-ups (a single thread's instruction stream is what bounds
          // this warp, so the loop is kept short)
          const uint32_t k_bytes = KEYS * HD * 2;
          for (int t = 0; t < n_tiles; ++t) {
            if (staged == 0) fill_pages(t);
            const int page = box_pages[staged];
            const int gt = base + t, stage = gt & 1;
            if (page >= 0) {
              if (lane == 0) {
                const int slot = (k_lo + t * KEYS) & (page_size - 1);
                unsigned char* kb = Ks + stage * STAGE_BYTES;
                unsigned char* vb = Vs + stage * STAGE_BYTES;
                if (gt >= 2) mbar_wait(&s_done[stage], ((gt - 2) >> 1) & 1, status, &gave_up);
                mbar_arrive_expect(&full_k[stage], k_bytes);
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
                  tma_load_5d(kb + h * KV_HALF, &k_map, h * 64, slot, g, page, layer, &full_k[stage]);
                if (gt >= 2) mbar_wait(&o_done[stage], ((gt - 2) >> 1) & 1, status, &gave_up);
                mbar_arrive_expect(&full_v[stage], k_bytes);
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
                  tma_load_5d(vb + h * KV_HALF, &v_map, h * 64, slot, g, page, layer, &full_v[stage]);
              }
            } else {
              if (gt >= 2) mbar_wait(&s_done[stage], ((gt - 2) >> 1) & 1, status, &gave_up);
              load_tile(t, box_pages + staged, false);
              if (gt >= 2) mbar_wait(&o_done[stage], ((gt - 2) >> 1) & 1, status, &gave_up);
              load_tile(t, box_pages + staged, true);
            }
            if (++staged == tiles_per_fill) staged = 0;
            __syncwarp();  // the lanes stay together (the staged pages are replaced by all of them)
          }
        } else {
          for (int t = 0; t < n_tiles; ++t) {
            if (staged == 0) fill_pages(t);
            const int* pages = box_pages + staged * n_boxes;
            const int gt = base + t, stage = gt & 1;
            if (gt >= 2) mbar_wait(&s_done[stage], ((gt - 2) >> 1) & 1, status, &gave_up);
            load_tile(t, pages, false);
            if (gt >= 2) mbar_wait(&o_done[stage], ((gt - 2) >> 1) & 1, status, &gave_up);
            load_tile(t, pages, true);
            if (++staged == tiles_per_fill) staged = 0;
          }
        }
      } else if (warp == MMA_WARP) {
        // ================================ MMA warp ================================
        // One thread issues everything; products run in the order of issue, so the S
        // that overwrites the columns of the S / P two tiles back follows that tile's O
        // by itself.
        if (lane == 0) {
          const uint64_t q_desc = smem_desc(Qs, 16), k_desc = smem_desc(Ks, 16), v_desc = smem_desc(Vs, KV_HALF);
          auto issue_s = [&](int t) {
            const int gt = base + t, stage = gt & 1;
            mbar_wait(&full_k[stage], (gt >> 1) & 1, status, &gave_up);
            tc_fence_after();
            const uint64_t kd = k_desc + (uint64_t)((stage * STAGE_BYTES) >> 4);
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk)
              umma_f16(tmem + COL_S0 + stage * KEYS, q_desc + (uint64_t)(((kk / 4) * Q_HALF + (kk % 4) * 32) >> 4),
                       kd + (uint64_t)(((kk / 4) * KV_HALF + (kk % 4) * 32) >> 4), IDESC_S, kk > 0 ? 1u : 0u);
            umma_commit(&s_done[stage]);
          };
          issue_s(0);
          for (int t = 0; t < n_tiles; ++t) {
            const int gt = base + t, stage = gt & 1;
            if (t + 1 < n_tiles) issue_s(t + 1);
            // all softmax threads have stored P_t (and rescaled O where needed)
            mbar_wait(&p_ready[stage], (gt >> 1) & 1, status, &gave_up);
            mbar_wait(&full_v[stage], (gt >> 1) & 1, status, &gave_up);
            tc_fence_after();
            const uint64_t vd = v_desc + (uint64_t)((stage * STAGE_BYTES) >> 4);
#pragma unroll
            for (int j = 0; j < KEYS / 16; ++j)
              umma_f16_ts(tmem + COL_O, tmem + COL_S0 + stage * KEYS + j * 8, vd + (uint64_t)((j * 16 * 128) >> 4),
                          IDESC_O, (t > 0 || j > 0) ? 1u : 0u);
            umma_commit(&o_done[stage]);
          }
        }
        __syncwarp();
      } else {
        // =============================== softmax warps ===============================
        const uint32_t my_lane = (uint32_t)(warp * 32) << 16;  // this warp's quarter of the TMEM lanes
        float m_ref = -INFINITY, l_run = 0.f;
        const float c = scale_log2;
        const bool warp_full = __all_sync(0xffffffffu, my_valid);
        int warp_max = my_pos, warp_min = my_valid ? my_pos : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          warp_max = max(warp_max, __shfl_xor_sync(0xffffffffu, warp_max, o));
          warp_min = min(warp_min, __shfl_xor_sync(0xffffffffu, warp_min, o));
        }
        for (int t = 0; t < n_tiles; ++t) {
          const int gt = base + t, stage = gt & 1;
          const uint32_t s_addr = tmem + my_lane + COL_S0 + stage * KEYS;
          mbar_wait(&s_done[stage], (gt >> 1) & 1, status, &gave_up);
          tc_fence_after();
          const int k0 = k_lo + t * KEYS;
          float s[KEYS];
          tmem_ld64(s_addr, s);
          const bool need_mask =
              !warp_full || k0 + KEYS - 1 > warp_min || (window > 0 && k0 <= warp_max - window);
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < KEYS; ++i) {
              const int j = k0 + i;
              const bool vis = my_pos >= 0 && j <= my_pos && (window <= 0 || j > my_pos - window);
              if (!vis) s[i] = -INFINITY;
            }
          }
          // four independent chains for the maximum (and below for the sum): a row is one
          // thread's, and a single chain of 64 dependent operations would be all latency
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int i = 0; i < KEYS; i += 8) {
            mx4[0] = max3(mx4[0], s[i], s[i + 1]);
            mx4[1] = max3(mx4[1], s[i + 2], s[i + 3]);
            mx4[2] = max3(mx4[2], s[i + 4], s[i + 5]);
            mx4[3] = max3(mx4[3], s[i + 6], s[i + 7]);
          }
          const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          // raise the reference maximum only when it pays (or when there is none yet)
          float alpha = 1.f;
          bool raise = false;
          if (mx != -INFINITY && (m_ref == -INFINITY || (mx - m_ref) * c > RESCALE_THRESHOLD)) {
            raise = true;
            alpha = (m_ref == -INFINITY) ? 0.f : exp2f((m_ref - mx) * c);
            m_ref = mx;
          }
          float sum = 0.f;
          uint32_t packed[KEYS / 2];
          if (m_ref == -INFINITY) {
#pragma unroll
            for (int i = 0; i < KEYS / 2; ++i) packed[i] = 0u;
          } else {
            const float mc = m_ref * c;
            const uint64_t c2 = f32x2(c, c), nmc2 = f32x2(-mc, -mc);
            uint64_t sum2[2] = {f32x2(0.f, 0.f), f32x2(0.f, 0.f)};
#pragma unroll
            for (int i = 0; i < KEYS; i += 4) {
              float x0, x1, x2, x3;
              f32x2_split(fma_f32x2(f32x2(s[i], s[i + 1]), c2, nmc2), x0, x1);
              f32x2_split(fma_f32x2(f32x2(s[i + 2], s[i + 3]), c2, nmc2), x2, x3);
              const float p0 = ex2_approx(x0), p1 = ex2_approx(x1), p2 = ex2_approx(x2), p3 = ex2_approx(x3);
              sum2[0] = add_f32x2(sum2[0], f32x2(p0, p1));
              sum2[1] = add_f32x2(sum2[1], f32x2(p2, p3));
              packed[i / 2] = pack_bf16(p0, p1);
              packed[i / 2 + 1] = pack_bf16(p2, p3);
            }
            float a0, a1, a2, a3;
            f32x2_split(sum2[0], a0, a1);
            f32x2_split(sum2[1], a2, a3);
            sum = (a0 + a1) + (a2 + a3);
          }
          l_run = l_run * alpha + sum;
          // P_t over the first 32 columns of S_t (this thread has read all of its row)
          tmem_st32_raw(s_addr, packed);
          // Where a row's reference maximum was raised, O is rescaled before this tile's P V may
          // run (warp-uniform decision), once O_{t-1} is complete; otherwise the warp does not
          // wait for O at all.  (The barrier of this parity completes next for O_{t+1}, which
          // needs this thread's P_{t+1}: a wait on it cannot fall behind.)
          if (t > 0 && __any_sync(0xffffffffu, raise)) {
            mbar_wait(&o_done[(gt - 1) & 1], ((gt - 1) >> 1) & 1, status, &gave_up);
            tc_fence_after();
#pragma unroll
            for (int cc = 0; cc < HD / 32; ++cc) {
              float part[32];
              tmem_ld32(tmem + my_lane + COL_O + cc * 32, part);
#pragma unroll
              for (int i = 0; i < 32; ++i) part[i] *= alpha;
              tmem_st32(tmem + my_lane + COL_O + cc * 32, part);
            }
          }
          tc_fence_before();
          mbar_arrive(&p_ready[stage]);
        }
        // ---- O / l -> out ----
        const int gl = base + n_tiles - 1;
        mbar_wait(&o_done[gl & 1], (gl >> 1) & 1, status, &gave_up);
        tc_fence_after();
        __nv_bfloat16* dst =
            out + (size_t)(tok0 + row_token(tid)) * out_stride + (g * group + row_head(tid)) * HD;
        if (!split) {
          const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll
          for (int cc = 0; cc < HD / 32; ++cc) {
            float part_o[32];
            tmem_ld32(tmem + my_lane + COL_O + cc * 32, part_o);
            if (my_valid) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 v;
                v.x = pack_bf16(part_o[i] * inv, part_o[i + 1] * inv);
                v.y = pack_bf16(part_o[i + 2] * inv, part_o[i + 3] * inv);
                v.z = pack_bf16(part_o[i + 4] * inv, part_o[i + 5] * inv);
                v.w = pack_bf16(part_o[i + 6] * inv, part_o[i + 7] * inv);
                *reinterpret_cast<uint4*>(dst + cc * 32 + i) = v;
              }
            }
          }
        } else {
          constexpr size_t SLOT = (size_t)ROWS * (HD + 2);
          float* slots = split_scratch + (size_t)item * parts * SLOT;
          write_partial<HD>(tmem + my_lane + COL_O, slots + part * SLOT + tid,
                            m_ref == -INFINITY ? -INFINITY : m_ref * c, l_run);
          // Every part counts itself when its partial is complete; the one that counts last adds
          // them all up (its own too, from where it left it: the sum does not depend on which
          // part that is).  Nobody waits for anybody.
          __threadfence();
          asm volatile("bar.sync 1, %0;\n" ::"n"(SOFTMAX_THREADS) : "memory");
          if (tid == 0) split_order_s = atomicAdd(&split_flags[2 * item], 1);
          asm volatile("bar.sync 1, %0;\n" ::"n"(SOFTMAX_THREADS) : "memory");
          if (split_order_s == n_parts - 1) {
            __threadfence();
            merge_parts<HD>(slots + tid, n_parts, dst, my_valid);
            if (tid == 0) split_flags[2 * item] = 0;  // zero again for the next launch
          }
        }
        tc_fence_before();
      }
    }
    base += n_tiles;
    // The softmax warps leave an item last (its O is complete then, so every product that
    // read Q or a stage of K/V has run); after this barrier Q and the page list are free.
    __syncthreads();
    if (tid == 0) {
      const unsigned int draw = atomicAdd(work_counter, 1u);
      work_s = gridDim.x + draw;
      if (draw == last_draw) *work_counter = 0u;  // the launch's last draw: ready for the next launch
    }
    __syncthreads();
    work = work_s;
    dead = *reinterpret_cast<volatile int*>(&gave_up) != 0;
  }
  if (dead && tid == MMA_WARP * 32) {
    // products issued after the wait that ran out may still be running: the tensor memory is
    // given back only once they are through (or this wait runs out too)
    umma_commit(&drained);
    for (int it = 0; it < MBAR_WAIT_POLLS && !mbar_try_wait(&drained, 0); ++it) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == LOAD_WARP) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace fg_tc5
