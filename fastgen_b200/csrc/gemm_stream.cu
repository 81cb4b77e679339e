// Weight-streaming matrix product for a decode batch on the 5th-generation tensor cores:
//   y[M, N] = x[M, K] * W[N, K]^T,  bfloat16 inputs, float32 accumulation, 8 < M <= 256.
//
// With a few dozen tokens the product is still bound by reading W once from HBM, but too
// wide for the mma.sync kernel of gemm_skinny.cu (every block would re-read all of x).
// Here the operands are swapped for tcgen05.mma: 128 rows of W are the M side of the
// instruction, the (padded) tokens the N side, the accumulator [128 rows, tokens] lives in
// tensor memory.  W and x arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle) in
// stages of 64 k elements through a ring of shared-memory stages.
//
// Work is cut "stream-K" fashion so that every SM streams the same number of bytes
// whatever N is: the (tile of 128 rows, stage of 64 k) units are numbered tile by tile and
// block i of G takes units [i T / G, (i + 1) T / G).  A block whose range starts inside
// a tile writes that tile's partial sums (float32) to scratch and counts an arrival; the
// block that holds the tile's first unit adds the partials of the blocks after it, in
// block order, and writes the result.  The block that waits is the one that reaches the
// tile last in its own range, the partials it waits for were written first in theirs, and
// a block that writes a partial never waits: no cycle.  The cut depends on N, K and the
// number of SMs only, so a token's result does not depend on what else is in the batch.
//
// Warps: one issues the TMA copies, one (a single thread) the tcgen05.mma, four read the
// accumulator back (tcgen05.ld, a row of W a thread) and write y.  Two accumulators
// alternate so that a tile's epilogue overlaps the next tile's products.  Waits are
// bounded and report through the status word.
//
// It stands where the reference calls F.linear on decode batches
// (fastgen/forward.py:438-440,470,491-496,513).
#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"
#include "tc5_primitives.cuh"

namespace {

using namespace fg_tc5;

constexpr int TILE_N = 128;   // rows of W a tile (the M side of the instruction)
constexpr int CHUNK_K = 64;   // k elements a stage: 128 bytes a row, the swizzle span
constexpr int GS_THREADS = 192;  // TMA warp, MMA warp, four epilogue warps
constexpr int W_STAGE = TILE_N * 128;
constexpr int MAX_STAGES = 12;

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], "
      "[%4];\n" ::"r"(smem_u32(dst)),
      "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}

// 16 consecutive columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ float ld_cg_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];\n" : "=f"(v) : "l"(p) : "memory");
  return v;
}

struct Cut {
  long long total;  // units in all
  int n_chunks;     // units a tile
  int grid;
  __device__ __host__ long long begin(int block) const { return (long long)block * total / grid; }
  // the block whose range holds unit u
  __device__ __host__ int block_of(long long u) const { return (int)(((u + 1) * grid + total - 1) / total) - 1; }
};

// A block's range, tile by tile: segment = (tile, first chunk, end chunk).
struct Segments {
  long long u, end;
  int n_chunks;
  __device__ Segments(const Cut& cut, int block) : u(cut.begin(block)), end(cut.begin(block + 1)), n_chunks(cut.n_chunks) {}
  __device__ bool next(int& tile, int& c0, int& c1) {
    if (u >= end) return false;
    tile = (int)(u / n_chunks);
    c0 = (int)(u - (long long)tile * n_chunks);
    const long long tile_end = (long long)(tile + 1) * n_chunks;
    const long long stop = tile_end < end ? tile_end : end;
    c1 = c0 + (int)(stop - u);
    u = stop;
    return true;
  }
};

template <typename TO>
__global__ void __launch_bounds__(GS_THREADS, 2)
gemm_stream_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                   TO* __restrict__ y, int ldy, int M, int N, int m_pad, int n_stages, Cut cut, float* partials,
                   int* arrivals, int tmem_cols, int* status) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  const int x_stage = m_pad * 128;
  const int stage_bytes = W_STAGE + x_stage;
  __shared__ __align__(8) uint64_t full[MAX_STAGES], empty[MAX_STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;

  pdl_trigger();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);  // one arrival an epilogue warp
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t idesc = instr_desc(m_pad, false);

  if (warp == 0) {
    // ================================ TMA warp ================================
    // The copies of consecutive stages are issued by different lanes (the lanes walk the
    // same list; lane it % ISSUERS issues stage it).
    {
      constexpr int ISSUERS = 4;
      // The weights do not depend on the kernel before this one: the first stages' W tiles
      // are on their way while that kernel finishes; x (its output) is touched after the wait.
      Segments pre(cut, blockIdx.x);
      int tile, c0, c1, it = 0;
      const long long n_units = cut.begin(blockIdx.x + 1) - cut.begin(blockIdx.x);
      const int n_pre = (int)(n_units < n_stages ? n_units : n_stages);
      int pre_chunk[MAX_STAGES];
      while (it < n_pre && pre.next(tile, c0, c1))
        for (int c = c0; c < c1 && it < n_pre; ++c, ++it) {
          pre_chunk[it] = c;
          if (lane == it % ISSUERS) {
            mbar_arrive_expect(&full[it], stage_bytes);
            tma_load_2d(smem + it * stage_bytes, &w_map, c * CHUNK_K, tile * TILE_N, &full[it]);
          }
        }
      pdl_wait();
      for (int i = 0; i < n_pre; ++i)
        if (lane == i % ISSUERS)
          tma_load_2d(smem + i * stage_bytes + W_STAGE, &x_map, pre_chunk[i] * CHUNK_K, 0, &full[i]);
      Segments seg(cut, blockIdx.x);
      it = 0;
      while (seg.next(tile, c0, c1))
        for (int c = c0; c < c1; ++c, ++it) {
          if (it < n_pre || lane != it % ISSUERS) continue;
          const int s = it % n_stages;
          mbar_wait(&empty[s], (it / n_stages - 1) & 1, status);
          mbar_arrive_expect(&full[s], stage_bytes);
          unsigned char* dst = smem + s * stage_bytes;
          tma_load_2d(dst, &w_map, c * CHUNK_K, tile * TILE_N, &full[s]);
          tma_load_2d(dst + W_STAGE, &x_map, c * CHUNK_K, 0, &full[s]);
        }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================================ MMA warp ================================
    if (lane == 0) {
      const uint64_t desc0 = smem_desc(smem, 16);
      Segments seg(cut, blockIdx.x);
      int tile, c0, c1, n_seg = 0;
      int s = 0, parity = 0;  // the stage in turn and the parity of its fill
      const uint64_t stage_desc = (uint64_t)(stage_bytes >> 4);
      uint64_t wd = desc0;
      while (seg.next(tile, c0, c1)) {
        const int buf = n_seg & 1;
        if (n_seg >= 2) mbar_wait(&acc_empty[buf], ((n_seg >> 1) - 1) & 1, status);
        tc_fence_after();
        const uint32_t d_tmem = tmem + buf * m_pad;
        for (int c = c0; c < c1; ++c) {
          mbar_wait(&full[s], parity, status);
          tc_fence_after();
          const uint64_t xd = wd + (uint64_t)(W_STAGE >> 4);
#pragma unroll
          for (int kk = 0; kk < CHUNK_K / 16; ++kk)
            umma_f16(d_tmem, wd + (uint64_t)(kk * 2), xd + (uint64_t)(kk * 2), idesc, (c > c0 || kk > 0) ? 1u : 0u);
          umma_commit(&empty[s]);  // the stage is free once these products have read it
          wd += stage_desc;
          if (++s == n_stages) {
            s = 0;
            parity ^= 1;
            wd = desc0;
          }
        }
        umma_commit(&acc_full[buf]);
        ++n_seg;
      }
    }
    __syncwarp();
  } else {
    // ================================ epilogue warps ================================
    pdl_wait();  // nothing is written to global memory before the kernel before this one is done
    const int quarter = warp & 3;  // the TMEM lanes a warp may read
    const int row = quarter * 32 + lane;
    const int etid = tid - 64;     // 0..127 among the epilogue threads
    Segments seg(cut, blockIdx.x);
    int tile, c0, c1, n_seg = 0;
    while (seg.next(tile, c0, c1)) {
      const int buf = n_seg & 1;
      mbar_wait(&acc_full[buf], (n_seg >> 1) & 1, status);
      tc_fence_after();
      const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + buf * m_pad;
      const int n = tile * TILE_N + row;
      const bool head = c0 == 0;
      const bool whole = head && c1 == cut.n_chunks;
      int expected = 0;
      if (head && !whole) {
        // blocks after this one hold the rest of the tile: wait for their partials
        expected = cut.block_of((long long)(tile + 1) * cut.n_chunks - 1) - (int)blockIdx.x;
        if (etid == 0) {
          int seen = 0;
          for (int spin = 0; spin < (1 << 24); ++spin) {
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(seen) : "l"(arrivals + tile) : "memory");
            if (seen >= expected) break;
          }
          if (seen < expected && status) atomicOr(status, FG_STATUS_WAIT_TIMEOUT);
          arrivals[tile] = 0;  // for the next launch
        }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
      }
      float* mine = partials + (size_t)blockIdx.x * m_pad * TILE_N;
      for (int j0 = 0; j0 < m_pad; j0 += 32) {
        float v[32];
        if (j0 + 32 <= m_pad) {
          tmem_ld32(taddr + j0, v);
        } else {
          float h[16];
          tmem_ld16(taddr + j0, h);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            v[i] = h[i];
            v[16 + i] = 0.f;
          }
        }
        if (!head) {
          // this block's share of the tile: to scratch, [token][row]
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (j0 + i < M) mine[(size_t)(j0 + i) * TILE_N + row] = v[i];
          continue;
        }
        for (int p = 1; p <= expected; ++p) {
          const float* theirs = partials + (size_t)(blockIdx.x + p) * m_pad * TILE_N;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (j0 + i < M) v[i] += ld_cg_f32(theirs + (size_t)(j0 + i) * TILE_N + row);
        }
        if (n < N) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (j0 + i < M) y[(size_t)(j0 + i) * ldy + n] = from_f32<TO>(v[i]);
        }
      }
      if (!head) {
        // publish: the partial is complete once all four warps are through
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        if (etid == 0) {
          int old;
          asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;\n" : "=r"(old) : "l"(arrivals + tile) : "memory");
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      ++n_seg;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, tmem_cols);
}

PFN_cuTensorMapEncodeTiled_v12000 encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

// a bfloat16 matrix [rows, cols] with row stride ld (elements), boxes of [box_rows, 64]
int matrix_map(CUtensorMap* out, const void* base, int rows, int cols, int ld, int box_rows) {
  auto encode = encoder();
  FG_CHECK_ARG(encode != nullptr, "fg_gemm_stream_bf16: the driver has no cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {CHUNK_K, (cuuint32_t)box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FG_CHECK_ARG(r == CUDA_SUCCESS, "fg_gemm_stream_bf16: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

int sm_count() {
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return n_sms;
}

}  // namespace

extern "C" int fg_gemm_stream_max_m() { return 256; }

// Floats of scratch (partials) and ints (arrival counts, zero before the first call and left
// at zero by every call) that a product with these sizes needs.
extern "C" long long fg_gemm_stream_scratch_floats(int M) {
  const int m_pad = (M + 15) / 16 * 16;
  return (long long)2 * sm_count() * m_pad * TILE_N;  // a partial a block, up to two blocks an SM
}
extern "C" int fg_gemm_stream_counters(int N) { return (N + TILE_N - 1) / TILE_N; }

// x: [M, K] bf16 (row stride ldx), w: [N, K] bf16 (row stride ldw), y: [M, N] bf16 or float32.
// Needs 1 <= M <= 256, K % 8 == 0, 16-byte aligned x and w with strides % 8 == 0.
extern "C" int fg_gemm_stream_bf16(const void* x, int ldx, const void* w, int ldw, void* y, int ldy, int out_dtype,
                                   int M, int N, int K, float* scratch, long long scratch_floats, int* counters,
                                   int n_counters, int* status, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  FG_CHECK_ARG(M <= 256, "fg_gemm_stream_bf16: M=%d exceeds 256", M);
  FG_CHECK_ARG(K > 0 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ldx >= K && ldw >= K && ldy >= N,
               "fg_gemm_stream_bf16: K=%d and the row strides (%d, %d) must be multiples of 8", K, ldx, ldw);
  FG_CHECK_ARG(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "fg_gemm_stream_bf16: x and w must be 16-byte aligned");
  const int m_pad = (M + 15) / 16 * 16;
  const int n_tiles = (N + TILE_N - 1) / TILE_N;
  const int n_chunks = (K + CHUNK_K - 1) / CHUNK_K;
  FG_CHECK_ARG(scratch != nullptr && scratch_floats >= fg_gemm_stream_scratch_floats(M) && counters != nullptr &&
                   n_counters >= n_tiles,
               "fg_gemm_stream_bf16: scratch of %lld floats / %d counters is too small", scratch_floats, n_counters);
  Cut cut;
  cut.total = (long long)n_tiles * n_chunks;
  cut.n_chunks = n_chunks;
  // Two blocks an SM where the ring allows it: one block's single TMA-issuing and
  // MMA-issuing threads sustain about 30 GB/s, less than an SM's share of the HBM stream.
  const int stage_bytes = W_STAGE + m_pad * 128;
  const int per_sm = 110 * 1024 / stage_bytes >= 3 ? 2 : 1;
  const int blocks = per_sm * sm_count();
  cut.grid = (int)(cut.total < blocks ? cut.total : blocks);
  int n_stages = ((per_sm == 2 ? 110 : 220) * 1024) / stage_bytes;
  if (n_stages > MAX_STAGES) n_stages = MAX_STAGES;
  FG_CHECK_ARG(n_stages >= 2, "fg_gemm_stream_bf16: no room for two stages at M=%d", M);
  int tmem_cols = 32;
  while (tmem_cols < 2 * m_pad) tmem_cols *= 2;
  CUtensorMap wm, xm;
  if (matrix_map(&wm, w, N, K, ldw, TILE_N)) return -1;
  if (matrix_map(&xm, x, M, K, ldx, m_pad)) return -1;
  const size_t smem = (size_t)n_stages * stage_bytes + 1024;
#define LAUNCH(TO)                                                                                              \
  do {                                                                                                          \
    auto kern = gemm_stream_kernel<TO>;                                                                         \
    static size_t attr = 0;                                                                                     \
    if (attr < smem) {                                                                                          \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
      FG_CHECK_ARG(e == cudaSuccess, "fg_gemm_stream_bf16: shared memory: %s", cudaGetErrorString(e));          \
      attr = smem;                                                                                              \
    }                                                                                                           \
    fg_launch_pdl(kern, dim3(cut.grid), dim3(GS_THREADS), smem, stream, wm, xm, (TO*)y, ldy, M, N, m_pad, n_stages, \
                  cut, scratch, counters, tmem_cols, status);                                                   \
  } while (0)
  if (out_dtype == FG_BF16)
    LAUNCH(__nv_bfloat16);
  else if (out_dtype == FG_F32)
    LAUNCH(float);
  else
    FG_CHECK_ARG(false, "fg_gemm_stream_bf16: bad output dtype %d", out_dtype);
#undef LAUNCH
  FG_CHECK_LAUNCH("fg_gemm_stream_bf16");
  return 0;
}
