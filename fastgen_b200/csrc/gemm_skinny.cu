// Weight-streaming matrix product for a few tokens (decode):
//   y[M, N] = x[M, K] * W[N, K]^T,  bfloat16 inputs, float32 accumulation, M <= 32.
//
// With so few tokens the product is bound by reading W once from HBM.  The roles
// of the operands are swapped for the tensor core: 16 rows of W are the "M" side
// of mma.sync m16n8k16 and 8 tokens the "N" side, so no row of the instruction is
// wasted on padding.  A thread's fragments are 16-byte pieces of W and x (the k
// index inside an instruction is permuted identically for both operands, which
// does not change the sum).  Every thread streams its own pieces through a ring
// of cp.async stages in shared memory that only it reads back, so the main loop
// has no barrier and many kilobytes per warp are in flight without holding
// registers.  A block owns 16 rows of W; its 8 warps split K in interleaved chunks
// of 64 and are summed in warp order at the end, so a row's result depends on
// nothing but K.
//
// Two fused variants serve the decode step:
//  * epilogue "SwiGLU": W holds gate and up rows interleaved in blocks of 8 (rows
//    16b..16b+7 gate, 16b+8..16b+15 up of features 8b..8b+7), so a block's 16 rows
//    are gate and up of the same 8 features and it writes silu(gate) * up
//    (fastgen/forward.py:491-495) -- the [gate | up] intermediate never exists;
//  * epilogue "QKV": the 16 output rows are 8 adjacent pairs of one head; they are
//    rotated by the token's position (fastgen/kernels/rope.py:77-89), queries go
//    to y, keys and values straight into their cache pages
//    (fastgen/forward.py:449-460), replacing a separate kernel and a round trip.
//
// It stands where the reference calls F.linear on decode batches
// (fastgen/forward.py:438-440,470,491-496,513); larger M goes to the library.
#include "common.cuh"

namespace {

constexpr int ROWS = 16;   // rows of W per block
constexpr int CHUNK = 64;  // k elements per warp step
constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;

enum { EPI_PLAIN = 0, EPI_QKV = 1, EPI_SWIGLU = 2 };

struct QkvEpilogue {
  const int* pos;
  const int* req;
  const float* freqs;  // [head_dim / 2] or null
  __nv_bfloat16* k_pages;
  __nv_bfloat16* v_pages;
  const int* block_table;
  int table_width, page_size, n_pages;
  int n_heads, n_kv_heads, head_dim;
  int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 16-byte asynchronous copy; `keep` asks for the line to stay in L1 (activations,
// read by every warp) while weights, read once, bypass it.  !pred: zero-fill.
template <bool KEEP>
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool pred) {
  const int bytes = pred ? 16 : 0;
  if (KEEP)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes)
                 : "memory");
  else
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                    uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16-byte pieces a thread copies per chunk (4 of W, the rest of x), ring depth, ring size.
// How many blocks share an SM is chosen with the ring (up to 8 tokens; the warps' sums then go
// to the ring's memory once it is through, not to memory of their own):
//  * TWO_AN_SM: four stages, 96 KiB a block.  The shared-memory carve-out is asked to be no
//    larger than the two blocks need (196 KiB), which leaves the L1 room for x: every block reads
//    all of x, 64 KiB at 8 tokens of 4,096, and a product of 28,672 rows took 40.5 us with the
//    largest carve-out against 38.7 (36.7 with one token).
//  * THREE_AN_SM: three stages, 72 KiB.  A launch of a little more than two blocks an SM runs
//    as one round and a fraction of a second one, and the fraction costs about as much as a
//    whole round (16 rows of 4,096 a block, 8 tokens: 296 blocks 7.8 us, 320 blocks 10.7, 384
//    blocks 12.9, 592 blocks 14.7); with three blocks an SM up to 444 blocks run at once, with
//    as many bytes in flight an SM (320 blocks 9.0 us, 384 blocks 9.7).
//  * ONE_AN_SM: six stages, 144 KiB, for a launch of no more blocks than SMs: every block has
//    an SM of its own then, and half as many bytes again in flight (2,048 rows of 8,192, 8
//    tokens: 10.0 -> 7.2 us; 2,048 rows of 4,096: 5.7 -> 4.4).
enum { TWO_AN_SM = 0, THREE_AN_SM = 1, ONE_AN_SM = 2 };

template <int NT, int MODE = TWO_AN_SM>
struct Ring {
  static_assert(MODE == TWO_AN_SM || NT == 1, "the other rings are for up to 8 tokens");
  static constexpr int PIECES = 4 + 2 * NT;
  static constexpr int STAGES =
      MODE == THREE_AN_SM ? 3 : (MODE == ONE_AN_SM ? 6 : (NT == 1 ? 4 : (NT == 2 ? 3 : 2)));  // 96 KiB: two blocks an SM
  static constexpr size_t BYTES = (size_t)STAGES * PIECES * THREADS * 16;
  static constexpr bool SUMS_IN_RING = NT == 1;
  // per cent of the largest carve-out to ask for (0: the driver's choice)
  static constexpr int CARVEOUT = NT != 1 ? 0 : (MODE == THREE_AN_SM ? 100 : (MODE == ONE_AN_SM ? 70 : 80));
};

// One block's product: 16 rows of W (from row n0) against the tokens' x.  The pieces a
// thread streams, its ring and its accumulators; the callers decide when the weights'
// first stages are issued (they may go ahead of data that is not ready yet).
template <int NT, int MODE = TWO_AN_SM>
struct BlockProduct {
  static constexpr int PIECES = Ring<NT, MODE>::PIECES;
  static constexpr int STAGES = Ring<NT, MODE>::STAGES;
  uint4* ring;  // [STAGES][PIECES][THREADS]
  const __nv_bfloat16 *wa, *wb, *xr[NT];
  bool row_a, row_b, tok_ok[NT];
  float acc[NT][4];
  int K, my_chunks, tid, warp, r, c;

  __device__ __forceinline__ void setup(uint4* ring_, const __nv_bfloat16* x, int ldx, const __nv_bfloat16* w, int ldw,
                                        int M, int N, int K_, int n0) {
    ring = ring_;
    K = K_;
    tid = threadIdx.x;
    warp = tid >> 5;
    const int lane = tid & 31;
    r = lane >> 2;
    c = lane & 3;
    // rows beyond N and tokens beyond M are zero-filled and discarded at the end
    row_a = n0 + r < N;
    row_b = n0 + r + 8 < N;
    wa = w + (size_t)(row_a ? n0 + r : 0) * ldw + c * 8;
    wb = w + (size_t)(row_b ? n0 + r + 8 : 0) * ldw + c * 8;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int tok = nt * 8 + r;
      tok_ok[nt] = tok < M;
      xr[nt] = x + (size_t)(tok_ok[nt] ? tok : 0) * ldx + c * 8;
      acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    }
    const int n_chunks = (K + CHUNK - 1) / CHUNK;
    my_chunks = warp < n_chunks ? (n_chunks - warp + WARPS - 1) / WARPS : 0;
  }

  // issue the copies of this thread's i-th chunk into stage i % STAGES: the pieces of
  // W, the pieces of x, or both
  __device__ __forceinline__ void issue(int i, bool do_w, bool do_x) {
    uint4* slot = ring + (size_t)(i % STAGES) * PIECES * THREADS + tid;
    const int k = (warp + i * WARPS) * CHUNK;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int kk = k + h * 32;
      const bool ok = kk + c * 8 < K;  // K is a multiple of 8: a 16-byte piece is all in or all out
      if (do_w) {
        cp_async_16<false>(slot + (2 * h) * THREADS, wa + kk, ok && row_a);
        cp_async_16<false>(slot + (2 * h + 1) * THREADS, wb + kk, ok && row_b);
      }
      if (do_x) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
          cp_async_16<true>(slot + (4 + nt * 2 + h) * THREADS, xr[nt] + kk, ok && tok_ok[nt]);
      }
    }
  }

  // the weights of the first stages (they depend on nothing that is computed in the step)
  __device__ __forceinline__ void first_weights() {
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s)
      if (s < my_chunks) issue(s, true, false);
  }

  // the x pieces of the first stages, the main loop, and the warps' sums into `red`
  __device__ __forceinline__ void run(float (*red)[ROWS][NT * 8]) {
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
      if (s < my_chunks) issue(s, false, true);
      cp_async_commit();
    }
    for (int i = 0; i < my_chunks; ++i) {
      if (i + STAGES - 1 < my_chunks) issue(i + STAGES - 1, true, true);
      cp_async_commit();
      cp_async_wait<STAGES - 1>();  // this thread's copies of chunk i have landed; only it reads them
      const uint4* slot = ring + (size_t)(i % STAGES) * PIECES * THREADS + tid;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint4 a_lo = slot[(2 * h) * THREADS], a_hi = slot[(2 * h + 1) * THREADS];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint4 b = slot[(4 + nt * 2 + h) * THREADS];
          mma(acc[nt], a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
          mma(acc[nt], a_lo.z, a_hi.z, a_lo.w, a_hi.w, b.z, b.w);
        }
      }
    }
    if (Ring<NT, MODE>::SUMS_IN_RING) __syncthreads();  // `red` is the ring's memory: every thread is through with its stages
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      red[warp][r][nt * 8 + 2 * c] = acc[nt][0];
      red[warp][r][nt * 8 + 2 * c + 1] = acc[nt][1];
      red[warp][r + 8][nt * 8 + 2 * c] = acc[nt][2];
      red[warp][r + 8][nt * 8 + 2 * c + 1] = acc[nt][3];
    }
    __syncthreads();
  }
};

// the warps' partial sums of (row, token), in warp order
template <int NT>
__device__ __forceinline__ float block_total(float (*red)[ROWS][NT * 8], int row, int tok) {
  float s = 0.f;
#pragma unroll
  for (int wi = 0; wi < WARPS; ++wi) s += red[wi][row][tok];
  return s;
}

template <int NT, typename TO>
__device__ __forceinline__ void epilogue_plain(float (*red)[ROWS][NT * 8], TO* y, int ldy, int M, int N, int n0) {
  for (int i = threadIdx.x; i < ROWS * NT * 8; i += THREADS) {
    const int tok = i / ROWS, row = i - tok * ROWS;  // consecutive threads write consecutive columns of y
    if (tok < M && n0 + row < N) y[(size_t)tok * ldy + n0 + row] = from_f32<TO>(block_total<NT>(red, row, tok));
  }
}

// rows 0..7 are the gates and rows 8..15 the ups of features n0/2 .. n0/2+7
template <int NT, typename TO>
__device__ __forceinline__ void epilogue_swiglu(float (*red)[ROWS][NT * 8], TO* y, int ldy, int M, int N, int n0) {
  for (int i = threadIdx.x; i < 8 * NT * 8; i += THREADS) {
    const int tok = i / 8, f = i - tok * 8;
    if (tok < M && n0 + 8 + f < N) {
      const float g = block_total<NT>(red, f, tok), u = block_total<NT>(red, f + 8, tok);
      // both are rounded to bfloat16 first, as a separate gate kernel would see them
      const float gr = __bfloat162float(__float2bfloat16_rn(g)), ur = __bfloat162float(__float2bfloat16_rn(u));
      y[(size_t)tok * ldy + n0 / 2 + f] = from_f32<TO>(gr / (1.f + expf(-gr)) * ur);
    }
  }
}

template <int NT, typename TO, int EPI, int MODE = TWO_AN_SM>
__global__ void __launch_bounds__(THREADS)
gemm_skinny_kernel(const __nv_bfloat16* x, int ldx, const __nv_bfloat16* __restrict__ w, int ldw,
                   TO* __restrict__ y, int ldy, int M, int N, int K, QkvEpilogue qkv) {
  extern __shared__ __align__(16) unsigned char ring_raw[];
  constexpr bool RED_IN_RING = Ring<NT, MODE>::SUMS_IN_RING;
  __shared__ float red_own[RED_IN_RING ? 1 : WARPS][ROWS][NT * 8];
  float (*red)[ROWS][NT * 8] = RED_IN_RING ? reinterpret_cast<float (*)[ROWS][NT * 8]>(ring_raw) : red_own;
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * ROWS;
  BlockProduct<NT, MODE> block;
  block.setup(reinterpret_cast<uint4*>(ring_raw), x, ldx, w, ldw, M, N, K, n0);

  // The weights do not depend on the kernel before this one: their first stages are on
  // their way while that kernel finishes.  x (its output) is only touched after the wait.
  pdl_trigger();
  // QKV epilogue: what depends on the token's position alone (angle, page) is worked out
  // now, while the weights stream, so that the end of the block is a rotation and a store.
  // Positions, requests and block tables are inputs of the step.
  int e_tok = -1, e_n = 0, e_kind = 0;  // kind 0: query, 1: key, 2: value; e_tok < 0: nothing to write
  float e_sin = 0.f, e_cos = 1.f;
  size_t e_dst = 0;
  if (EPI == EPI_QKV && tid < (ROWS / 2) * NT * 8) {
    const int hd = qkv.head_dim, q_width = qkv.n_heads * hd, kv_width = qkv.n_kv_heads * hd;
    const int tok = tid / (ROWS / 2), pr = tid - tok * (ROWS / 2);
    const int n = n0 + 2 * pr;
    const int slot_req = tok < M ? qkv.req[tok] : -1;
    if (n < N && slot_req >= 0) {
      const int p = qkv.pos[tok];
      e_kind = n < q_width ? 0 : (n < q_width + kv_width ? 1 : 2);
      if (e_kind != 2 && qkv.freqs != nullptr) sincosf((float)p * qkv.freqs[(n % hd) >> 1], &e_sin, &e_cos);
      e_tok = tok;
      e_n = n;
      if (e_kind != 0) {
        const int col = n - q_width - (e_kind == 2 ? kv_width : 0);
        const int g = col / hd, d = col - g * hd;
        const int logical = p / qkv.page_size;
        const int page = logical < qkv.table_width ? qkv.block_table[(size_t)slot_req * qkv.table_width + logical] : -1;
        if (page < 0 || page >= qkv.n_pages) {
          if (qkv.status) atomicOr(qkv.status, FG_STATUS_BAD_PAGE);
          e_tok = -1;
        } else {
          e_dst = (((size_t)page * qkv.n_kv_heads + g) * qkv.page_size + (p - logical * qkv.page_size)) * hd + d;
        }
      }
    }
  }
  block.first_weights();
  pdl_wait();
  block.run(red);
  if (EPI == EPI_PLAIN) {
    epilogue_plain<NT, TO>(red, y, ldy, M, N, n0);
  } else if (EPI == EPI_SWIGLU) {
    epilogue_swiglu<NT, TO>(red, y, ldy, M, N, n0);
  } else {
    // the block's 16 rows are 8 adjacent pairs of one head of q, k or v; a thread's pair,
    // angle and destination were worked out before the main loop
    if (e_tok >= 0) {
      const int pr = (e_n - n0) >> 1;
      float re = block_total<NT>(red, 2 * pr, e_tok), im = block_total<NT>(red, 2 * pr + 1, e_tok);
      if (e_kind != 2) {
        // the product is rounded to bfloat16 before the rotation, as a separate kernel would see it
        re = __bfloat162float(__float2bfloat16_rn(re));
        im = __bfloat162float(__float2bfloat16_rn(im));
        const float rr = re * e_cos - im * e_sin, ii = im * e_cos + re * e_sin;
        re = rr;
        im = ii;
      }
      const __nv_bfloat162 out2 = __floats2bfloat162_rn(re, im);
      if (e_kind == 0)
        *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(y) + (size_t)e_tok * ldy + e_n) = out2;
      else
        *reinterpret_cast<__nv_bfloat162*>((e_kind == 2 ? qkv.v_pages : qkv.k_pages) + e_dst) = out2;
    }
  }
}

template <int NT, typename TO, int EPI, int MODE = TWO_AN_SM>
int launch_one(const void* x, int ldx, const void* w, int ldw, void* y, int ldy, int M, int N, int K,
               const QkvEpilogue& qkv, cudaStream_t stream) {
  auto kern = gemm_skinny_kernel<NT, TO, EPI, MODE>;
  constexpr size_t smem = Ring<NT, MODE>::BYTES;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FG_CHECK_ARG(e == cudaSuccess, "fg_gemm_skinny: shared memory: %s", cudaGetErrorString(e));
    if (Ring<NT, MODE>::CARVEOUT) {
      e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, Ring<NT, MODE>::CARVEOUT);
      FG_CHECK_ARG(e == cudaSuccess, "fg_gemm_skinny: carve-out: %s", cudaGetErrorString(e));
    }
    attr_set = true;
  }
  fg_launch_pdl(kern, dim3((N + ROWS - 1) / ROWS), dim3(THREADS), smem, stream, (const __nv_bfloat16*)x, ldx,
                (const __nv_bfloat16*)w, ldw, (TO*)y, ldy, M, N, K, qkv);
  return 0;
}

template <typename TO, int EPI>
int launch(const void* x, int ldx, const void* w, int ldw, void* y, int ldy, int M, int N, int K,
           const QkvEpilogue& qkv, cudaStream_t stream) {
  if (M <= 8) {
    // how many blocks share an SM goes by the number of blocks (see Ring)
    static int n_sms = 0;
    if (n_sms == 0) {
      int dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const int blocks = (N + ROWS - 1) / ROWS;
    if (blocks > 2 * n_sms && blocks <= 3 * n_sms)
      return launch_one<1, TO, EPI, THREE_AN_SM>(x, ldx, w, ldw, y, ldy, M, N, K, qkv, stream);
    if (blocks <= n_sms) return launch_one<1, TO, EPI, ONE_AN_SM>(x, ldx, w, ldw, y, ldy, M, N, K, qkv, stream);
    return launch_one<1, TO, EPI>(x, ldx, w, ldw, y, ldy, M, N, K, qkv, stream);
  }
  if (M <= 16) return launch_one<2, TO, EPI>(x, ldx, w, ldw, y, ldy, M, N, K, qkv, stream);
  return launch_one<4, TO, EPI>(x, ldx, w, ldw, y, ldy, M, N, K, qkv, stream);
}

int check_common(const char* name, const void* x, int ldx, const void* w, int ldw, int ldy, int M, int N, int K,
                 int x_width) {
  FG_CHECK_ARG(M <= 32, "%s: M=%d exceeds 32", name, M);
  FG_CHECK_ARG(K > 0 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ldx >= x_width && ldw >= K && ldy >= N,
               "%s: K=%d and the row strides (%d, %d) must be multiples of 8", name, K, ldx, ldw);
  FG_CHECK_ARG(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "%s: x and w must be 16-byte aligned", name);
  return 0;
}

}  // namespace

extern "C" int fg_gemm_skinny_max_m() { return 32; }

// x: [M, K] bf16 (row stride ldx), w: [N, K] bf16 (row stride ldw), y: [M, N] bf16 or
// float32.  Needs M <= 32, K % 8 == 0, 16-byte aligned x and w with strides % 8 == 0.
extern "C" int fg_gemm_skinny_bf16(const void* x, int ldx, const void* w, int ldw, void* y, int ldy,
                                   int out_dtype, int M, int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (check_common("fg_gemm_skinny_bf16", x, ldx, w, ldw, ldy, M, N, K, K)) return -1;
  QkvEpilogue none{};
  if (out_dtype == FG_BF16)
    launch<__nv_bfloat16, EPI_PLAIN>(x, ldx, w, ldw, y, ldy, M, N, K, none, stream);
  else if (out_dtype == FG_F32)
    launch<float, EPI_PLAIN>(x, ldx, w, ldw, y, ldy, M, N, K, none, stream);
  else
    FG_CHECK_ARG(false, "fg_gemm_skinny_bf16: bad output dtype %d", out_dtype);
  FG_CHECK_LAUNCH("fg_gemm_skinny_bf16");
  return 0;
}

// y[M, F] = silu(x W1^T) * (x W3^T) for w = W1 and W3 interleaved in blocks of 8 rows
// ([2F, K]: rows 16b..16b+7 are rows 8b..8b+7 of W1, rows 16b+8..16b+15 those of W3).
extern "C" int fg_gemm_skinny_swiglu_bf16(const void* x, int ldx, const void* w, int ldw, void* y, int ldy,
                                          int M, int F, int K, cudaStream_t stream) {
  if (M == 0 || F == 0) return 0;
  FG_CHECK_ARG(F % 8 == 0, "fg_gemm_skinny_swiglu_bf16: the feed-forward width %d is not a multiple of 8", F);
  if (check_common("fg_gemm_skinny_swiglu_bf16", x, ldx, w, ldw, ldy, M, F, K, K)) return -1;
  QkvEpilogue none{};
  launch<__nv_bfloat16, EPI_SWIGLU>(x, ldx, w, ldw, y, ldy, M, 2 * F, K, none, stream);
  FG_CHECK_LAUNCH("fg_gemm_skinny_swiglu_bf16");
  return 0;
}

// The fused projection of queries, keys and values for single tokens and small
// batches: w = [wq; wk; wv] with N = (n_heads + 2 n_kv_heads) * head_dim.  Rotated
// queries go to y[:, :n_heads*head_dim]; rotated keys and the values go to the
// pages of (req[t], pos[t]).  freqs may be null (no rotation).
extern "C" int fg_gemm_skinny_qkv_bf16(const void* x, int ldx, const void* w, int ldw, void* y, int ldy,
                                       int M, int K, const int* pos, const int* req, const float* freqs,
                                       void* k_pages, void* v_pages, const int* block_table, int table_width,
                                       int page_size, int n_pages, int n_heads, int n_kv_heads, int head_dim,
                                       int* status, cudaStream_t stream) {
  const int N = (n_heads + 2 * n_kv_heads) * head_dim;
  if (M == 0) return 0;
  if (check_common("fg_gemm_skinny_qkv_bf16", x, ldx, w, ldw, ldy, M, n_heads * head_dim, K, K)) return -1;
  FG_CHECK_ARG(head_dim % 16 == 0, "fg_gemm_skinny_qkv_bf16: head size %d is not a multiple of 16", head_dim);
  FG_CHECK_ARG(ldy % 2 == 0 && ((uintptr_t)y & 3) == 0 && ((uintptr_t)k_pages & 3) == 0 &&
                   ((uintptr_t)v_pages & 3) == 0,
               "fg_gemm_skinny_qkv_bf16: outputs must be 4-byte aligned");
  QkvEpilogue qkv{pos, req, freqs, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, block_table, table_width,
                  page_size, n_pages, n_heads, n_kv_heads, head_dim, status};
  launch<__nv_bfloat16, EPI_QKV>(x, ldx, w, ldw, y, ldy, M, N, K, qkv, stream);
  FG_CHECK_LAUNCH("fg_gemm_skinny_qkv_bf16");
  return 0;
}
