// Weight-streaming matrix product for a few tokens (decode):
//   y[M, N] = x[M, K] * W[N, K]^T,  bfloat16 inputs, float32 accumulation, M <= 32.
//
// With so few tokens the product is bound by reading W once from HBM.  The roles
// of the operands are swapped for the tensor core: 16 rows of W are the "M" side
// of mma.sync m16n8k16 and 8 tokens the "N" side, so no row of the instruction is
// wasted on padding.  Fragments are loaded straight from global memory with
// 16-byte loads (the k index inside an instruction is permuted identically for
// both operands, which does not change the sum), so there is no shared-memory
// staging and no barrier in the main loop; each thread keeps several loads in
// flight.  A block owns 16 rows of W; its 8 warps split K in interleaved chunks
// of 64 and are summed in warp order at the end, so a row's result depends on
// nothing but K.
//
// It stands where the reference calls F.linear on decode batches
// (fastgen/forward.py:438-440,470,491-496,513); larger M goes to the library.
#include "common.cuh"

namespace {

constexpr int ROWS = 16;   // rows of W per block
constexpr int CHUNK = 64;  // k elements per warp step

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_keep(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                    uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT, typename TO, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ w, int ldw,
                   TO* __restrict__ y, int ldy, int M, int N, int K) {
  __shared__ float red[WARPS][ROWS][NT * 8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = blockIdx.x * ROWS;
  const int r = lane >> 2, c = lane & 3;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  // rows beyond N and tokens beyond M read row 0 and are discarded at the end
  const bool row_a = n0 + r < N, row_b = n0 + r + 8 < N;
  const __nv_bfloat16* wa = w + (size_t)(row_a ? n0 + r : 0) * ldw + c * 8;
  const __nv_bfloat16* wb = w + (size_t)(row_b ? n0 + r + 8 : 0) * ldw + c * 8;
  const __nv_bfloat16* xr[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int tok = nt * 8 + r;
    xr[nt] = x + (size_t)(tok < M ? tok : 0) * ldx + c * 8;
  }
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

  constexpr int UNROLL = NT <= 2 ? 4 : 2;
  const int n_full = K / CHUNK;  // whole chunks: loads without predicates
  int ch = warp;
  // main loop: UNROLL chunks per warp step, every load issued before the first product
  for (; ch + (UNROLL - 1) * WARPS < n_full; ch += WARPS * UNROLL) {
    uint4 a_lo[UNROLL][2], a_hi[UNROLL][2], b[UNROLL][NT][2];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (ch + u * WARPS) * CHUNK;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        a_lo[u][h] = ldg_stream(wa + k + h * 32);
        a_hi[u][h] = ldg_stream(wb + k + h * 32);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) b[u][nt][h] = ldg_keep(xr[nt] + k + h * 32);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          mma(acc[nt], a_lo[u][h].x, a_hi[u][h].x, a_lo[u][h].y, a_hi[u][h].y, b[u][nt][h].x, b[u][nt][h].y);
          mma(acc[nt], a_lo[u][h].z, a_hi[u][h].z, a_lo[u][h].w, a_hi[u][h].w, b[u][nt][h].z, b[u][nt][h].w);
        }
  }
  // the remaining chunks, the last of which may be partial (K is a multiple of 8,
  // so a 16-byte piece is all in or all out)
  const int n_chunks = (K + CHUNK - 1) / CHUNK;
  for (; ch < n_chunks; ch += WARPS) {
    const int k = ch * CHUNK;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int kk = k + h * 32;
      const bool ok = kk + c * 8 < K;
      const int ks = ok ? kk : 0;
      uint4 al = ldg_stream(wa + ks), ah = ldg_stream(wb + ks);
      if (!ok) al = ah = zero;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        uint4 bb = ldg_keep(xr[nt] + ks);
        if (!ok) bb = zero;
        mma(acc[nt], al.x, ah.x, al.y, ah.y, bb.x, bb.y);
        mma(acc[nt], al.z, ah.z, al.w, ah.w, bb.z, bb.w);
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    red[warp][r][nt * 8 + 2 * c] = acc[nt][0];
    red[warp][r][nt * 8 + 2 * c + 1] = acc[nt][1];
    red[warp][r + 8][nt * 8 + 2 * c] = acc[nt][2];
    red[warp][r + 8][nt * 8 + 2 * c + 1] = acc[nt][3];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < ROWS * NT * 8; i += WARPS * 32) {
    const int tok = i / ROWS, row = i - tok * ROWS;  // consecutive threads write consecutive columns of y
    if (tok < M && n0 + row < N) {
      float s = 0.f;
#pragma unroll
      for (int wi = 0; wi < WARPS; ++wi) s += red[wi][row][tok];
      y[(size_t)tok * ldy + n0 + row] = from_f32<TO>(s);
    }
  }
}

template <typename TO>
int launch(const void* x, int ldx, const void* w, int ldw, void* y, int ldy, int M, int N, int K,
           cudaStream_t stream) {
  const int grid = (N + ROWS - 1) / ROWS;
  const auto* xp = (const __nv_bfloat16*)x;
  const auto* wp = (const __nv_bfloat16*)w;
  // Few blocks (a small N): 16 warps a block, so that enough loads are in flight
  // on every SM; the split of K only depends on N and K, never on the batch.
  const bool wide = grid < 4 * 148 && K >= 16 * CHUNK;
#define FG_SKINNY(NT)                                                                                       \
  do {                                                                                                      \
    if (wide)                                                                                               \
      gemm_skinny_kernel<NT, TO, 16><<<grid, 16 * 32, 0, stream>>>(xp, ldx, wp, ldw, (TO*)y, ldy, M, N, K); \
    else                                                                                                    \
      gemm_skinny_kernel<NT, TO, 8><<<grid, 8 * 32, 0, stream>>>(xp, ldx, wp, ldw, (TO*)y, ldy, M, N, K);   \
  } while (0)
  if (M <= 8)
    FG_SKINNY(1);
  else if (M <= 16)
    FG_SKINNY(2);
  else
    FG_SKINNY(4);
#undef FG_SKINNY
  return 0;
}

}  // namespace

extern "C" int fg_gemm_skinny_max_m() { return 32; }

// x: [M, K] bf16 (row stride ldx), w: [N, K] bf16 (row stride ldw), y: [M, N] bf16 or
// float32.  Needs M <= 32, K % 8 == 0, 16-byte aligned x and w with strides % 8 == 0.
extern "C" int fg_gemm_skinny_bf16(const void* x, int ldx, const void* w, int ldw, void* y, int ldy,
                                   int out_dtype, int M, int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  FG_CHECK_ARG(M <= 32, "fg_gemm_skinny_bf16: M=%d exceeds 32", M);
  FG_CHECK_ARG(K > 0 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ldx >= K && ldw >= K && ldy >= N,
               "fg_gemm_skinny_bf16: K=%d and the row strides (%d, %d) must be multiples of 8", K, ldx, ldw);
  FG_CHECK_ARG(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0,
               "fg_gemm_skinny_bf16: x and w must be 16-byte aligned");
  if (out_dtype == FG_BF16)
    launch<__nv_bfloat16>(x, ldx, w, ldw, y, ldy, M, N, K, stream);
  else if (out_dtype == FG_F32)
    launch<float>(x, ldx, w, ldw, y, ldy, M, N, K, stream);
  else
    FG_CHECK_ARG(false, "fg_gemm_skinny_bf16: bad output dtype %d", out_dtype);
  FG_CHECK_LAUNCH("fg_gemm_skinny_bf16");
  return 0;
}
