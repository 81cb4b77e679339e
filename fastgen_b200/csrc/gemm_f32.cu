// True 32-bit matrix product  C[M, N] = A[M, K] * W[N, K]^T  on the CUDA cores.
//
// This is the GEMM of the float32 path: IEEE float32 fused multiply-adds, no
// tensor cores and no reduced-precision mode.  Every output element is the sum
// over k = 0 .. K-1 in ascending order in a single accumulator, so its value
// does not depend on M, on the tile it falls in, or on what else is in the batch.
// It stands where the reference calls F.linear (fastgen/forward.py:438-440,470,
// 491-496,513).
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each

__global__ void __launch_bounds__(256)
gemm_f32_nt_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw,
                   float* __restrict__ C, int ldc, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // tx: column group, ty: row group
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // each thread loads 4 elements of A and 4 of W per k-tile
  const int lr = tid >> 2;        // 0..63 row within tile
  const int lk = (tid & 3) * 4;   // 0,4,8,12
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int kk = k0 + lk + u;
      const int am = m0 + lr, wn = n0 + lr;
      As[lk + u][lr] = (am < M && kk < K) ? A[(size_t)am * lda + kk] : 0.f;
      Ws[lk + u][lr] = (wn < N && kk < K) ? W[(size_t)wn * ldw + kk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}
}  // namespace

extern "C" int fg_gemm_f32_nt(const float* A, int lda, const float* W, int ldw, float* C, int ldc,
                              int M, int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  FG_CHECK_ARG(K > 0 && lda >= K && ldw >= K && ldc >= N, "fg_gemm_f32_nt: bad sizes M=%d N=%d K=%d", M, N, K);
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  FG_CHECK_ARG(grid.y <= 65535, "fg_gemm_f32_nt: M=%d too large", M);
  gemm_f32_nt_kernel<<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, M, N, K);
  FG_CHECK_LAUNCH("fg_gemm_f32_nt");
  return 0;
}
