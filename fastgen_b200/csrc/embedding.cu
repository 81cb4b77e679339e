// Token embedding: out[t, :] = table[token[t], :].
// Replaces F.embedding of fastgen/forward.py:403-410.  The output is the
// residual stream, which the engine keeps in float32 in every mode.
#include "common.cuh"

template <typename TT, typename TO>
__global__ void embedding_kernel(const TT* __restrict__ table, const int* __restrict__ tokens,
                                 TO* __restrict__ out, int dim, int vocab, int* status) {
  const int t = blockIdx.x;
  int tok = tokens[t];
  if (tok < 0 || tok >= vocab) {
    if (threadIdx.x == 0 && status) atomicOr(status, FG_STATUS_BAD_TOKEN);
    for (int d = threadIdx.x; d < dim; d += blockDim.x) out[(size_t)t * dim + d] = from_f32<TO>(0.f);
    return;
  }
  const TT* row = table + (size_t)tok * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x)
    out[(size_t)t * dim + d] = from_f32<TO>(to_f32<TT>(row[d]));
}

extern "C" int fg_embedding(const void* table, int table_dtype, const int* tokens, void* out,
                            int out_dtype, int n_tokens, int dim, int vocab, int* status,
                            cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  FG_CHECK_ARG(dim > 0 && vocab > 0, "fg_embedding: bad sizes dim=%d vocab=%d", dim, vocab);
  const int threads = dim >= 1024 ? 256 : 128;
#define LAUNCH(TT, TO)                                                        \
  embedding_kernel<TT, TO><<<n_tokens, threads, 0, stream>>>(                 \
      (const TT*)table, tokens, (TO*)out, dim, vocab, status)
  if (table_dtype == FG_F32 && out_dtype == FG_F32) LAUNCH(float, float);
  else if (table_dtype == FG_BF16 && out_dtype == FG_F32) LAUNCH(__nv_bfloat16, float);
  else if (table_dtype == FG_BF16 && out_dtype == FG_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (table_dtype == FG_F32 && out_dtype == FG_BF16) LAUNCH(float, __nv_bfloat16);
  else FG_CHECK_ARG(false, "fg_embedding: bad dtypes %d %d", table_dtype, out_dtype);
#undef LAUNCH
  FG_CHECK_LAUNCH("fg_embedding");
  return 0;
}
