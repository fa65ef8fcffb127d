// out[M,N] (+)= a[M,K] * w[N,K]^T on the ordinary (non-tensor) cores, with true
// 32-bit multiply-adds: the matrix product of the 32-bit path, and the check
// beside the tensor-core kernels. garuda/src/simd/mod.rs:96-129 (`matmul`: each
// output is the dot of one matrix row with one input vector, :13-16).
//
// Every output element is one thread's sum over k = 0..K-1 in that order,
// whatever M is, so a token's result does not depend on the rest of the batch.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each

template <typename IT, typename OT, bool ACCUMULATE>
__global__ void __launch_bounds__(256)
gemm_simple_kernel(const IT* __restrict__ a, const IT* __restrict__ w, OT* __restrict__ out, int M, int N,
                   int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tm = (tid / 16) * TM, tn = (tid % 16) * TN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 columns per operand: 1024 elements, 4 per thread
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      const int r = e / BK, c = e % BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? gb::to_float<IT>(a[(size_t)gm * K + gk]) : 0.f;
      Ws[c][r] = (gn < N && gk < K) ? gb::to_float<IT>(w[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float av[TM], wv[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) av[i] = As[k][tm + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) wv[j] = Ws[k][tn + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + tm + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tn + j;
      if (gn >= N) continue;
      OT* o = out + (size_t)gm * N + gn;
      if (ACCUMULATE) *o = gb::from_float<OT>(gb::to_float<OT>(*o) + acc[i][j]);
      else *o = gb::from_float<OT>(acc[i][j]);
    }
  }
}

}  // namespace

// in_dtype: dtype of a and w; out_dtype: dtype of out. accumulate: out += product
// (out must then be 32-bit: it is the residual stream).
GB_EXPORT int gb_gemm_simple(const void* a, const void* w, void* out, int M, int N, int K, int in_dtype,
                             int out_dtype, int accumulate, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return GB_OK;
  if (K <= 0) return gb::fail(GB_BAD_ARGUMENT, "gemm: K = %d", K);
  if (accumulate && out_dtype != GB_F32)
    return gb::fail(GB_BAD_ARGUMENT, "gemm: accumulation needs a 32-bit output");
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  return GB_DISPATCH_DTYPE(in_dtype, IT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      if (accumulate)
        gemm_simple_kernel<IT, OT, true><<<grid, 256, 0, stream>>>((const IT*)a, (const IT*)w, (OT*)out, M, N, K);
      else
        gemm_simple_kernel<IT, OT, false><<<grid, 256, 0, stream>>>((const IT*)a, (const IT*)w, (OT*)out, M, N, K);
      return gb::check_launch("gemm_simple");
    });
  });
}
