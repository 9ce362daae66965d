// True 32-bit matrix product for the float32 path:  C[M,N] = A[M,K] . W[N,K]^T
// (the linear layers' y = x . W^T with W stored [out, in]; upstream does this with
// cublasGemmEx on bfloat16, base/src/engine.cu:643-671).
//
// Plain FMA on CUDA cores, no tensor cores: a tf32 product would drop mantissa bits
// and this path exists to show what bfloat16 hides.  Every output element is one
// chain of fmaf over k = 0..K-1 in ascending order, so a row's result does not
// depend on how many other rows the call holds or on which tile it falls into.
#include "common.cuh"

constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256)
sgemm_nt_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw,
                float* __restrict__ C, int ldc, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // loader: 64 rows x 16 k = 1024 elements per operand, 4 per thread
  const int lrow = tid >> 2;        // 0..63
  const int lk = (tid & 3) * 4;     // 0,4,8,12
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lk + u;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + u][lrow] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
      Ws[lk + u][lrow] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}

// Padding k beyond K with zeros adds exact zeros to the chain, so the result equals
// the unpadded chain.  Any M, N, K >= 1; leading dimensions in elements.
KVB_EXPORT int kvb_sgemm_nt(const float* A, int lda, const float* W, int ldw, float* C, int ldc,
                            int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return KVB_ERR_BAD_SIZE;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return KVB_ERR_BAD_SIZE;
  sgemm_nt_kernel<<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, M, N, K);
  return kvb_launch_result();
}
