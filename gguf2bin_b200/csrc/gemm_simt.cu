// True 32-bit matrix product on the CUDA cores (FFMA only, no tensor-core mode):
//   C[M,N] (=|+=) A[M,K] * W[N,K]^T        W row-major [out][in] as in the checkpoint,
// the layout the reference's GEMV reads (src/l3_math.c:17-20: row i at w + i*n_in).
// Elements of A and W may be float or bfloat16 and are widened exactly; every product
// and sum is 32-bit.  For one output element the sum runs over k in increasing order,
// whatever M is, so a row's result does not depend on the other rows of the batch.
//
// This is the product of the float32 path of the whole model, and the fallback of the
// bfloat16 path for sizes or dtypes the tensor-core kernels refuse.
#include "common.cuh"

G2B_DEFINE_LAST_ERROR

#define BM 64
#define BN 64
#define BK 16

enum { EPI_STORE_F32 = 0, EPI_STORE_BF16 = 1, EPI_ACCUM_F32 = 2 };

template <typename TA, typename TW, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA *__restrict__ A, const TW *__restrict__ W, void *__restrict__ Cv, int M,
                 int N, int K, int lda, int ldw, int ldc) {
  pdl_launch();
  pdl_wait();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // each thread loads 4 elements of each tile: row = e/BK, col = e%BK
#pragma unroll
    for (int e = tid; e < BM * BK; e += 256) {
      const int r = e / BK, c = e % BK;
      const int gm = m0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
      const int gn = n0 + r;
      Ws[c][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      const size_t o = (size_t)gm * ldc + gn;
      if (EPI == EPI_STORE_F32) ((float *)Cv)[o] = acc[i][j];
      else if (EPI == EPI_STORE_BF16) ((bf16 *)Cv)[o] = __float2bfloat16_rn(acc[i][j]);
      else ((float *)Cv)[o] += acc[i][j];
    }
  }
}

template <typename TA, typename TW>
static int launch(const void *A, const void *W, void *C, int M, int N, int K, int lda, int ldw,
                  int ldc, int epi, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) G2B_REFUSE("gemm_simt: M=%d is too large for one launch", M);
  switch (epi) {
    case EPI_STORE_F32:
      g2b_launch(gemm_simt_kernel<TA, TW, EPI_STORE_F32>, dim3(grid), dim3(256), 0, stream, 
          (const TA *)A, (const TW *)W, C, M, N, K, lda, ldw, ldc);
      break;
    case EPI_STORE_BF16:
      g2b_launch(gemm_simt_kernel<TA, TW, EPI_STORE_BF16>, dim3(grid), dim3(256), 0, stream, 
          (const TA *)A, (const TW *)W, C, M, N, K, lda, ldw, ldc);
      break;
    case EPI_ACCUM_F32:
      g2b_launch(gemm_simt_kernel<TA, TW, EPI_ACCUM_F32>, dim3(grid), dim3(256), 0, stream, 
          (const TA *)A, (const TW *)W, C, M, N, K, lda, ldw, ldc);
      break;
    default:
      G2B_REFUSE("gemm_simt: unknown epilogue %d", epi);
  }
  return g2b_check_launch("gemm_simt");
}

// epi: 0 store float, 1 store bfloat16, 2 add into float
extern "C" int g2b_gemm_simt(const void *A, int a_dtype, const void *W, int w_dtype, void *C,
                             int M, int N, int K, int lda, int ldw, int ldc, int epi,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) G2B_REFUSE("gemm_simt: K=%d", K);
  if (a_dtype == G2B_F32 && w_dtype == G2B_F32)
    return launch<float, float>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
  if (a_dtype == G2B_BF16 && w_dtype == G2B_BF16)
    return launch<bf16, bf16>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
  if (a_dtype == G2B_BF16 && w_dtype == G2B_F32)
    return launch<bf16, float>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
  if (a_dtype == G2B_F32 && w_dtype == G2B_BF16)
    return launch<float, bf16>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
  G2B_REFUSE("gemm_simt: unknown dtypes %d, %d", a_dtype, w_dtype);
}
