// y = x · Wᵀ for a weight [N, K] and any M, N, K and any mix of float32 / bfloat16 operands,
// with float32 multiply-adds on the CUDA cores (no tensor-core or reduced-precision mode):
// the matrix product of the true 32-bit path, and the fallback for sizes that the
// tensor-core kernels refuse. The role of the reference's `gemm8` and `linear8`
// (tools/cuda/linear.cu:418-463, :517-606 of the reference project), without its
// quantized formats.
//
// Epilogues: store; add into a float32 residual; SwiGLU over a weight [2N, K] (out =
// silu(gate) * up) whose rows are either [0, N) gate and [N, 2N) up, or alternate gate, up,
// gate, up ... (the layout that the tensor-core kernel's fused epilogue uses).
#include "common.cuh"

MB_DEFINE_LAST_ERROR

enum { EPI_STORE = 0, EPI_ADD = 1, EPI_SWIGLU = 2, EPI_SWIGLU_PAIRS = 3 };

#define BM 64
#define BN 64
#define BK 16

template <typename TA, typename TW, typename TC, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, TC* __restrict__ C,
                 int ldc, int M, int N, int K) {
  constexpr int NW = (EPI == EPI_SWIGLU || EPI == EPI_SWIGLU_PAIRS) ? 2 : 1;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[NW][BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tr = (tid / 16) * 4, tc = (tid % 16) * 4;
  float acc[NW][4][4];
#pragma unroll
  for (int w = 0; w < NW; ++w)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[w][i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 x 16 elements per tile, 256 threads: 4 each
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      const int r = e / BK, c = e % BK;
      const int gm = m0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? to_f32<TA>(A[(size_t)gm * lda + gk]) : 0.f;
      const int gn = n0 + r;
#pragma unroll
      for (int w = 0; w < NW; ++w)
        Ws[w][c][r] = (gn < N && gk < K)
                          ? to_f32<TW>(W[(EPI == EPI_SWIGLU_PAIRS ? (size_t)gn * 2 + w
                                                                   : (size_t)w * N + gn) * K + gk])
                          : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][tr + i];
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        float b[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Ws[w][k][tc + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[w][i][j] = fmaf(a[i], b[j], acc[w][i][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + tr + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tc + j;
      if (gn >= N) continue;
      TC* out = C + (size_t)gm * ldc + gn;
      if (EPI == EPI_STORE) {
        *out = from_f32<TC>(acc[0][i][j]);
      } else if (EPI == EPI_ADD) {
        *out = from_f32<TC>(to_f32<TC>(*out) + acc[0][i][j]);
      } else {
        const float g = acc[0][i][j];
        const float b = g / (1.0f + expf(-g));
        *out = from_f32<TC>(b * acc[NW - 1][i][j]);
      }
    }
  }
}

template <typename TA, typename TW, typename TC>
static int launch(const void* A, int lda, const void* W, void* C, int ldc, int M, int N, int K,
                  int epi, cudaStream_t s) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) MB_FAIL("mb_gemm_simt: %d rows are too many for one launch", M);
#define GO(E)                                                                                  \
  gemm_simt_kernel<TA, TW, TC, E><<<grid, 256, 0, s>>>((const TA*)A, lda, (const TW*)W, (TC*)C, \
                                                       ldc, M, N, K)
  if (epi == EPI_STORE) GO(EPI_STORE);
  else if (epi == EPI_ADD) GO(EPI_ADD);
  else if (epi == EPI_SWIGLU) GO(EPI_SWIGLU);
  else GO(EPI_SWIGLU_PAIRS);
#undef GO
  MB_CHECK_LAUNCH("mb_gemm_simt");
}

// C[M, N] (row stride ldc) = A[M, K] (row stride lda) · W[N, K]ᵀ. For EPI_ADD, C must be
// float32. For the SwiGLU epilogues, W is [2N, K].
MB_EXPORT int mb_gemm_simt(const void* A, int a_dtype, int lda, const void* W, int w_dtype,
                           void* C, int c_dtype, int ldc, int M, int N, int K, int epilogue,
                           void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) MB_FAIL("mb_gemm_simt: K = %d", K);
  if (epilogue < 0 || epilogue > 3) MB_FAIL("mb_gemm_simt: epilogue %d", epilogue);
  if (epilogue == EPI_ADD && c_dtype != MB_F32) MB_FAIL("mb_gemm_simt: the residual is float32");
  cudaStream_t s = (cudaStream_t)stream;
  typedef __nv_bfloat16 bf;
  const int key = (a_dtype << 2) | (w_dtype << 1) | c_dtype;
  switch (key) {
    case 0: return launch<float, float, float>(A, lda, W, C, ldc, M, N, K, epilogue, s);
    case 1: return launch<float, float, bf>(A, lda, W, C, ldc, M, N, K, epilogue, s);
    case 2: return launch<float, bf, float>(A, lda, W, C, ldc, M, N, K, epilogue, s);
    case 3: return launch<float, bf, bf>(A, lda, W, C, ldc, M, N, K, epilogue, s);
    case 4: return launch<bf, float, float>(A, lda, W, C, ldc, M, N, K, epilogue, s);
    case 5: return launch<bf, float, bf>(A, lda, W, C, ldc, M, N, K, epilogue, s);
    case 6: return launch<bf, bf, float>(A, lda, W, C, ldc, M, N, K, epilogue, s);
    default: return launch<bf, bf, bf>(A, lda, W, C, ldc, M, N, K, epilogue, s);
  }
}
