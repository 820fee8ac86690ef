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

// The output's type is looked at when a result is stored, not compiled in: eight variants of
// every kernel less to build.
__device__ __forceinline__ void put_out(void* C, int c_bf16, size_t at, float v, bool add) {
  if (c_bf16) {
    ((__nv_bfloat16*)C)[at] = __float2bfloat16_rn(v);  // a residual add is float32 only
  } else {
    float* out = (float*)C + at;
    *out = add ? *out + v : v;
  }
}

template <typename TA, typename TW, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, void* __restrict__ C,
                 int c_bf16, int ldc, int M, int N, int K) {
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
      const size_t at = (size_t)gm * ldc + gn;
      if (EPI == EPI_STORE || EPI == EPI_ADD) {
        put_out(C, c_bf16, at, acc[0][i][j], EPI == EPI_ADD);
      } else {
        const float g = acc[0][i][j];
        put_out(C, c_bf16, at, g / (1.0f + expf(-g)) * acc[NW - 1][i][j], false);
      }
    }
  }
}

// ---------------------------------------------------------------------------- few rows
// The same product for at most 16 rows of A (a decode step): the weight streams through once.
// A warp owns four weight rows (four output features, or two with their gate and up rows) and
// walks K in chunks of 128 (every lane 4 consecutive values of each of its rows, 16 bytes of
// float32), against up to eight rows of A at a time; 32 sums a warp, reduced by shuffles.
// a weight row's values are used once: they pass by the L1 cache, which keeps the rows of A
template <typename T> __device__ __forceinline__ float4 load4_once(const T* p);
template <> __device__ __forceinline__ float4 load4_once<float>(const float* p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
template <> __device__ __forceinline__ float4 load4_once<__nv_bfloat16>(const __nv_bfloat16* p) {
  uint2 raw;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];"
               : "=r"(raw.x), "=r"(raw.y)
               : "l"(p));
  const float2 lo = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x);
  const float2 hi = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

#define FEW_ROWS 8   // rows of A in one pass
#define FEW_MAX 16   // the most rows that take this kernel

template <typename TA, typename TW, int EPI>
__global__ void __launch_bounds__(256)
gemm_few_rows_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W,
                     void* __restrict__ C, int c_bf16, int ldc, int M, int N, int K) {
  constexpr bool GLU = EPI == EPI_SWIGLU || EPI == EPI_SWIGLU_PAIRS;
  constexpr int FEATS = GLU ? 2 : 4;  // output features of a warp
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * 8 + warp) * FEATS;
  if (n0 >= N) return;
  // the warp's four weight rows; a row beyond the weight is read as row n0's and not stored
  const TW* wr[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int row;
    if (EPI == EPI_SWIGLU) row = (j >> 1) * N + min(n0 + (j & 1), N - 1);     // g0 g1 u0 u1
    else if (EPI == EPI_SWIGLU_PAIRS) row = 2 * min(n0 + (j >> 1), N - 1) + (j & 1);  // g0 u0 g1 u1
    else row = min(n0 + j, N - 1);
    wr[j] = W + (size_t)row * K;
  }
  for (int m0 = 0; m0 < M; m0 += FEW_ROWS) {
    float acc[4][FEW_ROWS];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int m = 0; m < FEW_ROWS; ++m) acc[j][m] = 0.f;
    for (int k = lane * 4; k < K; k += 128) {
      float4 w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = load4_once<TW>(wr[j] + k);
#pragma unroll
      for (int m = 0; m < FEW_ROWS; ++m) {
        if (m0 + m >= M) break;  // uniform over the warp
        const float4 a = load4<TA>(A + (size_t)(m0 + m) * lda + k);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc[j][m] = fmaf(a.x, w[j].x, fmaf(a.y, w[j].y, fmaf(a.z, w[j].z, fmaf(a.w, w[j].w, acc[j][m]))));
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int m = 0; m < FEW_ROWS; ++m) acc[j][m] = warp_sum(acc[j][m]);
    // lane m stores row m0 + m
#pragma unroll
    for (int m = 0; m < FEW_ROWS; ++m) {
      if (lane != m || m0 + m >= M) continue;
#pragma unroll
      for (int f = 0; f < FEATS; ++f) {
        if (n0 + f >= N) continue;
        const size_t at = (size_t)(m0 + m) * ldc + n0 + f;
        if (EPI == EPI_STORE || EPI == EPI_ADD) {
          put_out(C, c_bf16, at, acc[f][m], EPI == EPI_ADD);
        } else {
          const float g = EPI == EPI_SWIGLU ? acc[f][m] : acc[2 * f][m];
          const float u = EPI == EPI_SWIGLU ? acc[2 + f][m] : acc[2 * f + 1][m];
          put_out(C, c_bf16, at, g / (1.0f + expf(-g)) * u, false);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------- many rows
// The same product for many rows: 128 x 128 tiles, 8 x 8 results a thread (two 4 x 4 quarters
// 64 apart in each direction, so that the shared-memory reads are 16 bytes wide and free of
// bank conflicts), K in steps of 16 through two buffers with the next step's global loads under
// way while this one is multiplied. Epilogues: store, residual add, and SwiGLU over weight rows
// that alternate gate and up (NW = 2 N weight rows, neighbouring columns of the tile pair up).
#define LM 128
#define LN 128
#define LK 16

// four values k .. k + 3 of a row as float32, zeros beyond K or for a row that does not exist
template <typename T>
__device__ __forceinline__ float4 row_piece(const T* __restrict__ base, bool row_ok, int k, int K,
                                            bool vec) {
  if (!row_ok || k >= K) return make_float4(0.f, 0.f, 0.f, 0.f);
  if (vec) return load4<T>(base + k);
  float4 v;
  v.x = to_f32<T>(base[k]);
  v.y = k + 1 < K ? to_f32<T>(base[k + 1]) : 0.f;
  v.z = k + 2 < K ? to_f32<T>(base[k + 2]) : 0.f;
  v.w = k + 3 < K ? to_f32<T>(base[k + 3]) : 0.f;
  return v;
}

template <typename TA, typename TW, int EPI>
__global__ void __launch_bounds__(256)
gemm_many_rows_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W,
                      void* __restrict__ C, int c_bf16, int ldc, int M, int NW, int K, int vec_a,
                      int vec_w) {
  __shared__ __align__(16) float As[2][LK][LM + 4];
  __shared__ __align__(16) float Ws[2][LK][LN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * LM, n0 = blockIdx.x * LN;
  // loads: thread t brings values 8 (t % 2) .. + 7 of row t / 2 of both tiles
  const int lr = tid >> 1, lk = (tid & 1) * 8;
  const bool a_ok = m0 + lr < M, w_ok = n0 + lr < NW;
  const TA* arow = A + (size_t)(m0 + lr) * lda;
  const TW* wrow = W + (size_t)(n0 + lr) * K;
  const int ty = tid >> 4, tx = tid & 15;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  float4 ra[2], rw[2];
  auto fetch = [&](int k) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      ra[h] = row_piece<TA>(arow, a_ok, k + lk + 4 * h, K, vec_a);
      rw[h] = row_piece<TW>(wrow, w_ok, k + lk + 4 * h, K, vec_w);
    }
  };
  auto put = [&](int buf) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int k = lk + 4 * h;
      As[buf][k][lr] = ra[h].x; As[buf][k + 1][lr] = ra[h].y;
      As[buf][k + 2][lr] = ra[h].z; As[buf][k + 3][lr] = ra[h].w;
      Ws[buf][k][lr] = rw[h].x; Ws[buf][k + 1][lr] = rw[h].y;
      Ws[buf][k + 2][lr] = rw[h].z; Ws[buf][k + 3][lr] = rw[h].w;
    }
  };
  int cur = 0;
  fetch(0);
  put(0);
  __syncthreads();
  for (int k0 = 0; k0 < K; k0 += LK) {
    const bool more = k0 + LK < K;
    if (more) fetch(k0 + LK);
#pragma unroll
    for (int k = 0; k < LK; ++k) {
      const float4 a0 = *(const float4*)&As[cur][k][ty * 4], a1 = *(const float4*)&As[cur][k][64 + ty * 4];
      const float4 b0 = *(const float4*)&Ws[cur][k][tx * 4], b1 = *(const float4*)&Ws[cur][k][64 + tx * 4];
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (more) {
      put(cur ^ 1);
      __syncthreads();
      cur ^= 1;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gm = m0 + (i >> 2) * 64 + ty * 4 + (i & 3);
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int gn = n0 + (j >> 2) * 64 + tx * 4 + (j & 3);
      if (gn >= NW) continue;
      if (EPI == EPI_SWIGLU_PAIRS) {
        if (j & 1) continue;  // gate at the even weight row, up at the odd one after it
        const float g = acc[i][j];
        put_out(C, c_bf16, (size_t)gm * ldc + (gn >> 1), g / (1.0f + expf(-g)) * acc[i][j + 1], false);
      } else {
        put_out(C, c_bf16, (size_t)gm * ldc + gn, acc[i][j], EPI == EPI_ADD);
      }
    }
  }
}

template <typename TA, typename TW>
static int launch(const void* A, int lda, const void* W, void* C, int c_bf16, int ldc, int M, int N,
                  int K, int epi, cudaStream_t s) {
  // few rows, and every row piece of 4 values a whole aligned load
  const int a_align = sizeof(TA) == 4 ? 15 : 7, w_align = sizeof(TW) == 4 ? 15 : 7;
  if (M <= FEW_MAX && K % 4 == 0 && lda % 4 == 0 && ((uintptr_t)A & a_align) == 0 &&
      ((uintptr_t)W & w_align) == 0) {
    const int feats = (epi == EPI_SWIGLU || epi == EPI_SWIGLU_PAIRS) ? 2 : 4;
    const int blocks = (N + 8 * feats - 1) / (8 * feats);
#define FEW(E)                                                                                \
  gemm_few_rows_kernel<TA, TW, E><<<blocks, 256, 0, s>>>((const TA*)A, lda, (const TW*)W, C,  \
                                                         c_bf16, ldc, M, N, K)
    if (epi == EPI_STORE) FEW(EPI_STORE);
    else if (epi == EPI_ADD) FEW(EPI_ADD);
    else if (epi == EPI_SWIGLU) FEW(EPI_SWIGLU);
    else FEW(EPI_SWIGLU_PAIRS);
#undef FEW
    MB_CHECK_LAUNCH("mb_gemm_simt");
  }
  if (M >= 64 && epi != EPI_SWIGLU) {
    const int NW = epi == EPI_SWIGLU_PAIRS ? 2 * N : N;
    dim3 big((NW + LN - 1) / LN, (M + LM - 1) / LM);
    if (big.y > 65535) MB_FAIL("mb_gemm_simt: %d rows are too many for one launch", M);
    const int vec_a = K % 4 == 0 && lda % 4 == 0 && ((uintptr_t)A & a_align) == 0;
    const int vec_w = K % 4 == 0 && ((uintptr_t)W & w_align) == 0;
#define MANY(E)                                                                               \
  gemm_many_rows_kernel<TA, TW, E><<<big, 256, 0, s>>>((const TA*)A, lda, (const TW*)W, C,    \
                                                       c_bf16, ldc, M, NW, K, vec_a, vec_w)
    if (epi == EPI_STORE) MANY(EPI_STORE);
    else if (epi == EPI_ADD) MANY(EPI_ADD);
    else MANY(EPI_SWIGLU_PAIRS);
#undef MANY
    MB_CHECK_LAUNCH("mb_gemm_simt");
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) MB_FAIL("mb_gemm_simt: %d rows are too many for one launch", M);
#define GO(E)                                                                                  \
  gemm_simt_kernel<TA, TW, E><<<grid, 256, 0, s>>>((const TA*)A, lda, (const TW*)W, C, c_bf16,  \
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
  const int c_bf16 = c_dtype == MB_BF16;
  if (a_dtype == MB_F32 && w_dtype == MB_F32)
    return launch<float, float>(A, lda, W, C, c_bf16, ldc, M, N, K, epilogue, s);
  if (a_dtype == MB_F32) return launch<float, bf>(A, lda, W, C, c_bf16, ldc, M, N, K, epilogue, s);
  if (w_dtype == MB_F32) return launch<bf, float>(A, lda, W, C, c_bf16, ldc, M, N, K, epilogue, s);
  return launch<bf, bf>(A, lda, W, C, c_bf16, ldc, M, N, K, epilogue, s);
}
