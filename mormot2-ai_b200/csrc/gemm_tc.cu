// y = x · Wᵀ for bfloat16 x [M, K] and W [N, K] on the fifth-generation tensor cores:
// operand tiles brought to shared memory by TMA (128-byte swizzle), tcgen05.mma issued by one
// thread with the float32 accumulator in tensor memory, tcgen05.ld for the epilogue.
//
// One kernel serves prefill and decode. The operand on the MMA's M side fills the 128 TMEM
// lanes of a tile, the other one its columns (16 to 256):
//   many tokens (prefill):  tokens on the lanes, output features on the columns;
//   few tokens (decode):    the WEIGHT rows on the lanes and the tokens on the columns, so that
//                           a step streams each weight byte once through full-width MMAs,
//                           whatever the batch; the tile is written back transposed.
// When there are fewer tiles than SMs the K range is split over more CTAs; the partial sums
// go to a float32 workspace that the caller provides and are added up in split order by a
// second kernel (deterministic, no atomics).
//
// Warp roles in a CTA of 192 threads: warp 0 loads (one elected lane), warp 1 allocates TMEM
// and issues the MMAs (one elected lane), warps 2-5 read the accumulator and store.
//
// This replaces the reference's `gemm8` / `linear8` (tools/cuda/linear.cu:418-606 of the
// reference project), which multiply in float32 on the CUDA cores.
#include "tc_common.cuh"

MB_DEFINE_LAST_ERROR

static thread_local int g_last_launches = 0;
// kernels that the last mb_gemm_tc of this thread launched (2 when K was split)
MB_EXPORT int mb_gemm_tc_last_launches() { return g_last_launches; }

enum { TC_STORE = 0, TC_ADD = 1, TC_PARTIAL = 2 };

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_SMEM_BUDGET (200 * 1024)

template <int BN> struct TcCfg {
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int RAW = TC_SMEM_BUDGET / (A_BYTES + B_BYTES);
  static constexpr int STAGES = RAW > 10 ? 10 : RAW;
  static constexpr int COLS = BN < 32 ? 32 : BN;  // TMEM columns: a power of two >= 32
  static constexpr int SMEM = STAGES * (A_BYTES + B_BYTES) + 1024 /*alignment*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void store_out(void* C, int c_dtype, size_t idx, float v, int mode) {
  if (c_dtype == MB_F32) {
    float* p = (float*)C + idx;
    *p = mode == TC_ADD ? *p + v : v;
  } else {
    ((__nv_bfloat16*)C)[idx] = __float2bfloat16_rn(v);
  }
}

// rowsA x rowsB outputs: element (a, b) is the dot product of row a of the lanes' operand and
// row b of the columns' operand. SWAP false: C[a * ldc + b]; true: C[b * ldc + a].
template <int BN, bool SWAP>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               void* __restrict__ C, int c_dtype, long long ldc, int rowsA, int rowsB, int K,
               int kb_per_split, int mode, float* __restrict__ partial, long long partial_stride,
               long long partial_ld, int* __restrict__ error) {
  using Cfg = TcCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  const uint32_t sA = base;
  const uint32_t sB = base + Cfg::STAGES * Cfg::A_BYTES;
  const uint32_t bars = sB + Cfg::STAGES * Cfg::B_BYTES;
  const uint32_t full0 = bars, empty0 = bars + 8 * Cfg::STAGES, accum = bars + 16 * Cfg::STAGES;
  const uint32_t slot = accum + 8;
  volatile uint32_t* slot_ptr = (volatile uint32_t*)(smem_raw + (slot - raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * TC_BM, n0 = blockIdx.y * BN;
  const int nkb_total = (K + TC_BK - 1) / TC_BK;
  const int kb0 = blockIdx.z * kb_per_split;
  const int nkb = min(kb_per_split, nkb_total - kb0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(accum, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) tmem_alloc(slot, Cfg::COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *slot_ptr;

  if (warp == 0) {
    if (elect_one()) {
      for (int i = 0; i < nkb; ++i) {
        const int s = i % Cfg::STAGES;
        const uint32_t ph = (i / Cfg::STAGES) & 1;
        mbar_wait(empty0 + 8 * s, ph ^ 1, error, 1);
        mbar_expect_tx(full0 + 8 * s, Cfg::A_BYTES + Cfg::B_BYTES);
        tma_load_2d(sA + s * Cfg::A_BYTES, &tmA, (kb0 + i) * TC_BK, m0, full0 + 8 * s);
        tma_load_2d(sB + s * Cfg::B_BYTES, &tmB, (kb0 + i) * TC_BK, n0, full0 + 8 * s);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, BN);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % Cfg::STAGES;
        const uint32_t ph = (i / Cfg::STAGES) & 1;
        mbar_wait(full0 + 8 * s, ph, error, 2);
        tc_fence_after_sync();
        const uint64_t da = umma_desc_k128(sA + s * Cfg::A_BYTES);
        const uint64_t db = umma_desc_k128(sB + s * Cfg::B_BYTES);
#pragma unroll
        for (int k = 0; k < TC_BK / 16; ++k)  // 16 values of K = 32 bytes further in the row
          umma_bf16(tmem, da + 2 * k, db + 2 * k, idesc, (i | k) != 0);
        umma_commit(empty0 + 8 * s);  // the stage is free once these MMAs have read it
      }
      umma_commit(accum);
    }
  } else {
    mbar_wait(accum, 0, error, 3);
    tc_fence_after_sync();
    const int q = warp & 3;  // the TMEM lanes a warp may read: 32 * (warp % 4) ..
    const int a = m0 + q * 32 + lane;
    const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16);
    float* part = partial ? partial + blockIdx.z * partial_stride : nullptr;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 16) {
      if (n0 + c0 >= rowsB) break;  // uniform over the warp
      float v[16];
      tmem_ld16(taddr + c0, v);
      if (a >= rowsA) continue;
      if (!SWAP) {
        const int b0 = n0 + c0;
        const bool whole = b0 + 16 <= rowsB;
        if (mode == TC_PARTIAL) {
          float* p = part + (size_t)a * partial_ld + b0;
          if (whole && (partial_ld & 3) == 0 && (partial_stride & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 16; j += 4)
              *(float4*)(p + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
            for (int j = 0; j < 16 && b0 + j < rowsB; ++j) p[j] = v[j];
          }
        } else if (c_dtype == MB_BF16 && whole && (ldc & 7) == 0 && ((uintptr_t)C & 15) == 0) {
          __nv_bfloat162 h[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
          uint4* p = (uint4*)((__nv_bfloat16*)C + (size_t)a * ldc + b0);
          p[0] = *(uint4*)&h[0];
          p[1] = *(uint4*)&h[4];
        } else if (c_dtype == MB_F32 && whole && (ldc & 3) == 0 && ((uintptr_t)C & 15) == 0) {
          float4* p = (float4*)((float*)C + (size_t)a * ldc + b0);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float4 o = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            if (mode == TC_ADD) {
              const float4 r = p[j];
              o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
            }
            p[j] = o;
          }
        } else {
          for (int j = 0; j < 16 && b0 + j < rowsB; ++j)
            store_out(C, c_dtype, (size_t)a * ldc + b0 + j, v[j], mode);
        }
      } else {
        for (int j = 0; j < 16; ++j) {
          const int b = n0 + c0 + j;
          if (b >= rowsB) break;
          if (mode == TC_PARTIAL) part[(size_t)b * partial_ld + a] = v[j];
          else store_out(C, c_dtype, (size_t)b * ldc + a, v[j], mode);
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, Cfg::COLS);
}

// C[M, N] = (or +=) the sum over the splits, added in split order
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits,
                                     long long stride, void* __restrict__ C, int c_dtype,
                                     long long ldc, int M, int N, int mode) {
  const size_t total = (size_t)M * N;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    float v = partial[i];
    for (int s = 1; s < splits; ++s) v += partial[s * stride + i];
    const size_t r = i / N, c = i - r * N;
    store_out(C, c_dtype, r * ldc + c, v, mode);
  }
}

template <int BN, bool SWAP>
static int launch_tc(const CUtensorMap& tmA, const CUtensorMap& tmB, void* C, int c_dtype,
                     long long ldc, int rowsA, int rowsB, int K, int splits, int kb_per_split,
                     int mode, float* partial, long long pstride, long long pld, int* error,
                     cudaStream_t s) {
  using Cfg = TcCfg<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, SWAP>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) MB_FAIL("mb_gemm_tc: shared memory of %d bytes: %s", Cfg::SMEM,
                                  cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid((rowsA + TC_BM - 1) / TC_BM, (rowsB + BN - 1) / BN, splits);
  gemm_tc_kernel<BN, SWAP><<<grid, TC_THREADS, Cfg::SMEM, s>>>(
      tmA, tmB, C, c_dtype, ldc, rowsA, rowsB, K, kb_per_split, mode, partial, pstride, pld, error);
  MB_CHECK_LAUNCH("mb_gemm_tc");
}

// 1 if the sizes can go through mb_gemm_tc, else 0 with the reason in mb_last_error().
MB_EXPORT int mb_gemm_tc_supported(const void* A, int lda, const void* W, int M, int N, int K) {
  if (K % 8 || lda % 8) { snprintf(g_mb_error, sizeof(g_mb_error), "K = %d (lda %d) is no multiple of 8", K, lda); return 0; }
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) { snprintf(g_mb_error, sizeof(g_mb_error), "operands are not 16-byte aligned"); return 0; }
  if (K < 8 || M <= 0 || N <= 0) return 0;
  return 1;
}

// C[M, N] (row stride ldc; bfloat16 or float32) = A[M, K] (row stride lda) · W[N, K]ᵀ, or
// C += ... (epilogue 1, float32 C). `workspace` (float32, may be null) lets the K range be
// split; `error` is a device word that receives a non-zero code if a wait in the kernel ran
// out (1 load, 2 MMA, 3 epilogue). `sms`: the number of SMs of the device.
MB_EXPORT int mb_gemm_tc(const void* A, int lda, const void* W, void* C, int c_dtype, int ldc,
                         int M, int N, int K, int epilogue, float* workspace,
                         long long workspace_floats, int* error, int sms, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!mb_gemm_tc_supported(A, lda, W, M, N, K)) return -1;
  if (epilogue != TC_STORE && epilogue != TC_ADD) MB_FAIL("mb_gemm_tc: epilogue %d", epilogue);
  if (epilogue == TC_ADD && c_dtype != MB_F32) MB_FAIL("mb_gemm_tc: the residual is float32");
  cudaStream_t s = (cudaStream_t)stream;
  const bool swap = M <= 64;
  int bn;
  if (swap) bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  else bn = N >= 256 ? 256 : (N > 64 ? 128 : 64);
  const int rowsA = swap ? N : M, rowsB = swap ? M : N;
  CUtensorMap tmA, tmB;
  if (swap) {
    if (!mb_make_map_bf16(&tmA, W, N, K, K, TC_BM, "mb_gemm_tc weight")) return -1;
    if (!mb_make_map_bf16(&tmB, A, M, K, lda, bn, "mb_gemm_tc input")) return -1;
  } else {
    if (!mb_make_map_bf16(&tmA, A, M, K, lda, TC_BM, "mb_gemm_tc input")) return -1;
    if (!mb_make_map_bf16(&tmB, W, N, K, K, bn, "mb_gemm_tc weight")) return -1;
  }
  const int tiles = ((rowsA + TC_BM - 1) / TC_BM) * ((rowsB + bn - 1) / bn);
  const int nkb = (K + TC_BK - 1) / TC_BK;
  int splits = 1;
  if (workspace && tiles < sms && nkb >= 8) {
    int want = (2 * sms + tiles - 1) / tiles;
    if (want > nkb / 4) want = nkb / 4;
    const long long per = (long long)M * N;
    if (want > workspace_floats / per) want = (int)(workspace_floats / per);
    if (want > 1) splits = want;
  }
  int per_split = (nkb + splits - 1) / splits;
  splits = (nkb + per_split - 1) / per_split;
  const int mode = splits > 1 ? TC_PARTIAL : epilogue;
  float* partial = splits > 1 ? workspace : nullptr;
  const long long pstride = (long long)M * N, pld = N;
  int rc;
#define GO(BN_, SW_)                                                                          \
  rc = launch_tc<BN_, SW_>(tmA, tmB, C, c_dtype, ldc, rowsA, rowsB, K, splits, per_split, mode, \
                           partial, pstride, pld, error, s)
  if (swap) {
    if (bn == 16) GO(16, true); else if (bn == 32) GO(32, true); else GO(64, true);
  } else {
    if (bn == 256) GO(256, false); else if (bn == 128) GO(128, false); else GO(64, false);
  }
#undef GO
  if (rc) return rc;
  g_last_launches = splits > 1 ? 2 : 1;
  if (splits > 1) {
    const size_t total = (size_t)M * N;
    const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    splitk_reduce_kernel<<<blocks, 256, 0, s>>>(workspace, splits, pstride, C, c_dtype, ldc, M, N,
                                                epilogue);
    MB_CHECK_LAUNCH("mb_gemm_tc reduce");
  }
  return 0;
}
