// y = x · Wᵀ for bfloat16 x [M, K] and W [N, K] on the fifth-generation tensor cores:
// operand tiles brought to shared memory by TMA (128-byte swizzle), tcgen05.mma issued by one
// thread with the float32 accumulator in tensor memory, tcgen05.ld for the epilogue.
//
// The operand on the MMA's M side fills the TMEM lanes of a tile, the other one its columns
// (16 to 256). Three forms:
//   many tokens (prefill):   tokens on the lanes of a PAIR of CTAs (256 of them), output
//                            features on the columns: gemm_tc_pair_kernel, further down;
//   65 to 128 tokens:        tokens on the 128 lanes of one CTA, features on the columns;
//   few tokens (decode):     the WEIGHT rows on the lanes and the tokens on the columns, so that
//                            a step streams each weight byte once through full-width MMAs,
//                            whatever the batch; the tile is written back transposed.
// In the decode form two CTAs share an SM; a weight with few 128-row tiles has its K range
// split over as many CTAs as fill those places, one with a few more gets tiles of fewer rows so
// that one round of CTAs covers it evenly. In the other forms K is split when there are fewer
// tiles than places. Partial sums go to a float32 workspace that the caller provides and are
// added up in split order by a second kernel (deterministic, no atomics) or by the caller's
// next kernel.
//
// Epilogues: store (bfloat16 or float32), add into the float32 residual, and SwiGLU for a
// weight whose rows alternate gate, up, gate, up ...: out[:, i] = silu(y[:, 2i]) * y[:, 2i+1].
//
// Warp roles in a CTA of 192 threads: warp 0 loads (one elected lane), warp 1 allocates TMEM
// and issues the MMAs (one elected lane), warps 2-5 read the accumulator and store.
//
// This replaces the reference's `gemm8` / `linear8` (tools/cuda/linear.cu:418-606 of the
// reference project), which multiply in float32 on the CUDA cores.
#include "tc_common.cuh"

MB_DEFINE_LAST_ERROR

static thread_local int g_last_launches = 0;
static thread_local int g_last_splits = 1;
// splits of K in the last mb_gemm_tc of this thread; with `defer` and more than one split the
// partial sums [splits][M][N] were left in the workspace for the caller's next kernel to add
MB_EXPORT int mb_gemm_tc_last_splits() { return g_last_splits; }
// kernels that the last mb_gemm_tc of this thread launched (2 when K was split)
MB_EXPORT int mb_gemm_tc_last_launches() { return g_last_launches; }

enum { TC_STORE = 0, TC_ADD = 1, TC_PARTIAL = 2, TC_SWIGLU = 3 };

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_A_TILE (TC_BM * TC_BK * 2)  // what an MMA reads from a stage's first operand
#define TC_MAX_STAGES 32
#define TC_MAX_SPLITS 8
#define TC_SMEM_MAX (227 * 1024)

template <int BN> struct TcCfg {
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int COLS = BN < 16 ? 16 : BN;  // TMEM columns of one accumulator (two are allocated)
};

__device__ __forceinline__ void store_out(void* C, int c_dtype, size_t idx, float v, int mode) {
  if (c_dtype == MB_F32) {
    float* p = (float*)C + idx;
    *p = mode == TC_ADD ? *p + v : v;
  } else {
    ((__nv_bfloat16*)C)[idx] = __float2bfloat16_rn(v);
  }
}

// silu(g) * u for an output that is rounded to bfloat16: the fast exponential and division
// are exact to a few units of the float32 result's last place
__device__ __forceinline__ float silu_mul(float g, float u) {
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}

// Sixteen neighbouring columns b0 .. b0 + 15 of accumulator row `a` in the prefill form
// (tokens on the lanes): store, add into the residual, leave as a partial sum, or SwiGLU.
__device__ __forceinline__ void store_row16(const float* v, void* C, int c_dtype, long long ldc,
                                            int a, int b0, int rowsB, int mode, float* part,
                                            long long partial_ld, long long partial_stride) {
  const bool whole = b0 + 16 <= rowsB;
  if (mode == TC_SWIGLU) {
    // columns 2i and 2i+1 are gate and up of output feature (b0 + 2i) / 2
    __nv_bfloat16* p = (__nv_bfloat16*)C + (size_t)a * ldc + (b0 >> 1);
    if (whole && (ldc & 7) == 0 && ((uintptr_t)C & 15) == 0) {
      __nv_bfloat162 h[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        h[j] = __floats2bfloat162_rn(silu_mul(v[4 * j], v[4 * j + 1]),
                                     silu_mul(v[4 * j + 2], v[4 * j + 3]));
      *(uint4*)p = *(uint4*)&h[0];
    } else {
      for (int j = 0; j < 16 && b0 + j + 1 < rowsB; j += 2)
        p[j >> 1] = __float2bfloat16_rn(silu_mul(v[j], v[j + 1]));
    }
  } else if (mode == TC_PARTIAL) {
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
}

// The epilogue of the forms with tokens on the lanes, for outputs made of whole 16-byte
// pieces. A thread holds one accumulator row; written from there, a warp's store would touch
// 32 rows with 32 bytes each. Instead the warp lays 32 rows x 128 bytes of finished output
// into its own shared memory (`stage_w`, 4 KB; 16-byte pieces, piece p of row r at
// p ^ (r & 7): no bank conflicts either way) and writes it out four whole rows of 128 bytes
// at a time. `row0`: the warp's first row of the output; `width`: the tile's columns.
__device__ __forceinline__ void staged_rows(uint32_t taddr, uint32_t stage_w, int lane, int row0,
                                            int n0, int width, int M, int N, void* C, int c_dtype,
                                            long long ldc, int mode, float* part,
                                            long long partial_ld) {
  const int acc_cols = mode == TC_SWIGLU ? 128 : (c_dtype == MB_BF16 && mode == TC_STORE ? 64 : 32);
  const uint32_t mine = stage_w + lane * 128;
#pragma unroll 1
  for (int c0 = 0; c0 < width; c0 += acc_cols) {
    if (n0 + c0 >= N) break;
    const int ncols = min(acc_cols, min(width - c0, N - (n0 + c0)));
#pragma unroll 1
    for (int g = 0; g * 16 < ncols; ++g) {
      float v[16];
      tmem_ld16(taddr + c0 + 16 * g, v);
      if (mode == TC_SWIGLU) {
        __nv_bfloat162 h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          h[j] = __floats2bfloat162_rn(silu_mul(v[4 * j], v[4 * j + 1]),
                                       silu_mul(v[4 * j + 2], v[4 * j + 3]));
        st_shared_v4(mine + ((g ^ (lane & 7)) << 4), *(uint4*)&h[0]);
      } else if (acc_cols == 64) {
        __nv_bfloat162 h[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        st_shared_v4(mine + (((2 * g) ^ (lane & 7)) << 4), *(uint4*)&h[0]);
        st_shared_v4(mine + (((2 * g + 1) ^ (lane & 7)) << 4), *(uint4*)&h[4]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          st_shared_v4(mine + (((4 * g + j) ^ (lane & 7)) << 4),
                       make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]),
                                  __float_as_uint(v[4 * j + 2]), __float_as_uint(v[4 * j + 3])));
      }
    }
    __syncwarp();
    const int pc = lane & 7;
    // bytes of output per accumulator column: 1 (SwiGLU), 2 (bfloat16), 4 (float32)
    const int pieces = mode == TC_SWIGLU ? ncols >> 4 : (acc_cols == 64 ? ncols >> 3 : ncols >> 2);
    if (acc_cols == 32) {
      float* dst = mode == TC_PARTIAL ? part : (float*)C;
      const long long ld = mode == TC_PARTIAL ? partial_ld : ldc;
      float4 old[8];
      if (mode == TC_ADD) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = 4 * i + (lane >> 3);
          if (pc < pieces && row0 + r < M)
            old[i] = *(const float4*)(dst + (size_t)(row0 + r) * ld + n0 + c0 + 4 * pc);
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = 4 * i + (lane >> 3);
        if (pc < pieces && row0 + r < M) {
          const uint4 u = ld_shared_v4(stage_w + r * 128 + ((pc ^ (r & 7)) << 4));
          float4 o = make_float4(__uint_as_float(u.x), __uint_as_float(u.y),
                                 __uint_as_float(u.z), __uint_as_float(u.w));
          if (mode == TC_ADD) { o.x += old[i].x; o.y += old[i].y; o.z += old[i].z; o.w += old[i].w; }
          *(float4*)(dst + (size_t)(row0 + r) * ld + n0 + c0 + 4 * pc) = o;
        }
      }
    } else {
      const int col = (mode == TC_SWIGLU ? (n0 + c0) >> 1 : n0 + c0) + 8 * pc;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = 4 * i + (lane >> 3);
        if (pc < pieces && row0 + r < M)
          *(uint4*)((__nv_bfloat16*)C + (size_t)(row0 + r) * ldc + col) =
              ld_shared_v4(stage_w + r * 128 + ((pc ^ (r & 7)) << 4));
      }
    }
    __syncwarp();  // the rows are read out before the next columns are laid over them
  }
}

// rowsA x rowsB outputs: element (a, b) is the dot product of row a of the lanes' operand and
// row b of the columns' operand. SWAP false: C[a * ldc + b]; true: C[b * ldc + a].
// A CTA owns `tile_rows` (<= 128) rows of the lanes' operand; its stages hold a_stage bytes of
// it each (tile_rows rows, rounded up to 8) and BN rows of the other operand.
template <int BN, bool SWAP>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               void* __restrict__ C, int c_dtype, long long ldc, int rowsA, int rowsB, int K,
               int kb_per_split, int mode, float* __restrict__ partial, long long partial_stride,
               long long partial_ld, int tile_rows, int stages, int a_stage, int tiles_a,
               int tiles_b, int num_tiles, int* __restrict__ error) {
  using Cfg = TcCfg<BN>;
  MB_TRACE_BEGIN();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  const uint32_t sA = base;
  // an MMA reads a full 128-row tile from a stage's start: the last stage must have that much
  // shared memory behind it (rows beyond tile_rows feed TMEM lanes that nobody reads)
  const uint32_t a_region = max(stages * a_stage, (stages - 1) * a_stage + TC_A_TILE);
  const uint32_t sB = base + a_region;
  const uint32_t bars = sB + stages * Cfg::B_BYTES;
  const uint32_t full0 = bars, empty0 = bars + 8 * stages;
  const uint32_t acc_full0 = bars + 16 * stages, acc_empty0 = acc_full0 + 16;
  const uint32_t slot = acc_empty0 + 16;
  volatile uint32_t* slot_ptr = (volatile uint32_t*)(smem_raw + (slot - raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb_total = (K + TC_BK - 1) / TC_BK;
  const int tiles_ab = tiles_a * tiles_b;
  // tokens on the lanes: the epilogue warps' staging rows lie behind the barriers (the host
  // adds their 16 KB); whole 16-byte pieces of output need a width, a row stride and a base
  // that are multiples of 16 bytes
  const uint32_t stage_w = bars + 1024 + (warp & 3) * 4096;
  const int out_cols = mode == TC_SWIGLU ? rowsB >> 1 : rowsB;
  const int per16 = (mode == TC_SWIGLU || (mode == TC_STORE && c_dtype == MB_BF16)) ? 8 : 4;
  const bool staged = !SWAP && out_cols % per16 == 0 &&
                      (mode == TC_PARTIAL ? (partial_ld % 4 == 0 && partial_stride % 4 == 0 &&
                                             ((uintptr_t)partial & 15) == 0)
                                          : (ldc % per16 == 0 && ((uintptr_t)C & 15) == 0));
  const uint32_t stage_bytes = (uint32_t)tile_rows * (TC_BK * 2) + Cfg::B_BYTES;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 4);  // the four epilogue warps
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) tmem_alloc(slot, 2 * Cfg::COLS);  // two accumulators
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *slot_ptr;
  // Everything above touched only this CTA's shared and tensor memory. What follows may run
  // while the kernel before in the stream is still at work (programmatic dependent launch):
  // each role waits for that kernel (mb_grid_wait) before it touches memory that depends on it.
  // In the decode form the lanes' operand is the WEIGHT, which depends on nothing: the load
  // warp fills the first round of stages with weight tiles before it waits, so the small
  // kernels between two products run under the stream of the next product's weights.
  if (warp == 0) {
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      int early = 0;
      if (SWAP && (int)blockIdx.x < num_tiles) {
        const int w = blockIdx.x, rem = w % tiles_ab;
        const int m0 = (rem % tiles_a) * tile_rows;
        const int kb0 = (w / tiles_ab) * kb_per_split;
        early = min(stages, min(kb_per_split, nkb_total - kb0));
        for (int i = 0; i < early; ++i) {
          mbar_expect_tx(full0 + 8 * i, stage_bytes);
          tma_load_2d(sA + i * a_stage, &tmA, (kb0 + i) * TC_BK, m0, full0 + 8 * i);
        }
      }
      mb_grid_wait();
      mb_grid_launch_next();
      for (int w = blockIdx.x; w < num_tiles; w += gridDim.x) {
        const int rem = w % tiles_ab;
        const int m0 = (rem % tiles_a) * tile_rows, n0 = (rem / tiles_a) * BN;
        const int kb0 = (w / tiles_ab) * kb_per_split;
        const int nkb = min(kb_per_split, nkb_total - kb0);
        for (int i = 0; i < nkb; ++i) {
          if (early > 0) {
            --early;  // this stage's barrier is armed and its weight tile is on the way
          } else {
            mbar_wait(empty0 + 8 * s, ph ^ 1, error, 1);
            mbar_expect_tx(full0 + 8 * s, stage_bytes);
            tma_load_2d(sA + s * a_stage, &tmA, (kb0 + i) * TC_BK, m0, full0 + 8 * s);
          }
          tma_load_2d(sB + s * Cfg::B_BYTES, &tmB, (kb0 + i) * TC_BK, n0, full0 + 8 * s);
          if (++s == stages) { s = 0; ph ^= 1; }
        }
      }
    } else {
      mb_grid_wait();
    }
  } else if (warp == 1) {
    mb_grid_wait();
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, BN);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      for (int w = blockIdx.x; w < num_tiles; w += gridDim.x, ++it) {
        const int kb0 = (w / tiles_ab) * kb_per_split;
        const int nkb = min(kb_per_split, nkb_total - kb0);
        const int b = it & 1;
        mbar_wait(acc_empty0 + 8 * b, ((it >> 1) & 1) ^ 1, error, 6);  // the epilogue left it
        tc_fence_after_sync();
        const uint32_t acc = tmem + b * Cfg::COLS;
        for (int i = 0; i < nkb; ++i) {
          mbar_wait(full0 + 8 * s, ph, error, 2);
          tc_fence_after_sync();
          const uint64_t da = umma_desc_k128(sA + s * a_stage);
          const uint64_t db = umma_desc_k128(sB + s * Cfg::B_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)  // 16 values of K = 32 bytes further in the row
            umma_bf16(acc, da + 2 * k, db + 2 * k, idesc, (i | k) != 0);
          umma_commit(empty0 + 8 * s);  // the stage is free once these MMAs have read it
          if (++s == stages) { s = 0; ph ^= 1; }
        }
        umma_commit(acc_full0 + 8 * b);
      }
    }
  } else {
    mb_grid_wait();
    const int q = warp & 3;  // the TMEM lanes a warp may read: 32 * (warp % 4) ..
    const int lane_row = q * 32 + lane;
    int it = 0;
    for (int w = blockIdx.x; w < num_tiles; w += gridDim.x, ++it) {
      const int rem = w % tiles_ab, z = w / tiles_ab;
      const int m0 = (rem % tiles_a) * tile_rows, n0 = (rem / tiles_a) * BN;
      const int b = it & 1;
      mbar_wait(acc_full0 + 8 * b, (it >> 1) & 1, error, 3);
      tc_fence_after_sync();
      const int a = m0 + lane_row;
      const bool mine = lane_row < tile_rows && a < rowsA;
      const uint32_t taddr = tmem + b * Cfg::COLS + ((uint32_t)(q * 32) << 16);
      float* part = partial ? partial + z * partial_stride : nullptr;
      if (staged) {
        staged_rows(taddr, stage_w, lane, a - lane, n0, BN, rowsA, rowsB, C, c_dtype, ldc, mode,
                    part, partial_ld);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty0 + 8 * b);
        continue;
      }
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (n0 + c0 >= rowsB) break;  // uniform over the warp
        float v[16];
        tmem_ld16(taddr + c0, v);
        if (SWAP && mode == TC_SWIGLU) {
          // lanes 2i and 2i+1 hold gate and up of output feature (m0 + lane_row) / 2
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float up = __shfl_xor_sync(0xffffffffu, v[j], 1);
            const int bb = n0 + c0 + j;
            if (mine && !(lane & 1) && bb < rowsB)
              ((__nv_bfloat16*)C)[(size_t)bb * ldc + (a >> 1)] =
                  __float2bfloat16_rn(silu_mul(v[j], up));
          }
          continue;
        }
        if (!mine) continue;
        if (!SWAP) {
          store_row16(v, C, c_dtype, ldc, a, n0 + c0, rowsB, mode, part, partial_ld,
                      partial_stride);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int bb = n0 + c0 + j;
            if (bb >= rowsB) continue;
            if (mode == TC_PARTIAL) part[(size_t)bb * partial_ld + a] = v[j];
            else store_out(C, c_dtype, (size_t)bb * ldc + a, v[j], mode);
          }
        }
      }
      // this warp has read its lanes of the accumulator: the MMA warp may overwrite it
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty0 + 8 * b);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 2 * Cfg::COLS);
  MB_TRACE_END(1);
}

// ---------------------------------------------------------------------------- CTA pairs
// The prefill form for many tokens: two CTAs of a cluster share one tile of 256 tokens x BN
// output features (up to 256). Each loads its 128 token rows and its half of the weight rows
// (half the shared-memory traffic of two separate 128 x 256 tiles, so six stages of 32 KB fit
// instead of four of 48 KB), rank 0 issues tcgen05.mma.cta_group::2 for both, and each CTA's epilogue
// warps read the 128 accumulator lanes that landed in its own tensor memory.
//   full[s]      in rank 0: both CTAs' TMA loads complete their bytes there
//   empty[s]     in both:   a multicast commit of rank 0's MMA thread frees the stage in both
//   acc_full[b]  in both:   multicast commit after a tile's last MMA
//   acc_empty[b] in rank 0: the eight epilogue warps of the pair arrive (rank 1's from afar)
// The tile's width BN (a multiple of 16 up to 256) is chosen so that the last round of tiles
// leaves few pairs idle.
#define TC2_A_HALF (128 * TC_BK * 2)  // one CTA's 128 token rows of a stage
#define TC2_COLS 256                  // tensor-memory columns of one accumulator
#define TC2_STAGING (4 * 4096)        // 32 rows x 128 bytes of output for each epilogue warp
template <int BN> struct Tc2Cfg {
  static constexpr int B_HALF = (BN / 2) * TC_BK * 2;  // one CTA's half of the weight rows
  static constexpr int STAGE = TC2_A_HALF + B_HALF;
  static constexpr int STAGES = (200 * 1024) / STAGE > 8 ? 8 : (200 * 1024) / STAGE;
  static constexpr int SMEM = 1024 + STAGES * STAGE + 1024 + TC2_STAGING;
};

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    void* __restrict__ C, int c_dtype, long long ldc, int M, int N, int K,
                    int kb_per_split, int mode, float* __restrict__ partial,
                    long long partial_stride, long long partial_ld, int tiles_m, int tiles_n,
                    int num_tiles, int* __restrict__ error) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  using Cfg = Tc2Cfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  const uint32_t sA = base, sB = base + STAGES * TC2_A_HALF;
  const uint32_t bars = sB + STAGES * Cfg::B_HALF;
  const uint32_t full0 = bars, empty0 = bars + 8 * STAGES;
  const uint32_t acc_full0 = bars + 16 * STAGES, acc_empty0 = acc_full0 + 16;
  const uint32_t slot = acc_empty0 + 16;
  volatile uint32_t* slot_ptr = (volatile uint32_t*)(smem_raw + (slot - raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int nkb_total = (K + TC_BK - 1) / TC_BK;
  const int tiles_mn = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 8);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) tmem_alloc_pair(slot, 2 * TC2_COLS);
  tc_fence_before_sync();
  cluster_sync_all();  // both CTAs' barriers and tensor memory exist before either is used
  tc_fence_after_sync();
  const uint32_t tmem = *slot_ptr;
  // the epilogue warps' staging rows lie behind the barriers; whole 16-byte pieces of output
  // need a width, a row stride and a base that are multiples of 16 bytes
  const uint32_t stage_w = bars + 1024 + (warp & 3) * 4096;
  const int out_cols = mode == TC_SWIGLU ? N >> 1 : N;
  const int per16 = (mode == TC_SWIGLU || (mode == TC_STORE && c_dtype == MB_BF16)) ? 8 : 4;
  const bool staged = out_cols % per16 == 0 &&
                      (mode == TC_PARTIAL ? (partial_ld % 4 == 0 && partial_stride % 4 == 0 &&
                                             ((uintptr_t)partial & 15) == 0)
                                          : (ldc % per16 == 0 && ((uintptr_t)C & 15) == 0));

  mb_grid_wait();
  mb_grid_launch_next();
  if (warp == 0) {
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      for (int w = pair; w < num_tiles; w += pairs) {
        const int rem = w % tiles_mn;
        const int m0 = (rem % tiles_m) * 256 + (int)rank * 128;
        const int n0 = (rem / tiles_m) * BN + (int)rank * (BN / 2);
        const int kb0 = (w / tiles_mn) * kb_per_split;
        const int nkb = min(kb_per_split, nkb_total - kb0);
        for (int i = 0; i < nkb; ++i) {
          mbar_wait(empty0 + 8 * s, ph ^ 1, error, 11);
          if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * Cfg::STAGE);
          const uint32_t full_lead = cluster_addr_of(full0 + 8 * s, 0);
          tma_load_2d_pair(sA + s * TC2_A_HALF, &tmA, (kb0 + i) * TC_BK, m0, full_lead);
          tma_load_2d_pair(sB + s * Cfg::B_HALF, &tmB, (kb0 + i) * TC_BK, n0, full_lead);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(256, BN);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      for (int w = pair; w < num_tiles; w += pairs, ++it) {
        const int kb0 = (w / tiles_mn) * kb_per_split;
        const int nkb = min(kb_per_split, nkb_total - kb0);
        const int b = it & 1;
        mbar_wait(acc_empty0 + 8 * b, ((it >> 1) & 1) ^ 1, error, 16);
        tc_fence_after_sync();
        const uint32_t acc = tmem + b * TC2_COLS;
        for (int i = 0; i < nkb; ++i) {
          mbar_wait(full0 + 8 * s, ph, error, 12);
          tc_fence_after_sync();
          const uint64_t da = umma_desc_k128(sA + s * TC2_A_HALF);
          const uint64_t db = umma_desc_k128(sB + s * Cfg::B_HALF);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)
            umma_bf16_pair(acc, da + 2 * k, db + 2 * k, idesc, (i | k) != 0);
          umma_commit_pair(empty0 + 8 * s, 3);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        umma_commit_pair(acc_full0 + 8 * b, 3);
      }
    }
  } else {
    const int q = warp & 3;
    const int lane_row = q * 32 + lane;
    int it = 0;
    for (int w = pair; w < num_tiles; w += pairs, ++it) {
      const int rem = w % tiles_mn, z = w / tiles_mn;
      const int n0 = (rem / tiles_m) * BN;
      const int a = (rem % tiles_m) * 256 + (int)rank * 128 + lane_row;
      const int b = it & 1;
      mbar_wait(acc_full0 + 8 * b, (it >> 1) & 1, error, 13);
      tc_fence_after_sync();
      const uint32_t taddr = tmem + b * TC2_COLS + ((uint32_t)(q * 32) << 16);
      float* part = partial ? partial + z * partial_stride : nullptr;
      if (staged) {
        staged_rows(taddr, stage_w, lane, a - lane, n0, BN, M, N, C, c_dtype, ldc, mode, part,
                    partial_ld);
      } else {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (n0 + c0 >= N) break;
        float v[16];
        tmem_ld16(taddr + c0, v);
        if (a < M)
          store_row16(v, C, c_dtype, ldc, a, n0 + c0, N, mode, part, partial_ld, partial_stride);
      }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(acc_empty0 + 8 * b);
        else mbar_arrive_cluster(cluster_addr_of(acc_empty0 + 8 * b, 0));
      }
    }
  }
  // Neither CTA leaves while the other may still read its shared memory or signal its barriers.
  tc_fence_before_sync();
  cluster_sync_all();
  if (warp == 1) tmem_dealloc_pair(tmem, 2 * TC2_COLS);
}

// How many CTA pairs the device runs at once (0: the pair kernel cannot run here).
static int pair_capacity(int sms) {
  static int pairs = -1;
  if (pairs >= 0) return pairs;
  pairs = 0;
  if (cudaFuncSetAttribute(gemm_tc_pair_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           Tc2Cfg<256>::SMEM) != cudaSuccess) {
    cudaGetLastError();
    return pairs;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * sms);
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = Tc2Cfg<256>::SMEM;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<256>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return pairs;
  }
  pairs = n > sms / 2 ? sms / 2 : n;
  return pairs;
}
MB_EXPORT int mb_gemm_tc_pairs(int sms) { return pair_capacity(sms); }

template <typename... KArgs, typename... Args>
static cudaError_t mb_launch_pair(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <int BN>
static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, void* C, int c_dtype,
                       long long ldc, int M, int N, int K, int kb_per_split, int mode,
                       float* partial, int tiles_m, int tiles_n, int splits, int pairs,
                       int* error, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Tc2Cfg<BN>::SMEM);
    if (e != cudaSuccess) MB_FAIL("mb_gemm_tc (pairs): shared memory of %d bytes: %s",
                                  Tc2Cfg<BN>::SMEM, cudaGetErrorString(e));
    configured = true;
  }
  const int num_tiles = tiles_m * tiles_n * splits;
  const int grid = 2 * (num_tiles < pairs ? num_tiles : pairs);
  mb_launch_pair(gemm_tc_pair_kernel<BN>, dim3(grid), dim3(TC_THREADS), Tc2Cfg<BN>::SMEM, s, tmA,
                 tmB, C, c_dtype, ldc, M, N, K, kb_per_split, mode, partial, (long long)M * N,
                 (long long)N, tiles_m, tiles_n, num_tiles, error);
  cudaError_t le = cudaGetLastError();
  if (le != cudaSuccess) MB_FAIL("mb_gemm_tc (pairs): %s", cudaGetErrorString(le));
  return 0;
}

// The tile width for N output features and tiles_m row tiles on `pairs` CTA pairs: the one
// whose rounds of tiles take the least time (measured: a full round of tiles of width w takes
// about w + 40 in units of 0.09 microseconds at K = 4096).
static int pair_tile_width(int N, int tiles_m, int pairs) {
  int best = 256;
  long long best_cost = -1;
  for (int w = 256; w >= 128; w -= 16) {
    const long long tiles = (long long)tiles_m * ((N + w - 1) / w);
    const long long rounds = (tiles + pairs - 1) / pairs;
    const long long cost = rounds * (w + 40);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = w; }
  }
  return best;
}

// C[M, N] = (or +=) the sum over the splits, added in split order
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits,
                                     long long stride, void* __restrict__ C, int c_dtype,
                                     long long ldc, int M, int N, int mode) {
  mb_grid_wait();
  mb_grid_launch_next();
  const size_t total = (size_t)M * N;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    float v = partial[i];
    for (int s = 1; s < splits; ++s) v += partial[s * stride + i];
    const size_t r = i / N, c = i - r * N;
    store_out(C, c_dtype, r * ldc + c, v, mode);
  }
}

struct TcPlan {
  int tile_rows, stages, a_stage, smem, splits, kb_per_split, max_ctas;
};

template <int BN, bool SWAP>
static int launch_tc(const CUtensorMap& tmA, const CUtensorMap& tmB, void* C, int c_dtype,
                     long long ldc, int rowsA, int rowsB, int K, const TcPlan& p, int mode,
                     float* partial, long long pstride, long long pld, int* error,
                     cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, SWAP>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_MAX);
    if (e != cudaSuccess) MB_FAIL("mb_gemm_tc: shared memory of %d bytes: %s", TC_SMEM_MAX,
                                  cudaGetErrorString(e));
    configured = true;
  }
  const int tiles_a = (rowsA + p.tile_rows - 1) / p.tile_rows, tiles_b = (rowsB + BN - 1) / BN;
  const int num_tiles = tiles_a * tiles_b * p.splits;
  const int grid = num_tiles < p.max_ctas ? num_tiles : p.max_ctas;
  mb_launch(gemm_tc_kernel<BN, SWAP>, dim3(grid), dim3(TC_THREADS), p.smem, s,
      tmA, tmB, C, c_dtype, ldc, rowsA, rowsB, K, p.kb_per_split, mode, partial, pstride, pld,
      p.tile_rows, p.stages, p.a_stage, tiles_a, tiles_b, num_tiles, error);
  MB_CHECK_LAUNCH("mb_gemm_tc");
}

// Stages and shared memory for tiles of tile_rows x BN within `budget` bytes.
static void plan_stages(TcPlan& p, int bn, int budget) {
  p.a_stage = ((p.tile_rows + 7) / 8) * 8 * TC_BK * 2;
  const int b_bytes = bn * TC_BK * 2;
  const int fixed = 1024 /*alignment*/ + 1024 /*barriers*/ + (TC_A_TILE - p.a_stage);
  int stages = (budget - fixed) / (p.a_stage + b_bytes);
  if (stages > TC_MAX_STAGES) stages = TC_MAX_STAGES;
  if (stages < 2) stages = 2;
  p.stages = stages;
  const int a_region = (stages - 1) * p.a_stage + TC_A_TILE;
  p.smem = 1024 + a_region + stages * b_bytes + 1024;
}

// 1 if the sizes can go through mb_gemm_tc, else 0 with the reason in mb_last_error().
MB_EXPORT int mb_gemm_tc_supported(const void* A, int lda, const void* W, int M, int N, int K) {
  if (K % 8 || lda % 8) { snprintf(g_mb_error, sizeof(g_mb_error), "K = %d (lda %d) is no multiple of 8", K, lda); return 0; }
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) { snprintf(g_mb_error, sizeof(g_mb_error), "operands are not 16-byte aligned"); return 0; }
  if (K < 8 || M <= 0 || N <= 0) return 0;
  return 1;
}

// C[M, N] (row stride ldc; bfloat16 or float32) = A[M, K] (row stride lda) · W[N, K]ᵀ
// (epilogue 0), C += ... (1, float32 C), or C[M, N / 2] = SwiGLU over a W whose rows alternate
// gate and up (3, bfloat16 C). `workspace` (float32, may be null) lets the K range be split;
// `error` is a device word that receives a non-zero code if a wait in the kernel ran out
// (1 load, 2 MMA, 3 epilogue). `sms`: the number of SMs of the device. `defer`: when K was split
// (mb_gemm_tc_last_splits() > 1) the partial sums stay in the workspace as [splits][M][N] and C
// is not touched: the caller's next kernel adds them up.
MB_EXPORT int mb_gemm_tc(const void* A, int lda, const void* W, void* C, int c_dtype, int ldc,
                         int M, int N, int K, int epilogue, float* workspace,
                         long long workspace_floats, int defer, int* error, int sms,
                         void* stream) {
  g_last_splits = 1;
  if (M <= 0 || N <= 0) return 0;
  if (!mb_gemm_tc_supported(A, lda, W, M, N, K)) return -1;
  if (epilogue != TC_STORE && epilogue != TC_ADD && epilogue != TC_SWIGLU)
    MB_FAIL("mb_gemm_tc: epilogue %d", epilogue);
  if (epilogue == TC_ADD && c_dtype != MB_F32) MB_FAIL("mb_gemm_tc: the residual is float32");
  if (epilogue == TC_SWIGLU && (c_dtype != MB_BF16 || (N & 1)))
    MB_FAIL("mb_gemm_tc: SwiGLU writes bfloat16 from an even number of rows (%d)", N);
  cudaStream_t s = (cudaStream_t)stream;
  const bool swap = M <= 64;
  int bn;
  if (swap) bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  else bn = N >= 256 ? 256 : (N > 64 ? 128 : 64);
  const int rowsA = swap ? N : M, rowsB = swap ? M : N;
  const int nkb = (K + TC_BK - 1) / TC_BK;
  TcPlan p;
  p.splits = 1;
  p.kb_per_split = nkb;
  if (swap) {
    // Two CTAs share an SM (about half the shared memory each), so 2 * sms CTAs run at once.
    // A weight with at least that many 128-row tiles streams tile by tile. One with fewer
    // tiles than that, but more than sms, gets tiles of fewer rows so that one round of
    // 2 * sms CTAs covers it evenly. One with at most sms tiles keeps its 128-row tiles (large
    // TMA boxes) and splits K so that tiles * splits fills the 2 * sms places.
    const int slots = 2 * sms;
    const int tiles128 = (N + TC_BM - 1) / TC_BM;
    int rows = TC_BM;
    if (tiles128 > sms && tiles128 < slots) {
      rows = (N + slots - 1) / slots;
      rows += rows & 1;  // gate/up pairs stay in one tile
    }
    p.tile_rows = rows;
    p.max_ctas = slots;
    plan_stages(p, bn, 110 * 1024);
    if (workspace && epilogue != TC_SWIGLU && tiles128 <= sms && nkb >= 8) {
      int want = slots / tiles128;
      if (want > TC_MAX_SPLITS) want = TC_MAX_SPLITS;  // what the consumer adds up in one round of loads
      if (want > nkb / 4) want = nkb / 4;
      const long long per = (long long)M * N;
      if (want > workspace_floats / per) want = (int)(workspace_floats / per);
      if (want > 1) p.splits = want;
    }
    p.kb_per_split = (nkb + p.splits - 1) / p.splits;
    p.splits = (nkb + p.kb_per_split - 1) / p.kb_per_split;
  } else {
    p.tile_rows = TC_BM;
    p.max_ctas = sms;
    plan_stages(p, bn, 200 * 1024);
    p.smem += 4 * 4096;  // the epilogue warps' staging rows
    const int tiles = ((rowsA + TC_BM - 1) / TC_BM) * ((rowsB + bn - 1) / bn);
    if (workspace && epilogue != TC_SWIGLU && tiles < sms && nkb >= 8) {
      int want = (2 * sms + tiles - 1) / tiles;
      if (want > nkb / 4) want = nkb / 4;
      const long long per = (long long)M * N;
      if (want > workspace_floats / per) want = (int)(workspace_floats / per);
      if (want > 1) p.splits = want;
    }
    p.kb_per_split = (nkb + p.splits - 1) / p.splits;
    p.splits = (nkb + p.kb_per_split - 1) / p.kb_per_split;
  }
  // more than 128 tokens: tiles of 256 tokens on CTA pairs, even where the last tile is
  // mostly empty (520 tokens: 10.2 ms a pass of the 8B shape against 11.4 on single CTAs)
  const int pairs = (!swap && N >= 256 && M > 128) ? pair_capacity(sms) : 0;
  if (pairs > 0) {
    const int tiles_m = (M + 255) / 256;
    const int bn = pair_tile_width(N, tiles_m, pairs);
    const int tiles_n = (N + bn - 1) / bn;
    const int tiles = tiles_m * tiles_n;
    p.splits = 1;
    if (workspace && epilogue != TC_SWIGLU && tiles < pairs && nkb >= 8) {
      int want = (2 * pairs + tiles - 1) / tiles;
      if (want > nkb / 4) want = nkb / 4;
      const long long per = (long long)M * N;
      if (want > workspace_floats / per) want = (int)(workspace_floats / per);
      if (want > 1) p.splits = want;
    }
    p.kb_per_split = (nkb + p.splits - 1) / p.splits;
    p.splits = (nkb + p.kb_per_split - 1) / p.kb_per_split;
    CUtensorMap tmA, tmB;
    if (!mb_make_map_bf16(&tmA, A, M, K, lda, 128, "mb_gemm_tc input")) return -1;
    if (!mb_make_map_bf16(&tmB, W, N, K, K, bn / 2, "mb_gemm_tc weight")) return -1;
    const int mode = p.splits > 1 ? TC_PARTIAL : epilogue;
    float* partial = p.splits > 1 ? workspace : nullptr;
    int rc = 0;
    switch (bn) {
#define PAIR(W_)                                                                                \
  case W_:                                                                                      \
    rc = launch_pair<W_>(tmA, tmB, C, c_dtype, (long long)ldc, M, N, K, p.kb_per_split, mode,   \
                         partial, tiles_m, tiles_n, p.splits, pairs, error, s);                 \
    break
      PAIR(256); PAIR(240); PAIR(224); PAIR(208); PAIR(192); PAIR(176); PAIR(160); PAIR(144);
      PAIR(128);
#undef PAIR
      default: MB_FAIL("mb_gemm_tc (pairs): tile width %d", bn);
    }
    if (rc) return rc;
    g_last_launches = (p.splits > 1 && !defer) ? 2 : 1;
    g_last_splits = p.splits;
    if (p.splits > 1 && !defer) {
      const size_t total = (size_t)M * N;
      const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
      mb_launch(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, s, workspace, p.splits,
                (long long)M * N, C, c_dtype, (long long)ldc, M, N, epilogue);
      MB_CHECK_LAUNCH("mb_gemm_tc reduce");
    }
    return 0;
  }
  CUtensorMap tmA, tmB;
  if (swap) {
    if (!mb_make_map_bf16(&tmA, W, N, K, K, p.tile_rows, "mb_gemm_tc weight")) return -1;
    if (!mb_make_map_bf16(&tmB, A, M, K, lda, bn, "mb_gemm_tc input")) return -1;
  } else {
    if (!mb_make_map_bf16(&tmA, A, M, K, lda, TC_BM, "mb_gemm_tc input")) return -1;
    if (!mb_make_map_bf16(&tmB, W, N, K, K, bn, "mb_gemm_tc weight")) return -1;
  }
  const int mode = p.splits > 1 ? TC_PARTIAL : epilogue;
  float* partial = p.splits > 1 ? workspace : nullptr;
  const long long pstride = (long long)M * N, pld = N;
  int rc;
#define GO(BN_, SW_)                                                                        \
  rc = launch_tc<BN_, SW_>(tmA, tmB, C, c_dtype, ldc, rowsA, rowsB, K, p, mode, partial,    \
                           pstride, pld, error, s)
  if (swap) {
    if (bn == 16) GO(16, true); else if (bn == 32) GO(32, true); else GO(64, true);
  } else {
    if (bn == 256) GO(256, false); else if (bn == 128) GO(128, false); else GO(64, false);
  }
#undef GO
  if (rc) return rc;
  g_last_launches = (p.splits > 1 && !defer) ? 2 : 1;
  g_last_splits = p.splits;
  if (p.splits > 1 && !defer) {
    const size_t total = (size_t)M * N;
    const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    mb_launch(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, s, workspace, p.splits, pstride, C, c_dtype, ldc, M,
                                                N, epilogue);
    MB_CHECK_LAUNCH("mb_gemm_tc reduce");
  }
  return 0;
}

// ------------------------------------------------------------------ the bounded wait, by itself
// One warp waits on a barrier that nothing ever completes, with a limit of `tries` (a few
// thousand: milliseconds), gives up, records `code` in *error and returns: the way every wait
// of the kernels above ends when what it waits for never comes. It holds no tensor memory and
// has no copy in flight, so there is nothing else to release.
__global__ void wait_selftest_kernel(int* error, int code, unsigned tries, int* gave_up) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(b, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait_tries(b, 0, error, code, tries);
    *gave_up = ok ? 0 : 1;
  }
}

MB_EXPORT int mb_wait_selftest(int* error, int code, unsigned tries, int* gave_up, void* stream) {
  if (tries == 0 || tries > (1u << 16)) MB_FAIL("mb_wait_selftest: 1 to 65536 tries, not %u", tries);
  wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(error, code, tries, gave_up);
  MB_CHECK_LAUNCH("mb_wait_selftest");
}
