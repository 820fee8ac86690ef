// Causal prefill attention over the paged cache on the fifth-generation tensor cores, for
// bfloat16 heads of 128 values: S = Q·Kᵀ and O += P·V are tcgen05.mma instructions with their
// accumulators in tensor memory, the tiles of Q, K and V come by TMA (128-byte swizzle), the
// softmax runs in float32 on four warps that read S from tensor memory, one row a thread.
//
// A CTA takes 128 consecutive new tokens of one sequence and one query head and walks the
// pages of the cache that these tokens see (64 keys a page):
//   warp 0      loads Q once, then K and V of page after page into rings of two stages each
//               (K one page ahead of V: its stage is free again after the first product);
//   warp 1      issues S = Q·Kᵀ (128 x 64), and when P is ready O += P·V (128 x 128);
//   warps 2-5   read S, mask it (causal bound and window by position), keep the row maximum
//               and sum, write P = exp2(S - max) as bfloat16 into shared memory for the second
//               product, and rescale O in tensor memory when a row's maximum has grown by
//               more than 2^8 since O was last rescaled (else the old maximum stays the
//               reference: the result is the same, the sum just carries the factor);
//               at the end they divide O by the row sums and store it.
// Two CTAs share an SM, so that one CTA's products run under the other's softmax.
//
// The formula is the reference's (src/infer/mormot.ai.infer.backend.cpu.pas:1296-1353 of the
// reference project); its own kernel is `attention` in tools/cuda/ops.cu:352-540.
#include "tc_common.cuh"

MB_DEFINE_LAST_ERROR

typedef __nv_bfloat16 bf16;

#define AT_ROWS 128
#define AT_HD 128
#define AT_STAGES 2
#define AT_THREADS 192
#define AT_Q_BYTES (AT_ROWS * AT_HD * 2)    // 32 KB: two 128 x 64 halves
#define AT_KV_BYTES (MB_PAGE * AT_HD * 2)   // 16 KB: two 64 x 64 halves
#define AT_P_BYTES (AT_ROWS * MB_PAGE * 2)  // 16 KB: 128 rows of 64 keys
// no slack for alignment: two CTAs must fit in one SM; the kernel checks that its dynamic
// shared memory starts on a 1024-byte boundary (it does when there is no static shared memory)
#define AT_SMEM (AT_Q_BYTES + AT_STAGES * 2 * AT_KV_BYTES + AT_P_BYTES + 256)
#define AT_TMEM_COLS 256                    // S: 64 columns, O: 128 columns

// Operand descriptor of an MN-major tile written by TMA with the 128-byte swizzle: rows of 64
// values (128 bytes) are consecutive values of the K dimension (here: keys), 8 rows make a
// swizzle atom of 1024 bytes, the atoms of further keys follow one another (stride byte
// offset 1024); a second block of 64 values along N would lie `lbo` bytes on (unused here:
// every MMA takes 64 values of N).
__device__ __forceinline__ uint64_t umma_desc_mn128(uint32_t smem_addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])),
        "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])),
        "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
        "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// 2^x by the special-function unit (x <= 8 here; -inf gives 0)
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__global__ void __launch_bounds__(AT_THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ,
                       const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, bf16* __restrict__ out,
                       int out_stride, const int* __restrict__ page_table, int max_pages,
                       int ring_pages, const int* __restrict__ seq_start,
                       const int* __restrict__ seq_past, const int* __restrict__ seq_slot, int nh,
                       int nkv, int window, float scale_log2, int* __restrict__ error) {
  extern __shared__ __align__(1024) uint8_t at_smem[];
  const uint32_t raw = smem_u32(at_smem);
  if (raw & 1023u) {  // swizzled tiles need it; never seen, but a wrong result must not follow
    if (threadIdx.x == 0 && error) atomicCAS(error, 0, 19);
    return;
  }
  const uint32_t sQ = raw;
  const uint32_t sK = sQ + AT_Q_BYTES;                  // [stage][16 KB]
  const uint32_t sV = sK + AT_STAGES * AT_KV_BYTES;
  const uint32_t sP = sV + AT_STAGES * AT_KV_BYTES;
  const uint32_t bars = sP + AT_P_BYTES;
  const uint32_t q_full = bars, k_full0 = bars + 8, k_empty0 = k_full0 + 8 * AT_STAGES;
  const uint32_t v_full0 = k_empty0 + 8 * AT_STAGES, v_empty0 = v_full0 + 8 * AT_STAGES;
  const uint32_t s_full = v_empty0 + 8 * AT_STAGES, s_free = s_full + 8, p_full = s_full + 16;
  const uint32_t o_done = s_full + 24, slot = s_full + 32;
  volatile uint32_t* slot_ptr = (volatile uint32_t*)(at_smem + (slot - raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heads fastest (the query heads of one KV head run side by side and share its pages in L2),
  // and the last row tiles, which see the most pages, first
  const int b = blockIdx.z, h = blockIdx.x;
  const int start = seq_start[b], n_new = seq_start[b + 1] - start;
  const int row0 = (int)(gridDim.y - 1 - blockIdx.y) * AT_ROWS;
  if (row0 >= n_new) return;  // the whole CTA, before anything is set up
  const int past = seq_past[b], slot_of_seq = seq_slot[b];
  const int g = h / (nh / nkv);
  const int first_pos = past + row0, last_pos = past + min(row0 + AT_ROWS - 1, n_new - 1);
  const int cta_lo = (window > 0 && first_pos + 1 > window) ? first_pos + 1 - window : 0;
  const int page0 = cta_lo / MB_PAGE, n_pages = last_pos / MB_PAGE - page0 + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < AT_STAGES; ++i) {
      mbar_init(k_full0 + 8 * i, 1);
      mbar_init(k_empty0 + 8 * i, 1);
      mbar_init(v_full0 + 8 * i, 1);
      mbar_init(v_empty0 + 8 * i, 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, 4);
    mbar_init(p_full, 4);
    mbar_init(o_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) tmem_alloc(slot, AT_TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *slot_ptr;
  const uint32_t tS = tmem, tO = tmem + 64;
  mb_grid_wait();  // q and the newest keys and values come from the kernel before
  mb_grid_launch_next();

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(q_full, AT_Q_BYTES);
      tma_load_2d(sQ, &tmQ, h * AT_HD, start + row0, q_full);
      tma_load_2d(sQ + AT_Q_BYTES / 2, &tmQ, h * AT_HD + 64, start + row0, q_full);
      // K of a page is free again after the first product of the page two before, V only after
      // its second product: K runs one page ahead of V so that neither load waits for the other
      auto row_of = [&](int j) {
        const int p = page0 + j;
        const int page =
            page_table[(size_t)slot_of_seq * max_pages + (ring_pages > 0 ? p % ring_pages : p)];
        return (page * nkv + g) * MB_PAGE;
      };
      auto load_k = [&](int j) {
        const int st = j % AT_STAGES, y = row_of(j);
        mbar_wait(k_empty0 + 8 * st, ((j / AT_STAGES) & 1) ^ 1, error, 11);
        mbar_expect_tx(k_full0 + 8 * st, AT_KV_BYTES);
        tma_load_2d(sK + st * AT_KV_BYTES, &tmK, 0, y, k_full0 + 8 * st);
        tma_load_2d(sK + st * AT_KV_BYTES + AT_KV_BYTES / 2, &tmK, 64, y, k_full0 + 8 * st);
      };
      load_k(0);
      for (int j = 0; j < n_pages; ++j) {
        if (j + 1 < n_pages) load_k(j + 1);
        const int st = j % AT_STAGES, y = row_of(j);
        mbar_wait(v_empty0 + 8 * st, ((j / AT_STAGES) & 1) ^ 1, error, 10);
        mbar_expect_tx(v_full0 + 8 * st, AT_KV_BYTES);
        tma_load_2d(sV + st * AT_KV_BYTES, &tmV, 0, y, v_full0 + 8 * st);
        tma_load_2d(sV + st * AT_KV_BYTES + AT_KV_BYTES / 2, &tmV, 64, y, v_full0 + 8 * st);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(AT_ROWS, MB_PAGE);             // K-major both
      constexpr uint32_t idesc_o = umma_idesc_bf16(AT_ROWS, 64) | (1u << 16);     // B MN-major
      mbar_wait(q_full, 0, error, 12);
      // S of page j + 1 is issued before the wait for P of page j, so that the softmax of a
      // page finds its scores ready and the first product runs under the softmax before it
      auto issue_s = [&](int j) {
        const int st = j % AT_STAGES;
        mbar_wait(k_full0 + 8 * st, (j / AT_STAGES) & 1, error, 13);
        if (j > 0) mbar_wait(s_free, (j - 1) & 1, error, 14);  // S of the page before was read
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < AT_HD / 16; ++k) {
          const uint64_t da = umma_desc_k128(sQ + (k / 4) * (AT_Q_BYTES / 2) + (k % 4) * 32);
          const uint64_t db =
              umma_desc_k128(sK + st * AT_KV_BYTES + (k / 4) * (AT_KV_BYTES / 2) + (k % 4) * 32);
          umma_bf16(tS, da, db, idesc_s, k > 0);
        }
        umma_commit(k_empty0 + 8 * st);  // K of this page has been read
        umma_commit(s_full);
      };
      issue_s(0);
      for (int j = 0; j < n_pages; ++j) {
        const int st = j % AT_STAGES;
        if (j + 1 < n_pages) issue_s(j + 1);
        mbar_wait(v_full0 + 8 * st, (j / AT_STAGES) & 1, error, 9);
        mbar_wait(p_full, j & 1, error, 15);  // P of this page is in shared memory
        tc_fence_after_sync();
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int k = 0; k < MB_PAGE / 16; ++k) {
            const uint64_t da = umma_desc_k128(sP + k * 32);
            const uint64_t db = umma_desc_mn128(
                sV + st * AT_KV_BYTES + half * (AT_KV_BYTES / 2) + k * 2048, AT_KV_BYTES / 2);
            umma_bf16(tO + half * 64, da, db, idesc_o, (j | k) != 0);
          }
        umma_commit(v_empty0 + 8 * st);  // V of this page has been read
        umma_commit(o_done);
      }
    }
  } else {
    const int q = warp & 3;  // the TMEM lanes of this warp
    const int row = q * 32 + lane;
    const int pos = past + row0 + row;  // position of this thread's token
    const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    float m_ref = -INFINITY, l = 0.f;
    for (int j = 0; j < n_pages; ++j) {
      mbar_wait(s_full, j & 1, error, 16);
      tc_fence_after_sync();
      float s[MB_PAGE];
#pragma unroll
      for (int c0 = 0; c0 < MB_PAGE; c0 += 16) tmem_ld16(tS + lane_addr + c0, s + c0);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
      const int key0 = (page0 + j) * MB_PAGE;
      float mx = -INFINITY;
      // a page that every row of the warp sees whole needs no mask (uniform over the warp)
      const bool whole = key0 + MB_PAGE - 1 <= pos - lane &&
                         (window == 0 || key0 >= lo + (31 - lane));
      if (whole) {
#pragma unroll
        for (int c = 0; c < MB_PAGE; ++c) {
          s[c] *= scale_log2;
          mx = fmaxf(mx, s[c]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < MB_PAGE; ++c) {
          const int key = key0 + c;
          s[c] = (key >= lo && key <= pos) ? s[c] * scale_log2 : -INFINITY;
          mx = fmaxf(mx, s[c]);
        }
      }
      // O is rescaled only when this row's maximum has grown by more than 2^8 (or appears for
      // the first time); until then the old reference stays and P may reach 2^8
      const bool grow = mx > m_ref + 8.0f || (m_ref == -INFINITY && mx > -INFINITY);
      if (j > 0) mbar_wait(o_done, (j - 1) & 1, error, 17);  // O and P are free again
      if (__any_sync(0xffffffffu, grow)) {
        const float f = grow ? (m_ref == -INFINITY ? 0.f : exp2f(m_ref - mx)) : 1.f;
        if (j > 0) {
          tc_fence_after_sync();
#pragma unroll 1
          for (int c0 = 0; c0 < AT_HD; c0 += 16) {
            float o[16];
            tmem_ld16(tO + lane_addr + c0, o);
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] *= f;
            tmem_st16(tO + lane_addr + c0, o);
          }
          tmem_wait_st();
        }
        l *= f;
        if (grow) m_ref = mx;
      }
      const float ref = m_ref == -INFINITY ? 0.f : m_ref;
      // P as the first operand of the second product: row `row` of a K-major tile of 128-byte
      // rows with the 128-byte swizzle (the 16-byte chunk c goes to chunk c ^ (row % 8))
      const uint32_t prow = sP + row * 128;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float p0 = ex2(s[c8 * 8 + 2 * i] - ref), p1 = ex2(s[c8 * 8 + 2 * i + 1] - ref);
          l += p0 + p1;
          __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
          w[i] = *reinterpret_cast<uint32_t*>(&v);
        }
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(prow + ((c8 ^ (row & 7)) << 4)),
                     "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                     : "memory");
      }
      fence_async_smem();  // the tensor core reads P through the asynchronous proxy
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    mbar_wait(o_done, (n_pages - 1) & 1, error, 18);
    tc_fence_after_sync();
    const float inv = 1.0f / l;
    const bool mine = row0 + row < n_new;
    bf16* dst = out + (size_t)(start + row0 + row) * out_stride + (size_t)h * AT_HD;
#pragma unroll 1
    for (int c0 = 0; c0 < AT_HD; c0 += 16) {
      float o[16];
      tmem_ld16(tO + lane_addr + c0, o);
      if (mine) {
        __nv_bfloat162 hv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) hv[i] = __floats2bfloat162_rn(o[2 * i] * inv, o[2 * i + 1] * inv);
        uint4* p = (uint4*)(dst + c0);
        p[0] = *(uint4*)&hv[0];
        p[1] = *(uint4*)&hv[4];
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, AT_TMEM_COLS);
}

// out[t, h, :] for the new tokens of B sequences over the cache, heads of 128 values.
// q: [T, q_cols] bfloat16 with head h of token t at q + t * q_stride + h * 128 (the fused qkv
// rows serve); kpool / vpool: [pool_rows, 128] with pool_rows = pages * kv_heads * 64.
// `error`: a device word that receives 9..19 if a wait in the kernel ran out.
MB_EXPORT int mb_attention_prefill_tc(const void* q, int q_stride, int q_cols, void* out,
                                      int out_stride, const void* kpool, const void* vpool,
                                      long long pool_rows, const int* page_table, int max_pages,
                                      int ring_pages, const int* seq_start, const int* seq_past,
                                      const int* seq_slot, int B, int T, int max_new, int nh,
                                      int nkv, int hd, int window, float scale, int* error,
                                      void* stream) {
  if (B <= 0 || max_new <= 0) return 0;
  if (hd != AT_HD) MB_FAIL("mb_attention_prefill_tc: heads of %d values (128 only)", hd);
  if (nkv <= 0 || nh % nkv) MB_FAIL("mb_attention_prefill_tc: %d heads on %d KV heads", nh, nkv);
  if (((uintptr_t)out & 15) || (out_stride & 7))
    MB_FAIL("mb_attention_prefill_tc: out is not 16-byte aligned (stride %d)", out_stride);
  if (B > 65535 || nh > 65535) MB_FAIL("mb_attention_prefill_tc: %d sequences, %d heads", B, nh);
  CUtensorMap tmQ, tmK, tmV;
  if (!mb_make_map_bf16(&tmQ, q, T, q_cols, q_stride, AT_ROWS, "mb_attention_prefill_tc q")) return -1;
  if (!mb_make_map_bf16(&tmK, kpool, pool_rows, hd, hd, MB_PAGE, "mb_attention_prefill_tc k")) return -1;
  if (!mb_make_map_bf16(&tmV, vpool, pool_rows, hd, hd, MB_PAGE, "mb_attention_prefill_tc v")) return -1;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM);
    if (e != cudaSuccess) MB_FAIL("mb_attention_prefill_tc: %s", cudaGetErrorString(e));
    configured = true;
  }
  const int tiles = (max_new + AT_ROWS - 1) / AT_ROWS;
  if (tiles > 65535) MB_FAIL("mb_attention_prefill_tc: %d new tokens in one sequence", max_new);
  dim3 grid(nh, tiles, B);
  mb_launch(attn_prefill_tc_kernel, grid, dim3(AT_THREADS), AT_SMEM, (cudaStream_t)stream, tmQ,
            tmK, tmV, (bf16*)out, out_stride, page_table, max_pages, ring_pages, seq_start,
            seq_past, seq_slot, nh, nkv, window, scale * 1.4426950408889634f, error);
  MB_CHECK_LAUNCH("mb_attention_prefill_tc");
}
