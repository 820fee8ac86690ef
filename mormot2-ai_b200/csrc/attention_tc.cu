// Causal prefill attention over the paged cache on the fifth-generation tensor cores, for
// bfloat16 heads of 128 values: S = Q·Kᵀ and O += P·V are tcgen05.mma instructions with their
// accumulators in tensor memory, the tiles of Q, K and V come by TMA (128-byte swizzle), the
// softmax runs in float32 on four warps that read S from tensor memory, one row a thread.
//
// A CTA takes 128 consecutive new tokens of one sequence and one query head and walks the
// pages of the cache that these tokens see (64 keys a page):
//   warp 0      loads Q once, then K and V of page after page into rings of three and two stages
//               (K ahead of V: its stage is free again after the first product);
//   warp 1      issues S = Q·Kᵀ (128 x 64) two pages ahead into one of two S buffers in tensor
//               memory, and when P of a page is ready O += P·V (128 x 128) with P as the
//               operand that lies in tensor memory;
//   warps 2-5   read S, mask it (causal bound and window by position), keep the row maximum
//               and sum, and write P = exp2(S - max) as bfloat16 over the S they have just read
//               (the second product takes it from there), so that the softmax of a page never
//               waits for the product of the page before; they rescale O in tensor memory only
//               when a row's maximum has grown by more than 2^8 since O was last rescaled
//               (else the old maximum stays the reference: the result is the same, the sum
//               just carries the factor), and only then wait for the products in flight;
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
#define AT_K_STAGES 3
#define AT_V_STAGES 2
#define AT_THREADS 192
#define AT_Q_BYTES (AT_ROWS * AT_HD * 2)    // 32 KB: two 128 x 64 halves
#define AT_KV_BYTES (MB_PAGE * AT_HD * 2)   // 16 KB: two 64 x 64 halves
// no slack for alignment: two CTAs must fit in one SM; the kernel checks that its dynamic
// shared memory starts on a 1024-byte boundary (it does when there is no static shared memory)
#define AT_SMEM (AT_Q_BYTES + (AT_K_STAGES + AT_V_STAGES) * AT_KV_BYTES + 256)
#define AT_TMEM_COLS 256                    // two S buffers of 64 columns, O: 128 columns

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
// two float32 values in one 64-bit register, and arithmetic on both at once
__device__ __forceinline__ unsigned long long pack2(float a, float b) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long r, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(r));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b,
                                                   unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// the largest of three in one instruction
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 64 consecutive float32 columns of this thread's TMEM lane: four loads in flight, one wait.
// The loaded registers pass through the wait (and through empty statements after it) so that
// no use of them can be scheduled before it.
#define AT_LD16(R, OFF)                                                                          \
  asm volatile(                                                                                  \
      "tcgen05.ld.sync.aligned.32x32b.x16.b32"                                                   \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"         \
      : "=r"(R[0]), "=r"(R[1]), "=r"(R[2]), "=r"(R[3]), "=r"(R[4]), "=r"(R[5]), "=r"(R[6]),      \
        "=r"(R[7]), "=r"(R[8]), "=r"(R[9]), "=r"(R[10]), "=r"(R[11]), "=r"(R[12]), "=r"(R[13]),  \
        "=r"(R[14]), "=r"(R[15])                                                                 \
      : "r"(taddr + OFF))
#define AT_HOLD16(TEXT, R)                                                                       \
  asm volatile(TEXT                                                                              \
               : "+r"(R[0]), "+r"(R[1]), "+r"(R[2]), "+r"(R[3]), "+r"(R[4]), "+r"(R[5]),         \
                 "+r"(R[6]), "+r"(R[7]), "+r"(R[8]), "+r"(R[9]), "+r"(R[10]), "+r"(R[11]),       \
                 "+r"(R[12]), "+r"(R[13]), "+r"(R[14]), "+r"(R[15])                              \
               :                                                                                 \
               : "memory")
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float* v) {
  uint32_t a[16], b[16], c[16], d[16];
  AT_LD16(a, 0);
  AT_LD16(b, 16);
  AT_LD16(c, 32);
  AT_LD16(d, 48);
  AT_HOLD16("tcgen05.wait::ld.sync.aligned;", a);
  AT_HOLD16("", b);
  AT_HOLD16("", c);
  AT_HOLD16("", d);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    v[i] = __uint_as_float(a[i]);
    v[16 + i] = __uint_as_float(b[i]);
    v[32 + i] = __uint_as_float(c[i]);
    v[48 + i] = __uint_as_float(d[i]);
  }
}

// 16 packed words (32 bfloat16 values) into this thread's TMEM lane
__device__ __forceinline__ void tmem_st16_u32(uint32_t taddr, const uint32_t* w) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
      ::"r"(taddr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]),
        "r"(w[7]), "r"(w[8]), "r"(w[9]), "r"(w[10]), "r"(w[11]), "r"(w[12]), "r"(w[13]),
        "r"(w[14]), "r"(w[15])
      : "memory");
}

// D[tmem] (+)= A[tmem] · B[smem]: the first operand (128 rows x 16 bfloat16 values, two values
// a 32-bit column, 8 columns) lies in tensor memory. Issued by one thread.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
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
  const uint32_t sV = sK + AT_K_STAGES * AT_KV_BYTES;
  const uint32_t bars = sV + AT_V_STAGES * AT_KV_BYTES;
  const uint32_t q_full = bars, k_full0 = bars + 8, k_empty0 = k_full0 + 8 * AT_K_STAGES;
  const uint32_t v_full0 = k_empty0 + 8 * AT_K_STAGES, v_empty0 = v_full0 + 8 * AT_V_STAGES;
  const uint32_t s_full0 = v_empty0 + 8 * AT_V_STAGES;  // one for each of the two S buffers
  const uint32_t p_full0 = s_full0 + 16;                // and for the P written over each
  // the second product of page j done: barrier j % 2 (a waiter may have skipped the page
  // before, and one barrier could then be two phases on, which a parity cannot tell)
  const uint32_t o_done0 = p_full0 + 16, slot = o_done0 + 16;
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
    for (int i = 0; i < AT_K_STAGES; ++i) {
      mbar_init(k_full0 + 8 * i, 1);
      mbar_init(k_empty0 + 8 * i, 1);
    }
    for (int i = 0; i < AT_V_STAGES; ++i) {
      mbar_init(v_full0 + 8 * i, 1);
      mbar_init(v_empty0 + 8 * i, 1);
    }
    mbar_init(s_full0, 1);
    mbar_init(s_full0 + 8, 1);
    mbar_init(p_full0, 4);
    mbar_init(p_full0 + 8, 4);
    mbar_init(o_done0, 1);
    mbar_init(o_done0 + 8, 1);
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
  const uint32_t tS = tmem, tO = tmem + 128;  // S (and then P) of page j in tS + 64 * (j % 2)
  mb_grid_wait();  // q and the newest keys and values come from the kernel before
  mb_grid_launch_next();

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(q_full, AT_Q_BYTES);
      tma_load_2d(sQ, &tmQ, h * AT_HD, start + row0, q_full);
      tma_load_2d(sQ + AT_Q_BYTES / 2, &tmQ, h * AT_HD + 64, start + row0, q_full);
      // the first products run two pages ahead of the second ones: so do the loads of K
      auto row_of = [&](int j) {
        const int p = page0 + j;
        const int entry = ring_pages > 0 ? p % ring_pages : p;
        int page = MB_INDEX_OK(entry < max_pages, 1, slot_of_seq, p, max_pages)
                       ? page_table[(size_t)slot_of_seq * max_pages + entry] : 0;
        if (!MB_INDEX_OK(page >= 0, 2, slot_of_seq, entry, page)) page = 0;
        return (page * nkv + g) * MB_PAGE;
      };
      auto load_k = [&](int j) {
        const int st = j % AT_K_STAGES, y = row_of(j);
        mbar_wait(k_empty0 + 8 * st, ((j / AT_K_STAGES) & 1) ^ 1, error, 11);
        mbar_expect_tx(k_full0 + 8 * st, AT_KV_BYTES);
        tma_load_2d(sK + st * AT_KV_BYTES, &tmK, 0, y, k_full0 + 8 * st);
        tma_load_2d(sK + st * AT_KV_BYTES + AT_KV_BYTES / 2, &tmK, 64, y, k_full0 + 8 * st);
      };
      load_k(0);
      if (n_pages > 1) load_k(1);
      for (int j = 0; j < n_pages; ++j) {
        if (j + 2 < n_pages) load_k(j + 2);
        const int st = j % AT_V_STAGES, y = row_of(j);
        mbar_wait(v_empty0 + 8 * st, ((j / AT_V_STAGES) & 1) ^ 1, error, 10);
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
      // S of page j goes into buffer j % 2, which held S and then P of page j - 2
      auto issue_s = [&](int j) {
        const int st = j % AT_K_STAGES;
        mbar_wait(k_full0 + 8 * st, (j / AT_K_STAGES) & 1, error, 13);
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < AT_HD / 16; ++k) {
          const uint64_t da = umma_desc_k128(sQ + (k / 4) * (AT_Q_BYTES / 2) + (k % 4) * 32);
          const uint64_t db =
              umma_desc_k128(sK + st * AT_KV_BYTES + (k / 4) * (AT_KV_BYTES / 2) + (k % 4) * 32);
          umma_bf16(tS + 64 * (j & 1), da, db, idesc_s, k > 0);
        }
        umma_commit(k_empty0 + 8 * st);  // K of this page has been read
        umma_commit(s_full0 + 8 * (j & 1));
      };
      issue_s(0);
      if (n_pages > 1) issue_s(1);
      for (int j = 0; j < n_pages; ++j) {
        const int st = j % AT_V_STAGES;
        mbar_wait(v_full0 + 8 * st, (j / AT_V_STAGES) & 1, error, 9);
        // P of this page is in tensor memory (a barrier per buffer: the softmax may be a page
        // ahead of this wait, and one barrier would then be two phases on)
        mbar_wait(p_full0 + 8 * (j & 1), (j >> 1) & 1, error, 15);
        tc_fence_after_sync();
        const uint32_t tP = tS + 64 * (j & 1);
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int k = 0; k < MB_PAGE / 16; ++k) {
            const uint64_t db = umma_desc_mn128(
                sV + st * AT_KV_BYTES + half * (AT_KV_BYTES / 2) + k * 2048, AT_KV_BYTES / 2);
            umma_bf16_ts(tO + half * 64, tP + 8 * k, db, idesc_o, (j | k) != 0);
          }
        umma_commit(v_empty0 + 8 * st);  // V of this page has been read
        umma_commit(o_done0 + 8 * (j & 1));
        if (j + 2 < n_pages) {
          // S of page j + 2 overwrites the P that the product just issued reads as an operand:
          // nothing orders a later instruction's result after an earlier one's operand read in
          // tensor memory, so wait until that product is done (S of page j + 1 is long ready,
          // the softmax does not wait for this)
          mbar_wait(o_done0 + 8 * (j & 1), (j >> 1) & 1, error, 14);
          issue_s(j + 2);
        }
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
      const uint32_t tSj = tS + 64 * (j & 1) + lane_addr;
      mbar_wait(s_full0 + 8 * (j & 1), (j >> 1) & 1, error, 16);
      tc_fence_after_sync();
      float s[MB_PAGE];
      tmem_ld64(tSj, s);
      const int key0 = (page0 + j) * MB_PAGE;
      // a page that every row of the warp sees whole needs no mask (uniform over the warp)
      const bool whole = key0 + MB_PAGE - 1 <= pos - lane &&
                         (window == 0 || key0 >= lo + (31 - lane));
      if (!whole) {
#pragma unroll
        for (int c = 0; c < MB_PAGE; ++c) {
          const int key = key0 + c;
          if (!(key >= lo && key <= pos)) s[c] = -INFINITY;
        }
      }
      // The maximum of the raw scores (the scale is positive, so it is the maximum of the
      // scaled ones too), two scores an instruction in four chains; the scale itself goes into
      // the multiply-add in front of the exponential below.
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < MB_PAGE; c += 2) mx4[(c >> 1) & 3] = max3(mx4[(c >> 1) & 3], s[c], s[c + 1]);
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      // O is rescaled only when this row's maximum has grown by more than 2^8 (or appears for
      // the first time); until then the old reference stays and P may reach 2^8
      const bool grow = mx > m_ref + 8.0f || (m_ref == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float f = grow ? (m_ref == -INFINITY ? 0.f : exp2f(m_ref - mx)) : 1.f;
        if (j > 0) {
          // the second product of the page before adds into O: it must be done (the one of
          // this page waits for the P written below)
          mbar_wait(o_done0 + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1, error, 17);
          tc_fence_after_sync();
#pragma unroll 1
          for (int c0 = 0; c0 < AT_HD; c0 += 16) {
            float o[16];
            tmem_ld16(tO + lane_addr + c0, o);
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] *= f;
            tmem_st16(tO + lane_addr + c0, o);
          }
        }
        l *= f;
        if (grow) m_ref = mx;
      }
      const float ref = m_ref == -INFINITY ? 0.f : m_ref;
      // P over the S just read, as the first operand of the second product: this thread's row,
      // two bfloat16 values a column, keys in order
      // (two scores a multiply-add and two a sum: the exponentials need the issue slots)
      const unsigned long long scale2 = pack2(scale_log2, scale_log2), ref2 = pack2(-ref, -ref);
      unsigned long long l4[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int c16 = 0; c16 < 2; ++c16) {
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x0, x1;
          unpack2(fma2(pack2(s[c16 * 32 + 2 * i], s[c16 * 32 + 2 * i + 1]), scale2, ref2), x0, x1);
          const float p0 = ex2(x0), p1 = ex2(x1);
          l4[i & 3] = add2(l4[i & 3], pack2(p0, p1));
          __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
          w[i] = *reinterpret_cast<uint32_t*>(&v);
        }
        tmem_st16_u32(tSj + 16 * c16, w);
      }
      {
        float a0, a1;
        unpack2(add2(add2(l4[0], l4[1]), add2(l4[2], l4[3])), a0, a1);
        l += a0 + a1;
      }
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full0 + 8 * (j & 1));
    }
    // the last product done means all are (the tensor core works in the order of issue)
    mbar_wait(o_done0 + 8 * ((n_pages - 1) & 1), ((n_pages - 1) >> 1) & 1, error, 18);
    tc_fence_after_sync();
    const float inv = 1.0f / l;
    // A thread holds one row of O; written from there, a warp's store would touch 32 rows with
    // 16 bytes each. Q's shared memory is free now (every product is done): the warp lays its
    // 32 rows of 256 bytes there (16-byte piece p of row r at p ^ (r & 7): no bank conflicts
    // either way) and writes them out two whole rows at a time.
    const uint32_t stage = sQ + (uint32_t)q * (32 * AT_HD * 2);
#pragma unroll 1
    for (int c0 = 0; c0 < AT_HD; c0 += 16) {
      float o[16];
      tmem_ld16(tO + lane_addr + c0, o);
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        __nv_bfloat162 v = __floats2bfloat162_rn(o[2 * i] * inv, o[2 * i + 1] * inv);
        w[i] = *reinterpret_cast<uint32_t*>(&v);
      }
      const int pc = c0 >> 3;
      st_shared_v4(stage + lane * (AT_HD * 2) + ((pc ^ (lane & 7)) << 4),
                   make_uint4(w[0], w[1], w[2], w[3]));
      st_shared_v4(stage + lane * (AT_HD * 2) + (((pc + 1) ^ (lane & 7)) << 4),
                   make_uint4(w[4], w[5], w[6], w[7]));
    }
    __syncwarp();
    const int pc = lane & 15;
#pragma unroll 4
    for (int i = 0; i < 16; ++i) {
      const int r = 2 * i + (lane >> 4);
      if (row0 + q * 32 + r < n_new) {
        const uint4 v = ld_shared_v4(stage + r * (AT_HD * 2) + ((pc ^ (r & 7)) << 4));
        *(uint4*)(out + (size_t)(start + row0 + q * 32 + r) * out_stride + (size_t)h * AT_HD +
                  8 * pc) = v;
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
  if (!(scale > 0.f))  // the row maximum is taken over the scores before they are scaled
    MB_FAIL("mb_attention_prefill_tc: a scale of %g (it must be positive)", (double)scale);
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
