// Attention over the paged cache on the tensor cores (bfloat16 storage, float32 softmax and
// accumulation), for head sizes 64 and 128.
//
// Decode (`mb_attention_decode`, `mb_attention_decode_clusters`): one new token per sequence.
// The query heads that share a KV head are the 16 rows of the m16n8k16 MMA, so the keys and
// values of a sequence are read once for the whole group. The pages of a sequence are split
// over `splits` CTAs (grid.x), the four warps of a CTA take 16 keys of every page each, every
// warp keeps an online softmax of its own, the warps are merged in shared memory, and the
// splits either by a second kernel through scratch memory or, as the CTAs of one thread-block
// cluster, through each other's shared memory (the reference's flash-decoding split +
// `attnmerge`, tools/cuda/ops.cu:325-329, :589-617 of the reference project; its formula
// src/infer/mormot.ai.infer.backend.cpu.pas:1296-1353). The split count is fixed by the
// cache's capacity, not by the lengths, so a captured launch stays valid.
//
// Operands go from global memory straight into MMA fragments with 16-byte loads: the sum over
// the head dimension (for q·k) and over the keys (for p·v) does not care about order, so the
// fragments use a permutation of the dimensions under which every thread's values lie
// contiguous in memory.
#include "mma_common.cuh"
#include "tc_common.cuh"

MB_DEFINE_LAST_ERROR

typedef __nv_bfloat16 bf16;

#define DEC_WARPS 4

// scores of one page: sc[u][e] = q(row) · k(key) for the keys u*8 + 2c + (e & 1) of the page and
// the rows r (e < 2) and r + 8 (e >= 2) of the warp's 16 query rows
template <int HD>
__device__ __forceinline__ void qk_page(const uint4* qa, const uint4* qb, const bf16* kbase, int r,
                                        int c, float sc[8][4]) {
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    sc[u][0] = sc[u][1] = sc[u][2] = sc[u][3] = 0.f;
    const bf16* krow = kbase + (size_t)(u * 8 + r) * HD + c * 8;
#pragma unroll
    for (int ch = 0; ch < HD / 32; ++ch) {
      const uint4 kb = ldg16(krow + ch * 32);
      mma_bf16(sc[u], qa[ch].x, qb[ch].x, qa[ch].y, qb[ch].y, kb.x, kb.y);
      mma_bf16(sc[u], qa[ch].z, qb[ch].z, qa[ch].w, qb[ch].w, kb.z, kb.w);
    }
  }
}

// o += p · v for one page: 16 keys a step; logical column q of output tile j is the dim
// db*64 + q*8 + j, so a thread ends up with 8 consecutive dims per accumulator column
template <int HD>
__device__ __forceinline__ void pv_page(const float sc[8][4], const bf16* vbase, int r, int c,
                                        float o[HD / 64][8][4]) {
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    const uint32_t a0 = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
    const uint32_t a1 = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
    const uint32_t a2 = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
    const uint32_t a3 = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
    const bf16* vrow = vbase + (size_t)(kk * 16 + 2 * c) * HD + r * 8;
#pragma unroll
    for (int db = 0; db < HD / 64; ++db) {
      const uint4 va = ldg16(vrow + db * 64);
      const uint4 vb = ldg16(vrow + HD + db * 64);
      const uint4 vc = ldg16(vrow + 8 * HD + db * 64);
      const uint4 vd = ldg16(vrow + 9 * HD + db * 64);
      const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
      const uint32_t wc[4] = {vc.x, vc.y, vc.z, vc.w}, wd[4] = {vd.x, vd.y, vd.z, vd.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int w = j >> 1;
        const uint32_t b0 = (j & 1) ? pack_hi(wa[w], wb[w]) : pack_lo(wa[w], wb[w]);
        const uint32_t b1 = (j & 1) ? pack_hi(wc[w], wd[w]) : pack_lo(wc[w], wd[w]);
        mma_bf16(o[db][j], a0, a1, a2, a3, b0, b1);
      }
    }
  }
}

// q fragments of the rows r and r + 8 (null: a row that is not there): 8 consecutive dims per
// 32-dim chunk and thread
template <int HD>
__device__ __forceinline__ void load_q(const bf16* q0, const bf16* q1, int c, uint4* qa, uint4* qb) {
#pragma unroll
  for (int ch = 0; ch < HD / 32; ++ch) {
    qa[ch] = q0 ? ldg16(q0 + ch * 32 + c * 8) : make_uint4(0, 0, 0, 0);
    qb[ch] = q1 ? ldg16(q1 + ch * 32 + c * 8) : make_uint4(0, 0, 0, 0);
  }
}

// 16 bytes of a tile in shared memory
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}

// `bytes` contiguous bytes from global to shared memory (both 16-byte aligned), completing `bar`
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

#define DEC_STAGES 3

__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}

// One CTA per (token, KV head [x 16 query heads of its group], split). Warp 4 streams the
// pages of this split (every `splits`-th page of the sequence) into shared memory, a whole K
// tile and a whole V tile per page (16 KB each for heads of 128) by bulk asynchronous copies,
// three pages ahead. Warps 0-3 take 16 keys of every page each.
template <int HD>
__global__ void __launch_bounds__((DEC_WARPS + 1) * 32, 2)
attn_decode_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ kpool,
                   const bf16* __restrict__ vpool, const int* __restrict__ page_table,
                   int max_pages, int ring_pages, const int* __restrict__ tok_slot,
                   const int* __restrict__ tok_pos, int nh,
                   int nkv, int window, float scale_log2, float* __restrict__ part_o,
                   float* __restrict__ part_ml, bf16* __restrict__ out, int out_stride,
                   int in_clusters, int* __restrict__ error) {
  constexpr int CH = HD / 32;  // 32-dim chunks of q·k
  constexpr int DB = HD / 64;  // 64-dim blocks of p·v
  constexpr uint32_t TILE = MB_PAGE * HD * 2;  // bytes of a page's keys (or values)
  MB_TRACE_BEGIN();
  extern __shared__ __align__(128) uint8_t dec_smem[];
  // [stages][K tile | V tile], then the barriers; after the loop the tiles' memory holds the
  // warps' partial results for the merge
  const uint32_t tiles = smem_u32(dec_smem);
  const uint32_t bars = tiles + DEC_STAGES * 2 * TILE;
  const uint32_t full0 = bars, empty0 = bars + 8 * DEC_STAGES;

  const int s = blockIdx.x, S = gridDim.x, t = blockIdx.z;
  const int G = nh / nkv, subs = (G + 15) / 16;
  const int g = blockIdx.y / subs, sub = blockIdx.y % subs;
  const int h0 = g * G + sub * 16;
  const int rows_valid = min(16, G - sub * 16);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, c = lane & 3;

  const int pos = tok_pos[t];
  const int slot = tok_slot[t];
  const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
  const int p_first = lo / MB_PAGE + s, p_last = pos / MB_PAGE;
  const int n_pages = p_first <= p_last ? (p_last - p_first) / S + 1 : 0;  // p_first + i * S

  if (threadIdx.x == 0) {
    for (int i = 0; i < DEC_STAGES; ++i) {
      mbar_init(full0 + 8 * i, 1);
      mbar_init(empty0 + 8 * i, DEC_WARPS);
    }
    mbar_fence_init();
  }
  __syncthreads();

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[DB][8][4];
#pragma unroll
  for (int db = 0; db < DB; ++db)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[db][j][e] = 0.f;

  if (warp == DEC_WARPS) {
    // producer: the lanes fetch the ids of up to 32 pages at once, lane 0 issues the copies.
    // Only the page that holds the newest position is written by the kernel before this one
    // (the index arrays and all older pages were settled long before): the copies of the older
    // pages start at once, the wait for that kernel comes before the first copy of the newest
    // page (and at the latest at the end).
    bool waited = false;
    int st = 0;
    uint32_t ph = 0;
    for (int i0 = 0; i0 < n_pages; i0 += 32) {
      int mine = 0;
      if (i0 + lane < n_pages) {
        const int p = p_first + (i0 + lane) * S;
        const int entry = ring_pages > 0 ? p % ring_pages : p;
        mine = MB_INDEX_OK(entry < max_pages, 1, slot, p, max_pages)
                   ? page_table[(size_t)slot * max_pages + entry] : 0;
        if (!MB_INDEX_OK(mine >= 0, 2, slot, entry, mine)) mine = 0;
      }
      const int n = min(32, n_pages - i0);
      for (int i = 0; i < n; ++i) {
        const int page = __shfl_sync(0xffffffffu, mine, i);
        if (!waited && p_first + (i0 + i) * S == p_last) {
          mb_grid_wait();
          waited = true;
        }
        if (lane == 0) {
          mbar_wait(empty0 + 8 * st, ph ^ 1, error, 4);
          mbar_expect_tx(full0 + 8 * st, 2 * TILE);
          const size_t at = ((size_t)page * nkv + g) * MB_PAGE * HD;
          bulk_copy(tiles + st * 2 * TILE, kpool + at, TILE, full0 + 8 * st);
          bulk_copy(tiles + st * 2 * TILE + TILE, vpool + at, TILE, full0 + 8 * st);
        }
        if (++st == DEC_STAGES) { st = 0; ph ^= 1; }
      }
    }
    if (!waited) mb_grid_wait();
    mb_grid_launch_next();
  } else {
    mb_grid_wait();  // q comes from the kernel before
    uint4 qa[CH], qb[CH];
    {
      const bf16* qrow = q + (size_t)t * q_stride + (size_t)(h0 + r) * HD;
      load_q<HD>(r < rows_valid ? qrow : nullptr, r + 8 < rows_valid ? qrow + 8 * HD : nullptr, c,
                 qa, qb);
    }
    int st = 0;
    uint32_t ph = 0;
    for (int i = 0; i < n_pages; ++i) {
      const int key0 = (p_first + i * S) * MB_PAGE + 16 * warp;  // this warp's 16 keys
      mbar_wait(full0 + 8 * st, ph, error, 5);
      const uint32_t ks = tiles + st * 2 * TILE + (uint32_t)(16 * warp) * HD * 2;
      const uint32_t vs = ks + TILE;
      float sc[2][4];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        sc[u][0] = sc[u][1] = sc[u][2] = sc[u][3] = 0.f;
        const uint32_t krow = ks + (uint32_t)(u * 8 + r) * HD * 2 + c * 16;
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
          const uint4 kb = lds16(krow + ch * 64);
          mma_bf16(sc[u], qa[ch].x, qb[ch].x, qa[ch].y, qb[ch].y, kb.x, kb.y);
          mma_bf16(sc[u], qa[ch].z, qb[ch].z, qa[ch].w, qb[ch].w, kb.z, kb.w);
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = key0 + u * 8 + 2 * c + e;
          const bool ok = key >= lo && key <= pos;
          sc[u][e] = ok ? sc[u][e] * scale_log2 : -INFINITY;
          sc[u][2 + e] = ok ? sc[u][2 + e] * scale_log2 : -INFINITY;
          mx0 = fmaxf(mx0, sc[u][e]);
          mx1 = fmaxf(mx1, sc[u][2 + e]);
        }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
      // this warp's 16 keys of the page may all lie outside [lo, pos]: keep exp2 off inf - inf
      const float base0 = n0 == -INFINITY ? 0.f : n0, base1 = n1 == -INFINITY ? 0.f : n1;
      const float c0 = exp2f(m0 - base0), c1 = exp2f(m1 - base1);
      m0 = n0;
      m1 = n1;
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          sc[u][e] = exp2f(sc[u][e] - base0);
          sc[u][2 + e] = exp2f(sc[u][2 + e] - base1);
          s0 += sc[u][e];
          s1 += sc[u][2 + e];
        }
      l0 = l0 * c0 + s0;
      l1 = l1 * c1 + s1;
      const uint32_t a0 = pack_bf16(sc[0][0], sc[0][1]), a1 = pack_bf16(sc[0][2], sc[0][3]);
      const uint32_t a2 = pack_bf16(sc[1][0], sc[1][1]), a3 = pack_bf16(sc[1][2], sc[1][3]);
      const uint32_t vrow = vs + (uint32_t)(2 * c) * HD * 2 + r * 16;
#pragma unroll
      for (int db = 0; db < DB; ++db) {
        const uint4 va = lds16(vrow + db * 128);
        const uint4 vb = lds16(vrow + HD * 2 + db * 128);
        const uint4 vc = lds16(vrow + 8 * HD * 2 + db * 128);
        const uint4 vd = lds16(vrow + 9 * HD * 2 + db * 128);
        const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
        const uint32_t wc[4] = {vc.x, vc.y, vc.z, vc.w}, wd[4] = {vd.x, vd.y, vd.z, vd.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[db][j][0] *= c0;
          o[db][j][1] *= c0;
          o[db][j][2] *= c1;
          o[db][j][3] *= c1;
          const int w = j >> 1;
          const uint32_t b0 = (j & 1) ? pack_hi(wa[w], wb[w]) : pack_lo(wa[w], wb[w]);
          const uint32_t b1 = (j & 1) ? pack_hi(wc[w], wd[w]) : pack_lo(wc[w], wd[w]);
          mma_bf16(o[db][j], a0, a1, a2, a3, b0, b1);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * st);  // this warp is done with the stage
      if (++st == DEC_STAGES) { st = 0; ph ^= 1; }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  }
  // every copy has landed and been read: the tiles' memory now holds the warps' results
  __syncthreads();
  float* sm_o = (float*)dec_smem;                       // [DEC_WARPS][16][HD]
  float* sm_m = sm_o + DEC_WARPS * 16 * HD;             // [DEC_WARPS][16]
  float* sm_l = sm_m + DEC_WARPS * 16;                  // [DEC_WARPS][16]
  float* sm_c = sm_l + DEC_WARPS * 16;                  // [16][HD] the CTA's own result
  float* sm_cml = sm_c + 16 * HD;                       // [16] its maxima, [16] its sums
  if (warp < DEC_WARPS) {
    if (c == 0) {
      sm_m[warp * 16 + r] = m0;
      sm_m[warp * 16 + r + 8] = m1;
      sm_l[warp * 16 + r] = l0;
      sm_l[warp * 16 + r + 8] = l1;
    }
#pragma unroll
    for (int db = 0; db < DB; ++db)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int d0 = db * 64 + (2 * c) * 8 + j, d1 = d0 + 8;
        sm_o[(warp * 16 + r) * HD + d0] = o[db][j][0];
        sm_o[(warp * 16 + r) * HD + d1] = o[db][j][1];
        sm_o[(warp * 16 + r + 8) * HD + d0] = o[db][j][2];
        sm_o[(warp * 16 + r + 8) * HD + d1] = o[db][j][3];
      }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows_valid * HD; idx += blockDim.x) {
    const int row = idx / HD, d = idx - row * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm_m[w * 16 + row]);
    float L = 0.f, acc = 0.f;
    if (M > -INFINITY) {
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) {
        const float f = exp2f(sm_m[w * 16 + row] - M);  // 0 for a warp without keys
        L += sm_l[w * 16 + row] * f;
        acc += sm_o[(w * 16 + row) * HD + d] * f;
      }
    }
    if (!in_clusters) {  // through the caller's scratch: the merge kernel adds the splits up
      const size_t at = ((size_t)t * nh + h0 + row) * S + s;
      part_o[at * HD + d] = acc;
      if (d == 0) {
        part_ml[at * 2] = M;
        part_ml[at * 2 + 1] = L;
      }
    } else if (S == 1) {
      out[(size_t)t * out_stride + (size_t)(h0 + row) * HD + d] = __float2bfloat16_rn(acc / L);
    } else {
      sm_c[row * HD + d] = acc;
      if (d == 0) {
        sm_cml[row] = M;
        sm_cml[16 + row] = L;
      }
    }
  }
  if (in_clusters && S > 1) {
    // The splits of a (token, group) are the CTAs of one cluster: each adds up a share of the
    // outputs from all the CTAs' shared memory, in split order.
    cluster_sync_all();
    const int total = rows_valid * HD, share = (total + S - 1) / S;
    const int hi = min(total, (s + 1) * share);
    const uint32_t c_addr = smem_u32(sm_c), ml_addr = smem_u32(sm_cml);
    for (int idx = s * share + threadIdx.x; idx < hi; idx += blockDim.x) {
      const int row = idx / HD, d = idx - row * HD;
      float M = -INFINITY;
      for (int k = 0; k < S; ++k)
        M = fmaxf(M, ld_cluster_f32(cluster_addr_of(ml_addr + 4 * row, k)));
      float L = 0.f, acc = 0.f;
      for (int k = 0; k < S; ++k) {
        const float m = ld_cluster_f32(cluster_addr_of(ml_addr + 4 * row, k));
        const float l = ld_cluster_f32(cluster_addr_of(ml_addr + 4 * (16 + row), k));
        const float v = ld_cluster_f32(cluster_addr_of(c_addr + 4 * (row * HD + d), k));
        const float f = m == -INFINITY ? 0.f : exp2f(m - M);
        L += l * f;
        acc += v * f;
      }
      out[(size_t)t * out_stride + (size_t)(h0 + row) * HD + d] = __float2bfloat16_rn(acc / L);
    }
    cluster_sync_all();  // no CTA leaves while another may still read its shared memory
  }
  MB_TRACE_END(4);
}

// out[t, h, :] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), the splits in order
template <int HD>
__global__ void attn_merge_kernel(const float* __restrict__ part_o,
                                  const float* __restrict__ part_ml, int S, bf16* __restrict__ out,
                                  int out_stride, int nh) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int t = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const size_t at = ((size_t)t * nh + h) * S;
  float M = -INFINITY;
  for (int s = 0; s < S; ++s) M = fmaxf(M, part_ml[(at + s) * 2]);
  float L = 0.f, acc = 0.f;
  for (int s = 0; s < S; ++s) {
    const float m = part_ml[(at + s) * 2];
    if (m == -INFINITY) continue;
    const float f = exp2f(m - M);
    L += part_ml[(at + s) * 2 + 1] * f;
    acc += part_o[(at + s) * HD + d] * f;
  }
  out[(size_t)t * out_stride + (size_t)h * HD + d] = __float2bfloat16_rn(acc / L);
}

// floats of scratch that mb_attention_decode needs for T tokens
MB_EXPORT long long mb_attention_decode_scratch(int T, int nh, int hd, int splits) {
  return (long long)T * nh * splits * (hd + 2);
}

static int decode_checks(const void* q, int q_stride, const void* kpool, const void* vpool, int T,
                         int nh, int nkv, int hd, int splits) {
  if (hd != 64 && hd != 128)
    MB_FAIL("mb_attention_decode: heads of %d values are not supported (64 or 128)", hd);
  if (nkv <= 0 || nh % nkv) MB_FAIL("mb_attention_decode: %d heads on %d KV heads", nh, nkv);
  if (splits <= 0 || splits > 65535) MB_FAIL("mb_attention_decode: %d splits", splits);
  if (((uintptr_t)kpool & 15) || ((uintptr_t)vpool & 15))
    MB_FAIL("mb_attention_decode: the cache pools are not 16-byte aligned");
  if (((uintptr_t)q & 15) || (q_stride & 7))
    MB_FAIL("mb_attention_decode: q is not 16-byte aligned (stride %d)", q_stride);
  if (T > 65535) MB_FAIL("mb_attention_decode: %d tokens are too many for one launch", T);
  return 0;
}

// in_clusters: the splits of a (token, group) form a cluster and are merged through their
// shared memory (no scratch, no second kernel); else through part_o / part_ml
static int decode_launch(const void* q, int q_stride, void* out, int out_stride,
                         const void* kpool, const void* vpool, const int* page_table,
                         int max_pages, int ring_pages, const int* tok_slot, const int* tok_pos,
                         int T, int nh, int nkv, int hd, int window, float scale, int splits,
                         float* part_o, float* part_ml, int in_clusters, int* error,
                         cudaStream_t s) {
  const int G = nh / nkv, subs = (G + 15) / 16;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(splits, nkv * subs, T), mgrid(T, nh);
#define GO(HD_)                                                                                \
  {                                                                                            \
    constexpr int smem = DEC_STAGES * 2 * MB_PAGE * HD_ * 2 + 64;                              \
    static bool configured = false;                                                            \
    if (!configured) {                                                                         \
      cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD_>,                            \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
      if (e != cudaSuccess) MB_FAIL("mb_attention_decode: %s", cudaGetErrorString(e));         \
      configured = true;                                                                       \
    }                                                                                          \
    if (in_clusters && splits > 1) {                                                           \
      mb_launch_clusters(attn_decode_kernel<HD_>, grid, dim3((DEC_WARPS + 1) * 32), smem, s,   \
                         splits, (const bf16*)q, q_stride, (const bf16*)kpool,                 \
                         (const bf16*)vpool, page_table, max_pages, ring_pages, tok_slot,      \
                         tok_pos, nh, nkv, window, scale_log2, part_o, part_ml, (bf16*)out,    \
                         out_stride, 1, error);                                                \
    } else {                                                                                   \
      mb_launch(attn_decode_kernel<HD_>, grid, dim3((DEC_WARPS + 1) * 32), smem, s,            \
                (const bf16*)q, q_stride, (const bf16*)kpool, (const bf16*)vpool, page_table,  \
                max_pages, ring_pages, tok_slot, tok_pos, nh, nkv, window, scale_log2, part_o, \
                part_ml, (bf16*)out, out_stride, in_clusters, error);                          \
      if (!in_clusters)                                                                        \
        mb_launch(attn_merge_kernel<HD_>, mgrid, dim3(HD_), 0, s, (const float*)part_o,        \
                  (const float*)part_ml, splits, (bf16*)out, out_stride, nh);                  \
    }                                                                                          \
  }
  if (hd == 64) GO(64) else GO(128)
#undef GO
  MB_CHECK_LAUNCH("mb_attention_decode");
}

// out[t, h, :] for every token t (each with its own sequence and position: a decode step, or
// any few tokens). `splits` CTAs share a sequence's pages (CTA s takes the pages s, s + splits,
// ...); the caller chooses it from the batch and the SM count, not from the lengths of the
// moment, so that a captured launch stays valid. The splits leave their partial results in
// `scratch` (float32, at least mb_attention_decode_scratch(...) values; its contents are not
// kept between calls) and a second kernel adds them up. `error`: a device word that receives
// 4 or 5 if a wait of the kernel's copy pipeline ran out.
MB_EXPORT int mb_attention_decode(const void* q, int q_stride, void* out, int out_stride,
                                  const void* kpool, const void* vpool, const int* page_table,
                                  int max_pages, int ring_pages, const int* tok_slot,
                                  const int* tok_pos, int T, int nh, int nkv,
                                  int hd, int window, float scale, int splits, float* scratch,
                                  long long scratch_floats, int* error, void* stream) {
  if (T <= 0) return 0;
  if (decode_checks(q, q_stride, kpool, vpool, T, nh, nkv, hd, splits)) return -1;
  const long long need = mb_attention_decode_scratch(T, nh, hd, splits);
  if (scratch == nullptr || scratch_floats < need)
    MB_FAIL("mb_attention_decode: %lld floats of scratch, %lld needed", scratch_floats, need);
  return decode_launch(q, q_stride, out, out_stride, kpool, vpool, page_table, max_pages,
                       ring_pages, tok_slot, tok_pos, T, nh, nkv, hd, window, scale, splits,
                       scratch, scratch + (size_t)T * nh * splits * hd, 0, error,
                       (cudaStream_t)stream);
}

// The same with the splits of a (token, group of heads) as the CTAs of one thread-block
// cluster: they add their partial results up through each other's shared memory, so there is
// no scratch and no second kernel. At most MB_DECODE_CLUSTER_SPLITS splits (the portable
// cluster size); one split writes its result directly.
#define MB_DECODE_CLUSTER_SPLITS 8
MB_EXPORT int mb_attention_decode_clusters(const void* q, int q_stride, void* out,
                                           int out_stride, const void* kpool, const void* vpool,
                                           const int* page_table, int max_pages, int ring_pages,
                                           const int* tok_slot, const int* tok_pos, int T,
                                           int nh, int nkv, int hd, int window, float scale,
                                           int splits, int* error, void* stream) {
  if (T <= 0) return 0;
  if (decode_checks(q, q_stride, kpool, vpool, T, nh, nkv, hd, splits)) return -1;
  if (splits > MB_DECODE_CLUSTER_SPLITS)
    MB_FAIL("mb_attention_decode_clusters: %d splits (a cluster holds at most %d)", splits,
            MB_DECODE_CLUSTER_SPLITS);
  if (((uintptr_t)out & 1)) MB_FAIL("mb_attention_decode_clusters: out is not aligned");
  return decode_launch(q, q_stride, out, out_stride, kpool, vpool, page_table, max_pages,
                       ring_pages, tok_slot, tok_pos, T, nh, nkv, hd, window, scale, splits,
                       nullptr, nullptr, 1, error, (cudaStream_t)stream);
}

// ------------------------------------------------------------------ prefill
// Causal attention of the new tokens of every sequence over the cache (which already holds
// their own keys and values). A CTA takes 64 consecutive new tokens of one sequence and one
// query head; each of its four warps owns 16 of them as the rows of the MMA and walks the pages
// from the first key its rows may see to the last, with an online softmax per row. The four
// warps read the same pages, so all but the first read hit the L1 cache.
// the same pieces as qk_page / pv_page with the page's tiles in shared memory
template <int HD, int KP>
__device__ __forceinline__ void qk_page_smem(const uint4* qa, const uint4* qb, uint32_t ks, int r,
                                             int c, float sc[8][4]) {
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    sc[u][0] = sc[u][1] = sc[u][2] = sc[u][3] = 0.f;
    const uint32_t krow = ks + (uint32_t)(u * 8 + r) * KP + c * 16;
#pragma unroll
    for (int ch = 0; ch < HD / 32; ++ch) {
      const uint4 kb = lds16(krow + ch * 64);
      mma_bf16(sc[u], qa[ch].x, qb[ch].x, qa[ch].y, qb[ch].y, kb.x, kb.y);
      mma_bf16(sc[u], qa[ch].z, qb[ch].z, qa[ch].w, qb[ch].w, kb.z, kb.w);
    }
  }
}

template <int HD, int VP>
__device__ __forceinline__ void pv_page_smem(const float sc[8][4], uint32_t vs, int r, int c,
                                             float o[HD / 64][8][4]) {
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    const uint32_t a0 = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
    const uint32_t a1 = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
    const uint32_t a2 = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
    const uint32_t a3 = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
    const uint32_t vrow = vs + (uint32_t)(kk * 16 + 2 * c) * VP + r * 16;
#pragma unroll
    for (int db = 0; db < HD / 64; ++db) {
      const uint4 va = lds16(vrow + db * 128);
      const uint4 vb = lds16(vrow + VP + db * 128);
      const uint4 vc = lds16(vrow + 8 * VP + db * 128);
      const uint4 vd = lds16(vrow + 9 * VP + db * 128);
      const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
      const uint32_t wc[4] = {vc.x, vc.y, vc.z, vc.w}, wd[4] = {vd.x, vd.y, vd.z, vd.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int w = j >> 1;
        const uint32_t b0 = (j & 1) ? pack_hi(wa[w], wb[w]) : pack_lo(wa[w], wb[w]);
        const uint32_t b1 = (j & 1) ? pack_hi(wc[w], wd[w]) : pack_lo(wc[w], wd[w]);
        mma_bf16(o[db][j], a0, a1, a2, a3, b0, b1);
      }
    }
  }
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

#define PRE_STAGES 3

// A CTA takes 64 consecutive new tokens of one sequence and one query head; each of its four
// warps owns 16 tokens as the rows of the MMA and keeps an online softmax per row. The pages
// that any of the CTA's tokens may see are brought to shared memory by all threads with 16-byte
// asynchronous copies, two pages ahead of the page in work. The rows of a tile are padded in
// shared memory (keys to a pitch of 2 HD + 64 bytes, values to 2 HD + 16), which makes every
// fragment read of qk_page_smem / pv_page_smem free of bank conflicts.
template <int HD>
__global__ void __launch_bounds__(DEC_WARPS * 32, 2)
attn_prefill_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out,
                    int out_stride, const bf16* __restrict__ kpool,
                    const bf16* __restrict__ vpool, const int* __restrict__ page_table,
                    int max_pages, int ring_pages, const int* __restrict__ seq_start,
                    const int* __restrict__ seq_past, const int* __restrict__ seq_slot, int nh,
                    int nkv, int window, float scale_log2) {
  mb_grid_wait();
  mb_grid_launch_next();
  constexpr int CH = HD / 32, DB = HD / 64;
  constexpr int KP = HD * 2 + 64, VP = HD * 2 + 16;     // row pitches in bytes
  constexpr uint32_t STAGE = MB_PAGE * (KP + VP);
  constexpr int CHUNKS = HD / 8;                        // 16-byte chunks of a row
  extern __shared__ __align__(128) uint8_t pre_smem[];
  const uint32_t tiles = smem_u32(pre_smem);

  const int b = blockIdx.z, h = blockIdx.y;
  const int start = seq_start[b], n_new = seq_start[b + 1] - start;
  if ((int)blockIdx.x * 64 >= n_new) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, c = lane & 3;
  const int past = seq_past[b], slot = seq_slot[b];
  const int g = h / (nh / nkv);
  // the pages that the CTA's tokens see: from the first token's first key to the last token
  const int cta_first = past + blockIdx.x * 64;
  const int cta_last = past + min((int)blockIdx.x * 64 + 63, n_new - 1);
  const int cta_lo = (window > 0 && cta_first + 1 > window) ? cta_first + 1 - window : 0;
  const int page0 = cta_lo / MB_PAGE, n_pages = cta_last / MB_PAGE - page0 + 1;

  auto issue = [&](int i) {  // page i of the CTA into stage i % PRE_STAGES
    if (i < n_pages) {
      const int p = page0 + i;
      const int entry = ring_pages > 0 ? p % ring_pages : p;
      int page = MB_INDEX_OK(entry < max_pages, 1, slot, p, max_pages)
                     ? page_table[(size_t)slot * max_pages + entry] : 0;
      if (!MB_INDEX_OK(page >= 0, 2, slot, entry, page)) page = 0;
      const bf16* ksrc = kpool + ((size_t)page * nkv + g) * MB_PAGE * HD;
      const bf16* vsrc = vpool + ((size_t)page * nkv + g) * MB_PAGE * HD;
      const uint32_t kd = tiles + (i % PRE_STAGES) * STAGE, vd = kd + MB_PAGE * KP;
      for (int e = threadIdx.x; e < MB_PAGE * CHUNKS; e += DEC_WARPS * 32) {
        const int row = e / CHUNKS, ch = e % CHUNKS;
        cp_async16(kd + row * KP + ch * 16, ksrc + row * HD + ch * 8);
        cp_async16(vd + row * VP + ch * 16, vsrc + row * HD + ch * 8);
      }
    }
    cp_async_commit();
  };

  const int row0 = blockIdx.x * 64 + warp * 16;
  const bool live = row0 < n_new;  // a warp without rows still loads and synchronizes
  const int ra = row0 + r, rb = ra + 8;
  const bool has_a = ra < n_new, has_b = rb < n_new;
  const int pa = past + ra, pb = past + rb;  // positions of the two rows
  const int la = (window > 0 && pa + 1 > window) ? pa + 1 - window : 0;
  const int lb = (window > 0 && pb + 1 > window) ? pb + 1 - window : 0;
  const int first_pos = past + row0, last_pos = past + min(row0 + 15, n_new - 1);
  const int lo_w = (window > 0 && first_pos + 1 > window) ? first_pos + 1 - window : 0;

#pragma unroll
  for (int i = 0; i < PRE_STAGES - 1; ++i) issue(i);

  uint4 qa[CH], qb[CH];
  {
    const bf16* qrow = q + (size_t)(start + ra) * q_stride + (size_t)h * HD;
    load_q<HD>(has_a ? qrow : nullptr, has_b ? qrow + (size_t)8 * q_stride : nullptr, c, qa, qb);
  }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[DB][8][4];
#pragma unroll
  for (int db = 0; db < DB; ++db)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[db][j][e] = 0.f;

  for (int i = 0; i < n_pages; ++i) {
    cp_async_wait<PRE_STAGES - 2>();  // page i has landed (for this thread's copies)
    __syncthreads();                  // ... for everyone's; and page i - 1 has been read by all
    issue(i + PRE_STAGES - 1);        // into the stage that page i - 1 occupied
    const int p = page0 + i;
    // the pages before this warp's window and after its last row are not its business
    if (live && p >= lo_w / MB_PAGE && p <= last_pos / MB_PAGE) {
      const uint32_t ks = tiles + (i % PRE_STAGES) * STAGE, vs = ks + MB_PAGE * KP;
      const int key0 = p * MB_PAGE;
      float sc[8][4];
      qk_page_smem<HD, KP>(qa, qb, ks, r, c, sc);
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = key0 + u * 8 + 2 * c + e;
          sc[u][e] = (key >= la && key <= pa) ? sc[u][e] * scale_log2 : -INFINITY;
          sc[u][2 + e] = (key >= lb && key <= pb) ? sc[u][2 + e] * scale_log2 : -INFINITY;
          mx0 = fmaxf(mx0, sc[u][e]);
          mx1 = fmaxf(mx1, sc[u][2 + e]);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
      // a row may have no key in this page (and none so far): keep exp2 away from inf - inf
      const float base0 = n0 == -INFINITY ? 0.f : n0, base1 = n1 == -INFINITY ? 0.f : n1;
      const float c0 = exp2f(m0 - base0), c1 = exp2f(m1 - base1);
      m0 = n0;
      m1 = n1;
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          sc[u][e] = exp2f(sc[u][e] - base0);
          sc[u][2 + e] = exp2f(sc[u][2 + e] - base1);
          s0 += sc[u][e];
          s1 += sc[u][2 + e];
        }
      }
      l0 = l0 * c0 + s0;
      l1 = l1 * c1 + s1;
#pragma unroll
      for (int db = 0; db < DB; ++db)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[db][j][0] *= c0;
          o[db][j][1] *= c0;
          o[db][j][2] *= c1;
          o[db][j][3] *= c1;
        }
      pv_page_smem<HD, VP>(sc, vs, r, c, o);
    }
  }
  cp_async_wait<0>();
  if (!live) return;
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = 1.0f / l0, i1 = 1.0f / l1;
  // a thread holds the dims db*64 + 16c .. + 15 of its two rows
#pragma unroll
  for (int db = 0; db < DB; ++db) {
    uint32_t w[4][4];  // [row a lo, row a hi, row b lo, row b hi][4 registers of 2 bf16]
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      w[0][j >> 1] = pack_bf16(o[db][j][0] * i0, o[db][j + 1][0] * i0);
      w[1][j >> 1] = pack_bf16(o[db][j][1] * i0, o[db][j + 1][1] * i0);
      w[2][j >> 1] = pack_bf16(o[db][j][2] * i1, o[db][j + 1][2] * i1);
      w[3][j >> 1] = pack_bf16(o[db][j][3] * i1, o[db][j + 1][3] * i1);
    }
    if (has_a) {
      uint4* dst = (uint4*)(out + (size_t)(start + ra) * out_stride + (size_t)h * HD + db * 64 + 16 * c);
      dst[0] = make_uint4(w[0][0], w[0][1], w[0][2], w[0][3]);
      dst[1] = make_uint4(w[1][0], w[1][1], w[1][2], w[1][3]);
    }
    if (has_b) {
      uint4* dst = (uint4*)(out + (size_t)(start + rb) * out_stride + (size_t)h * HD + db * 64 + 16 * c);
      dst[0] = make_uint4(w[2][0], w[2][1], w[2][2], w[2][3]);
      dst[1] = make_uint4(w[3][0], w[3][1], w[3][2], w[3][3]);
    }
  }
}

// out[t, h, :] for the new tokens of B sequences (packed one after another: sequence b holds
// the rows seq_start[b] .. seq_start[b + 1]) over the cache. `max_new`: the most new tokens of
// one sequence. `error`: a device word that receives 4 or 5 if a wait of the copy pipeline ran out.
MB_EXPORT int mb_attention_prefill(const void* q, int q_stride, void* out, int out_stride,
                                   const void* kpool, const void* vpool, const int* page_table,
                                   int max_pages, int ring_pages, const int* seq_start,
                                   const int* seq_past, const int* seq_slot, int B, int max_new,
                                   int nh, int nkv, int hd, int window, float scale, int* error,
                                   void* stream) {
  if (B <= 0 || max_new <= 0) return 0;
  if (hd != 64 && hd != 128)
    MB_FAIL("mb_attention_prefill: heads of %d values are not supported (64 or 128)", hd);
  if (nkv <= 0 || nh % nkv) MB_FAIL("mb_attention_prefill: %d heads on %d KV heads", nh, nkv);
  if (((uintptr_t)q & 15) || (q_stride & 7) || ((uintptr_t)out & 15) || (out_stride & 7))
    MB_FAIL("mb_attention_prefill: q or out is not 16-byte aligned (strides %d, %d)", q_stride,
            out_stride);
  if (B > 65535 || nh > 65535) MB_FAIL("mb_attention_prefill: %d sequences, %d heads", B, nh);
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid((max_new + 63) / 64, nh, B);
  const float scale_log2 = scale * 1.4426950408889634f;
#define GO(HD_)                                                                                \
  {                                                                                            \
    constexpr int smem = PRE_STAGES * MB_PAGE * (4 * HD_ + 80);                                \
    static bool configured = false;                                                            \
    if (!configured) {                                                                         \
      cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD_>,                           \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
      if (e != cudaSuccess) MB_FAIL("mb_attention_prefill: %s", cudaGetErrorString(e));        \
      configured = true;                                                                       \
    }                                                                                          \
    mb_launch(attn_prefill_kernel<HD_>, grid, dim3(DEC_WARPS * 32), smem, s, (const bf16*)q,   \
              q_stride, (bf16*)out, out_stride, (const bf16*)kpool, (const bf16*)vpool,        \
              page_table, max_pages, ring_pages, seq_start, seq_past, seq_slot, nh, nkv,       \
              window, scale_log2);                                                             \
  }
  if (hd == 64) GO(64) else GO(128)
#undef GO
  (void)error;
  MB_CHECK_LAUNCH("mb_attention_prefill");
}

// ------------------------------------------------------------------ without an allocation
// See no_alloc.h: the same decode attention with its scratch in an array of the library's own.
#include "no_alloc.h"

// The scratch itself. In host code this name is only a handle for cudaGetSymbolAddress; it is
// not a device address and must never be given to a kernel as one.
static __device__ __align__(256) float g_static_scratch[MB_ATTENTION_DECODE_STATIC_FLOATS];

#define MB_MAX_DEVICES 64
static float* g_static_scratch_ptr[MB_MAX_DEVICES];  // device address per device, null: not looked up

MB_EXPORT int mb_attention_decode_static(const void* q, int q_stride, void* out, int out_stride,
                                         const void* kpool, const void* vpool,
                                         const int* page_table, int max_pages, int ring_pages,
                                         const int* tok_slot, const int* tok_pos,
                                         int T, int nh, int nkv, int hd,
                                         int window, float scale, int splits, int* error,
                                         void* stream) {
  if (T <= 0) return 0;
  if (nh <= 0 || hd <= 0 || splits <= 0)
    MB_FAIL("mb_attention_decode_static: %d heads of %d, %d splits", nh, hd, splits);
  const long long need = mb_attention_decode_scratch(T, nh, hd, splits);
  if (need > MB_ATTENTION_DECODE_STATIC_FLOATS)
    MB_FAIL("mb_attention_decode_static: %d tokens x %d heads x %d splits x (%d + 2) = %lld "
            "values of scratch, the built-in array holds %lld; use fewer splits or "
            "mb_attention_decode with a buffer of your own",
            T, nh, splits, hd, need, (long long)MB_ATTENTION_DECODE_STATIC_FLOATS);
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) MB_FAIL("mb_attention_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (device < 0 || device >= MB_MAX_DEVICES)
    MB_FAIL("mb_attention_decode_static: device %d (at most %d devices)", device, MB_MAX_DEVICES);
  if (g_static_scratch_ptr[device] == nullptr) {
    // once per device, with that device current: the array's address on this device
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      MB_FAIL("mb_attention_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_static_scratch_ptr[device] = p;
  }
  return mb_attention_decode(q, q_stride, out, out_stride, kpool, vpool, page_table, max_pages,
                             ring_pages, tok_slot, tok_pos, T, nh, nkv, hd, window,
                             scale, splits, g_static_scratch_ptr[device],
                             MB_ATTENTION_DECODE_STATIC_FLOATS, error, stream);
}
