// Blackwell (sm_100a) building blocks in inline PTX: mbarriers with bounded waits, TMA tile
// loads, tensor memory (TMEM) allocation, tcgen05.mma with shared-memory operand descriptors,
// tcgen05.ld for the epilogue. Every wait has an iteration limit: when it runs out the kernel
// records where in its error word and goes on to its end (the result is then wrong, but the
// kernel returns, frees its TMEM, and the host reads the word).
#pragma once
#include <cuda.h>
#include "common.cuh"

// ---------------------------------------------------------------------------- addresses
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\t"
      "elect.sync rx|px, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, px;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// The limit of every wait: each try_wait already suspends for a while in hardware, so this is
// seconds, far beyond any healthy wait, and still an end.
#ifndef MB_WAIT_LIMIT
#define MB_WAIT_LIMIT (1u << 22)
#endif

// false after `limit` tries; then *error (global) holds `code` and the caller goes on.
__device__ __forceinline__ bool mbar_wait_tries(uint32_t bar, uint32_t parity, int* error, int code,
                                                uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  if (error) atomicCAS(error, 0, code);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error, int code) {
  return mbar_wait_tries(bar, parity, error, code, MB_WAIT_LIMIT);
}

// ---------------------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// A 2-D tile at (x = innermost coordinate in elements, y = row) into shared memory; completes
// `bar` with the tile's bytes. x times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// 16 bytes to and from shared memory by its 32-bit address
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
               ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}

// ---------------------------------------------------------------------------- TMEM
// One whole warp allocates `cols` columns (a power of two, at least 32); the address lands in
// shared memory at `slot`.
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------- MMA
// Shared-memory operand descriptor of a K-major tile of rows x 64 bfloat16 (128 bytes a row)
// written by TMA with the 128-byte swizzle: 8-row groups of 1024 bytes one after another.
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4 (1: unused here)
//   bits [32,46) stride byte offset >> 4 (1024 >> 4: from one 8-row group to the next)
//   bits [46,48) version 1 (sm_100)        bits [61,64) layout 2 = SWIZZLE_128B
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor of kind::f16 with bfloat16 A and B (both K-major), float32 D:
//   bits [4,6) D format 1 = F32, [7,10) A format 1 = BF16, [10,13) B format 1 = BF16,
//   bit 15 / 16 A / B major 0 = K, bits [17,23) N >> 3, bits [24,29) M >> 4.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] · B[smem]ᵀ, issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The barrier gets one arrival when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar)
               : "memory");
}

// 16 consecutive float32 columns of this thread's TMEM lane (lane = 32 * (warp % 4) + lane id).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32"
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  // the loaded registers pass through the wait, so that no use of them can be scheduled
  // before it
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]),
                 "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]),
                 "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// ---------------------------------------------------------------------------- CTA pairs
// Two CTAs of a cluster (ranks 0 and 1) work on one MMA tile of 256 rows: each holds its 128
// rows of the first operand and half of the second one's rows in its own shared memory at the
// same offsets, and 128 lanes of the accumulator in its own tensor memory. Rank 0 issues the
// MMAs for both.
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Every thread of both CTAs arrives; returns when all have (release / acquire over the cluster).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The cluster-wide address of this CTA's shared address `addr` as it lies in CTA `rank`.
__device__ __forceinline__ uint32_t cluster_addr_of(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
               : "memory");
}
// As tma_load_2d, into this CTA's shared memory, but the barrier (a cluster-wide address) may
// lie in the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x,
                                                 int y, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(cluster_bar)
      : "memory");
}
// One warp of EACH CTA of the pair calls these (the same warp index in both).
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols)
               : "memory");
}
// D[tmem of both CTAs] (+)= A · Bᵀ over the pair: M = 256 (128 rows from each CTA), N rows of
// B of which each CTA holds half. Issued by one thread of rank 0.
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The barrier at this shared offset in every CTA of `cta_mask` gets one arrival when the pair's
// MMAs issued so far have finished.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
      " [%0], %1;"
      ::"r"(bar), "h"(cta_mask)
      : "memory");
}

// ---------------------------------------------------------------------------- host: tensor maps
typedef CUresult (*MbEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static MbEncodeTiled mb_encode_tiled() {
  static MbEncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (MbEncodeTiled)p;
  }
  return fn;
}

// A map over a row-major bfloat16 matrix [rows, cols] with `ld` elements from row to row,
// tiles of box_rows x 64 columns, 128-byte swizzle, zeros outside. Returns false with a
// message in g_mb_error if the matrix cannot be mapped (alignment).
__attribute__((unused)) static bool mb_make_map_bf16(CUtensorMap* map, const void* base, long long rows, long long cols,
                             long long ld, int box_rows, const char* what) {
  MbEncodeTiled enc = mb_encode_tiled();
  if (!enc) {
    snprintf(g_mb_error, sizeof(g_mb_error), "cuTensorMapEncodeTiled is not available");
    return false;
  }
  if (((uintptr_t)base & 15) || ((ld * 2) & 15)) {
    snprintf(g_mb_error, sizeof(g_mb_error),
             "%s: base %p with a row stride of %lld values is not 16-byte aligned", what, base, ld);
    return false;
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_mb_error, sizeof(g_mb_error), "%s: cuTensorMapEncodeTiled failed (%d) for [%lld, %lld] ld %lld box %d",
             what, (int)r, rows, cols, ld, box_rows);
    return false;
  }
  return true;
}
