// Warp-level tensor-core pieces of the attention kernels: the m16n8k16 bfloat16 MMA with float32
// accumulators, packing, and 16-byte read-only loads.
#pragma once
#include "common.cuh"

// D (4 floats) += A (4 regs of 2 bf16, 16x16 row-major) · B (2 regs, 16x8 column-major)
__device__ __forceinline__ void mma_bf16(float* d, uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint4 ldg16(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

// the two low halves / the two high halves of a and b as one register of two bf16
__device__ __forceinline__ uint32_t pack_lo(uint32_t a, uint32_t b) {
  return __byte_perm(a, b, 0x5410);
}
__device__ __forceinline__ uint32_t pack_hi(uint32_t a, uint32_t b) {
  return __byte_perm(a, b, 0x7632);
}
