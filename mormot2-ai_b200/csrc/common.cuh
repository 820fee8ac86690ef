// Shared by every kernel file of the library: element types, the error word, reductions.
//
// All entry points are extern "C", take device pointers and a stream, launch asynchronously
// and return 0, or a negative code after storing a message that mb_last_error() returns.
// Nothing here allocates device memory: the caller owns every buffer.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

enum MbDtype { MB_F32 = 0, MB_BF16 = 1 };

// Cache pages hold this many positions (cache/pages.py uses the same number).
#define MB_PAGE 64

static thread_local char g_mb_error[512];

#define MB_FAIL(...)                                             \
  do {                                                           \
    snprintf(g_mb_error, sizeof(g_mb_error), __VA_ARGS__);       \
    return -1;                                                   \
  } while (0)

#define MB_CHECK_LAUNCH(name)                                                   \
  do {                                                                          \
    cudaError_t e_ = cudaGetLastError();                                        \
    if (e_ != cudaSuccess) MB_FAIL("%s: %s", name, cudaGetErrorString(e_));     \
    return 0;                                                                   \
  } while (0)

#define MB_EXPORT extern "C" __attribute__((visibility("default")))

// Programmatic dependent launch: a kernel launched through mb_launch may be scheduled while the
// kernel before it in the stream is still draining; it must call mb_grid_wait() before it
// touches global memory (the wait returns when the kernels before have completed and their
// writes are visible). Every kernel that is launched this way waits at its very top, on every
// path, so that completion stays transitive along a chain of kernels. mb_grid_launch_next()
// lets the next kernel's CTAs be placed as soon as all CTAs of this one have started.
__device__ __forceinline__ void mb_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void mb_grid_launch_next() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
static cudaError_t mb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same with the CTAs of the grid's x direction in clusters of `cluster_x` (which divides it).
template <typename... KArgs, typename... Args>
static cudaError_t mb_launch_clusters(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Debug builds (-DMB_DEBUG_BOUNDS, what MORMOT_B200_DEBUG=1 asks of the build): every lookup in
// a page table checks its index and the page it finds before it uses them. The first
// violation of a library is kept in a device word with three numbers that describe it, the
// access goes to row 0 of the pool instead (a place that exists), and the host reads the word
// with mb_debug_fault() (Runtime.check does). This stands in for a memory checker where none
// can be run. Codes: 1 a position outside the slot's table row, 2 a negative page.
#ifdef MB_DEBUG_BOUNDS
__device__ int g_mb_debug_fault[4];
__device__ __forceinline__ bool mb_index_ok(bool ok, int code, int a, int b, int c) {
  if (!ok && atomicCAS(&g_mb_debug_fault[0], 0, code) == 0) {
    g_mb_debug_fault[1] = a;
    g_mb_debug_fault[2] = b;
    g_mb_debug_fault[3] = c;
  }
  return ok;
}
#define MB_INDEX_OK(cond, code, a, b, c) mb_index_ok((cond), (code), (a), (b), (c))
#define MB_DEFINE_DEBUG_FAULT                                                          \
  MB_EXPORT int mb_debug_fault(int* out4) {                                            \
    const int zero[4] = {0, 0, 0, 0};                                                  \
    if (cudaMemcpyFromSymbol(out4, g_mb_debug_fault, sizeof(zero)) != cudaSuccess) return -2; \
    if (out4[0] && cudaMemcpyToSymbol(g_mb_debug_fault, zero, sizeof(zero)) != cudaSuccess)   \
      return -2;                                                                       \
    return 1;                                                                          \
  }
#else
#define MB_INDEX_OK(cond, code, a, b, c) true
#define MB_DEFINE_DEBUG_FAULT \
  MB_EXPORT int mb_debug_fault(int*) { return 0; } /* 0: not a debug build */
#endif

// -DMB_TRACE (a probe's build): every CTA of the kernels that carry MB_TRACE_BEGIN / _END leaves
// its start and end (global nanosecond timer) and the kernel's id in a buffer of the library.
#ifdef MB_TRACE
#define MB_TRACE_CAP (1 << 17)
__device__ unsigned long long g_mb_trace[MB_TRACE_CAP][2];
__device__ unsigned int g_mb_trace_n;
__device__ __forceinline__ unsigned long long mb_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define MB_TRACE_BEGIN() const unsigned long long mb_t0_ = mb_now()
#define MB_TRACE_END(id_)                                                         \
  do {                                                                            \
    if (threadIdx.x == 0) {                                                       \
      const unsigned long long t1_ = mb_now(); /* before the atomic's round trip */ \
      const unsigned int i_ = atomicAdd(&g_mb_trace_n, 1u);                       \
      if (i_ < MB_TRACE_CAP) {                                                    \
        g_mb_trace[i_][0] = (mb_t0_ & 0x00ffffffffffffffull) | ((unsigned long long)(id_) << 56); \
        g_mb_trace[i_][1] = t1_;                                                  \
      }                                                                           \
    }                                                                             \
  } while (0)
#define MB_DEFINE_TRACE                                                           \
  MB_EXPORT int mb_trace_read(unsigned long long* out, int cap) {                 \
    unsigned int n = 0;                                                           \
    cudaDeviceSynchronize();                                                      \
    cudaMemcpyFromSymbol(&n, g_mb_trace_n, 4);                                    \
    if ((int)n > cap) n = cap;                                                    \
    if (n > MB_TRACE_CAP) n = MB_TRACE_CAP;                                       \
    cudaMemcpyFromSymbol(out, g_mb_trace, (size_t)n * 16);                        \
    const unsigned int zero = 0;                                                  \
    cudaMemcpyToSymbol(g_mb_trace_n, &zero, 4);                                   \
    return (int)n;                                                                \
  }
#else
#define MB_TRACE_BEGIN() do {} while (0)
#define MB_TRACE_END(id_) do {} while (0)
#define MB_DEFINE_TRACE
#endif

#define MB_DEFINE_LAST_ERROR                                       \
  MB_DEFINE_TRACE                                                  \
  MB_EXPORT const char* mb_last_error() { return g_mb_error; }    \
  MB_DEFINE_DEBUG_FAULT

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Four consecutive values as float32 (p aligned to the four values' size) and back
template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) {
  return *(const float4*)p;
}
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *(const uint2*)p;
  const float2 lo = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x);
  const float2 hi = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *(float4*)p = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *(const unsigned int*)&lo;
  raw.y = *(const unsigned int*)&hi;
  *(uint2*)p = raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = (lane < (int)((blockDim.x + 31) >> 5)) ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// Where position `pos` of the sequence in `slot` lies in a pool [pages][kv_heads][MB_PAGE][hd]:
// the index of its row for KV head `g`. ring_pages > 0: the line keeps a ring of that many pages.
__device__ __forceinline__ size_t kv_row(const int* __restrict__ page_table, int max_pages,
                                         int ring_pages, int slot, int pos, int kv_heads, int g) {
  int lp = pos / MB_PAGE;
  if (ring_pages > 0) lp %= ring_pages;
  if (!MB_INDEX_OK(pos >= 0 && slot >= 0 && lp < max_pages, 1, slot, pos, max_pages)) return 0;
  const int page = page_table[(size_t)slot * max_pages + lp];
  if (!MB_INDEX_OK(page >= 0, 2, slot, lp, page)) return 0;
  return ((size_t)page * kv_heads + g) * MB_PAGE + (pos % MB_PAGE);
}
