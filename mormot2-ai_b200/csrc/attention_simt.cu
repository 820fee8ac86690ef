// Causal grouped-query attention over the paged cache for any head size up to 256 and any
// number of heads and groups, in float32 arithmetic on the CUDA cores, for float32 or
// bfloat16 storage. One warp per (token, query head) walks the keys of the token's own
// sequence in tiles of 32 with an online softmax (a lane has one key of the tile for q·k and
// four neighbouring values of every key's row for p·v; 16-byte loads where the head size and
// the strides are multiples of four, single values else). It serves prefill and decode of the
// true 32-bit path and is the fallback of the bfloat16 path.
//
// The formula is the reference's (paths within the reference project):
// src/infer/mormot.ai.infer.backend.cpu.pas:1296-1353 — head h reads KV head
// h div (heads div kv_heads); keys max(0, pos+1-window)..pos; s = q·k·scale; p = exp(s - max);
// y = (sum p v) / (sum p) — and the tiled form of tools/cuda/ops.cu:352-540.
#include "common.cuh"

MB_DEFINE_LAST_ERROR

#define ATT_WARPS 4
#define ATT_MAX_D 8  // head sizes up to 32 * 8

template <typename T, bool VEC>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                      const T* __restrict__ kpool, const T* __restrict__ vpool,
                      const int* __restrict__ page_table, int max_pages, int ring_pages,
                      const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                      const int* __restrict__ seq_slot, int nh, int nkv, int hd, int window,
                      float scale) {
  extern __shared__ __align__(16) float qs[];  // ATT_WARPS x hd
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * ATT_WARPS + warp;
  if (h >= nh) return;
  const int g = h / (nh / nkv);
  const int pos = tok_pos[t];
  const int slot = seq_slot[tok_seq[t]];
  float* qv = qs + warp * hd;
  const T* qp = q + (size_t)t * q_stride + (size_t)h * hd;
  for (int i = lane; i < hd; i += 32) qv[i] = to_f32<T>(qp[i]);
  __syncwarp();

  int lo = 0;
  if (window > 0 && pos + 1 > window) lo = pos + 1 - window;
  float m = -INFINITY, l = 0.f;
  // VEC: values 4 * lane .. + 3 of every 128; else values lane, lane + 32, ...
  float acc[ATT_MAX_D];
#pragma unroll
  for (int d = 0; d < ATT_MAX_D; ++d) acc[d] = 0.f;

  for (int k0 = lo; k0 <= pos; k0 += 32) {
    const int kp = k0 + lane;
    const bool valid = kp <= pos;
    size_t row = 0;
    float s = -INFINITY;
    if (valid) {
      row = kv_row(page_table, max_pages, ring_pages, slot, kp, nkv, g);
      const T* kr = kpool + row * hd;
      float dot = 0.f;
      if (VEC) {
        for (int i = 0; i < hd; i += 4) {
          const float4 kk = load4<T>(kr + i), qq = *(const float4*)(qv + i);
          dot = fmaf(qq.x, kk.x, fmaf(qq.y, kk.y, fmaf(qq.z, kk.z, fmaf(qq.w, kk.w, dot))));
        }
      } else {
        for (int i = 0; i < hd; ++i) dot = fmaf(qv[i], to_f32<T>(kr[i]), dot);
      }
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);  // 0 on the first tile (m = -inf)
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int d = 0; d < ATT_MAX_D; ++d) acc[d] *= corr;
    m = m_new;
    const int n = min(32, pos - k0 + 1);
    for (int j = 0; j < n; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const unsigned lo32 = __shfl_sync(0xffffffffu, (unsigned)(row & 0xffffffffu), j);
      const unsigned hi32 = __shfl_sync(0xffffffffu, (unsigned)(row >> 32), j);
      const T* vr = vpool + (((size_t)hi32 << 32) | lo32) * hd;
      if (VEC) {
#pragma unroll
        for (int d = 0; d < ATT_MAX_D / 4; ++d) {
          const int i = 4 * lane + 128 * d;
          if (i < hd) {
            const float4 vv = load4<T>(vr + i);
            acc[4 * d] = fmaf(pj, vv.x, acc[4 * d]);
            acc[4 * d + 1] = fmaf(pj, vv.y, acc[4 * d + 1]);
            acc[4 * d + 2] = fmaf(pj, vv.z, acc[4 * d + 2]);
            acc[4 * d + 3] = fmaf(pj, vv.w, acc[4 * d + 3]);
          }
        }
      } else {
#pragma unroll
        for (int d = 0; d < ATT_MAX_D; ++d) {
          const int i = lane + 32 * d;
          if (i < hd) acc[d] = fmaf(pj, to_f32<T>(vr[i]), acc[d]);
        }
      }
    }
  }
  const float inv = 1.0f / l;
  T* op = out + (size_t)t * out_stride + (size_t)h * hd;
  if (VEC) {
#pragma unroll
    for (int d = 0; d < ATT_MAX_D / 4; ++d) {
      const int i = 4 * lane + 128 * d;
      if (i < hd)
        store4<T>(op + i, make_float4(acc[4 * d] * inv, acc[4 * d + 1] * inv, acc[4 * d + 2] * inv,
                                      acc[4 * d + 3] * inv));
    }
  } else {
#pragma unroll
    for (int d = 0; d < ATT_MAX_D; ++d) {
      const int i = lane + 32 * d;
      if (i < hd) op[i] = from_f32<T>(acc[d] * inv);
    }
  }
}

// The same with the keys and values of a tile staged in shared memory, for blocks whose four
// heads read the same KV head (groups of four query heads or a multiple): the block loads the
// tile's 32 keys and values once, with whole rows per warp instruction, and every warp reads
// its scores' operands from there (a lane's own key row by 16-byte pieces, row pitch hd + 4
// floats: no bank conflicts; a value row across the lanes).
template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_shared_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out,
                        int out_stride, const T* __restrict__ kpool, const T* __restrict__ vpool,
                        const int* __restrict__ page_table, int max_pages, int ring_pages,
                        const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                        const int* __restrict__ seq_slot, int nh, int nkv, int hd, int window,
                        float scale) {
  extern __shared__ __align__(16) float sm[];
  const int pitch = hd + 4, pieces = hd / 4;
  float* qs = sm;                                  // [ATT_WARPS][hd]
  float* ks = qs + ATT_WARPS * hd;                 // [32][pitch]
  float* vs = ks + 32 * pitch;                     // [32][pitch]
  size_t* rows = (size_t*)(vs + 32 * pitch);       // [32] pool rows of the tile's keys
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * ATT_WARPS + warp;     // nh is a multiple of ATT_WARPS here
  const int g = (blockIdx.y * ATT_WARPS) / (nh / nkv);
  const int pos = tok_pos[t];
  const int slot = seq_slot[tok_seq[t]];
  float* qv = qs + warp * hd;
  const T* qp = q + (size_t)t * q_stride + (size_t)h * hd;
  for (int i = lane; i < hd; i += 32) qv[i] = to_f32<T>(qp[i]);

  int lo = 0;
  if (window > 0 && pos + 1 > window) lo = pos + 1 - window;
  float m = -INFINITY, l = 0.f;
  float acc[ATT_MAX_D];
#pragma unroll
  for (int d = 0; d < ATT_MAX_D; ++d) acc[d] = 0.f;

  for (int k0 = lo; k0 <= pos; k0 += 32) {
    const int n = min(32, pos - k0 + 1);
    __syncthreads();                               // the tile before has been read
    if (threadIdx.x < n)
      rows[threadIdx.x] = kv_row(page_table, max_pages, ring_pages, slot, k0 + threadIdx.x, nkv, g);
    __syncthreads();
    for (int e = threadIdx.x; e < n * pieces; e += ATT_WARPS * 32) {
      const int key = e / pieces, piece = e - key * pieces;
      const size_t at = rows[key] * hd + 4 * piece;
      *(float4*)(ks + key * pitch + 4 * piece) = load4<T>(kpool + at);
      *(float4*)(vs + key * pitch + 4 * piece) = load4<T>(vpool + at);
    }
    __syncthreads();
    const bool valid = lane < n;
    float s = -INFINITY;
    if (valid) {
      const float* kr = ks + lane * pitch;
      float dot = 0.f;
      for (int i = 0; i < hd; i += 4) {
        const float4 kk = *(const float4*)(kr + i), qq = *(const float4*)(qv + i);
        dot = fmaf(qq.x, kk.x, fmaf(qq.y, kk.y, fmaf(qq.z, kk.z, fmaf(qq.w, kk.w, dot))));
      }
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int d = 0; d < ATT_MAX_D; ++d) acc[d] *= corr;
    m = m_new;
    for (int j = 0; j < n; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
      for (int d = 0; d < ATT_MAX_D / 4; ++d) {
        const int i = 4 * lane + 128 * d;
        if (i < hd) {
          const float4 vv = *(const float4*)(vs + j * pitch + i);
          acc[4 * d] = fmaf(pj, vv.x, acc[4 * d]);
          acc[4 * d + 1] = fmaf(pj, vv.y, acc[4 * d + 1]);
          acc[4 * d + 2] = fmaf(pj, vv.z, acc[4 * d + 2]);
          acc[4 * d + 3] = fmaf(pj, vv.w, acc[4 * d + 3]);
        }
      }
    }
  }
  const float inv = 1.0f / l;
  T* op = out + (size_t)t * out_stride + (size_t)h * hd;
#pragma unroll
  for (int d = 0; d < ATT_MAX_D / 4; ++d) {
    const int i = 4 * lane + 128 * d;
    if (i < hd)
      store4<T>(op + i, make_float4(acc[4 * d] * inv, acc[4 * d + 1] * inv, acc[4 * d + 2] * inv,
                                    acc[4 * d + 3] * inv));
  }
}

// out[t, h, :] for every token t of the step and head h. q: head h of token t at
// q + t * q_stride + h * hd (the q part of the fused qkv rows); out likewise with out_stride.
MB_EXPORT int mb_attention_simt(const void* q, int q_stride, void* out, int out_stride,
                                const void* kpool, const void* vpool, int dtype,
                                const int* page_table, int max_pages, int ring_pages,
                                const int* tok_seq, const int* tok_pos, const int* seq_slot,
                                int T, int nh, int nkv, int hd, int window, float scale,
                                void* stream) {
  if (T <= 0) return 0;
  if (hd <= 0 || hd > 32 * ATT_MAX_D)
    MB_FAIL("mb_attention_simt: heads of %d values are not supported (at most %d)", hd,
            32 * ATT_MAX_D);
  if (nkv <= 0 || nh % nkv) MB_FAIL("mb_attention_simt: %d heads on %d KV heads", nh, nkv);
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(T, (nh + ATT_WARPS - 1) / ATT_WARPS);
  const size_t smem = (size_t)ATT_WARPS * hd * sizeof(float);
  // four values with one load: the size of four values divides every row's address
  const int four = dtype == MB_F32 ? 15 : 7;
  const bool vec = hd % 4 == 0 && q_stride % 4 == 0 && out_stride % 4 == 0 &&
                   (((uintptr_t)q | (uintptr_t)out | (uintptr_t)kpool | (uintptr_t)vpool) & four) == 0;
  // the four heads of every block share a KV head: the tile goes through shared memory
  if (vec && (nh / nkv) % ATT_WARPS == 0) {
    const size_t shared = ((size_t)ATT_WARPS * hd + 2 * 32 * (hd + 4)) * sizeof(float) +
                          32 * sizeof(size_t);
#define GOS(T_)                                                                               \
  {                                                                                           \
    static bool configured = false;                                                           \
    if (!configured) {                                                                        \
      cudaFuncSetAttribute(attention_shared_kernel<T_>,                                       \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);          \
      configured = true;                                                                      \
    }                                                                                         \
    attention_shared_kernel<T_><<<grid, ATT_WARPS * 32, shared, s>>>(                         \
        (const T_*)q, q_stride, (T_*)out, out_stride, (const T_*)kpool, (const T_*)vpool,     \
        page_table, max_pages, ring_pages, tok_seq, tok_pos, seq_slot, nh, nkv, hd, window,   \
        scale);                                                                               \
  }
    if (dtype == MB_F32) GOS(float) else GOS(__nv_bfloat16)
#undef GOS
    MB_CHECK_LAUNCH("mb_attention_simt");
  }
#define GO(T_, V_)                                                                            \
  attention_simt_kernel<T_, V_><<<grid, ATT_WARPS * 32, smem, s>>>(                           \
      (const T_*)q, q_stride, (T_*)out, out_stride, (const T_*)kpool, (const T_*)vpool,       \
      page_table, max_pages, ring_pages, tok_seq, tok_pos, seq_slot, nh, nkv, hd, window, scale)
  if (dtype == MB_F32) {
    if (vec) GO(float, true); else GO(float, false);
  } else {
    if (vec) GO(__nv_bfloat16, true); else GO(__nv_bfloat16, false);
  }
#undef GO
  MB_CHECK_LAUNCH("mb_attention_simt");
}
