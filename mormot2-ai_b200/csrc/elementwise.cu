// Bandwidth-bound kernels around the matrix products: embedding rows, RMSNorm (plain, and
// fused with the sum of split partial products into the residual), SwiGLU, and the fused
// per-head norm + rotary position + cache write. One file for float32 and bfloat16
// activations; sums, norms, angles and the residual are float32 in both.
//
// Formulas as the reference computes them (paths within the reference project):
//   RMSNorm   src/infer/mormot.ai.infer.backend.cpu.pas:1769-1795, tools/cuda/ops.cu:116-150
//   SwiGLU    src/infer/mormot.ai.infer.backend.cpu.pas:1827-1833, tools/cuda/ops.cu:155-178
//   q/k norm + RoPE + cache store   tools/cuda/ops.cu:211-314,
//             angles src/infer/mormot.ai.infer.decoder.pas:2539-2561
#include "common.cuh"

MB_DEFINE_LAST_ERROR

// ------------------------------------------------------------------ embedding
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ x, int H, int V) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= V) id = 0;  // the host refuses such ids before the step
  const TW* row = table + (size_t)id * H;
  float* out = x + (size_t)t * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) out[c] = to_f32<TW>(row[c]);
}

MB_EXPORT int mb_embed(const void* table, int table_dtype, const int* ids, float* x, int T,
                       int H, int V, void* stream) {
  if (T <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == MB_F32)
    mb_launch(embed_kernel<float>, dim3(T), dim3(threads), 0, s, (const float*)table, ids, x, H, V);
  else
    mb_launch(embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, s, (const __nv_bfloat16*)table, ids, x, H, V);
  MB_CHECK_LAUNCH("mb_embed");
}

// ------------------------------------------------------------------ RMSNorm
// One block per output row. Before the norm, `parts` partial products [parts][T][H] (float32,
// the split-K results of the product before) are added to the residual row in place, in the
// order of the splits: x += p0 + p1 + ...; then y = w * (x * inv).
template <typename TW, typename TO>
__global__ void rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ partial,
                               int parts, size_t part_stride, const TW* __restrict__ w,
                               float eps, TO* __restrict__ y, const int* __restrict__ rows,
                               int H) {
  mb_grid_wait();
  mb_grid_launch_next();
  __shared__ float red[33];
  extern __shared__ float rowbuf[];  // H floats when parts > 0
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * H;
  float sum = 0.f;
  if (parts > 0) {
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      float v = xr[c];
      for (int p = 0; p < parts; ++p) v += partial[p * part_stride + (size_t)src * H + c];
      xr[c] = v;
      rowbuf[c] = v;
      sum = fmaf(v, v, sum);
    }
  } else {
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      const float v = xr[c];
      sum = fmaf(v, v, sum);
    }
  }
  sum = block_sum(sum, red);
  if (y == nullptr) return;
  const float inv = 1.0f / sqrtf(sum / (float)H + eps);
  TO* yr = y + (size_t)r * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = parts > 0 ? rowbuf[c] : xr[c];
    const float n = v * inv;  // rounded to float32 before the weight, as the reference does
    yr[c] = from_f32<TO>(to_f32<TW>(w[c]) * n);
  }
}


// The same for rows of 4 * RMS_THREADS * VEC values at most (a multiple of 4): the row is read
// once with 16-byte loads, kept in registers, and written with 8- or 16-byte stores.
template <typename TW, typename TO, int VEC, int RMS_THREADS>
__global__ void __launch_bounds__(RMS_THREADS)
rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ partial, int parts,
                   size_t part_stride, const TW* __restrict__ w, float eps, TO* __restrict__ y,
                   const int* __restrict__ rows, int H) {
  mb_grid_wait();
  mb_grid_launch_next();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * H;
  float4 v[VEC];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = (i * RMS_THREADS + threadIdx.x) * 4;
    v[i] = c < H ? *(const float4*)(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (parts > 0) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RMS_THREADS + threadIdx.x) * 4;
      if (c >= H) continue;
      const float* pp = partial + (size_t)src * H + c;
      int p = 0;
      for (; p + 4 <= parts; p += 4) {  // four loads in flight, added in split order
        const float4 a0 = __ldg((const float4*)(pp + (size_t)p * part_stride));
        const float4 a1 = __ldg((const float4*)(pp + (size_t)(p + 1) * part_stride));
        const float4 a2 = __ldg((const float4*)(pp + (size_t)(p + 2) * part_stride));
        const float4 a3 = __ldg((const float4*)(pp + (size_t)(p + 3) * part_stride));
        v[i].x = (((v[i].x + a0.x) + a1.x) + a2.x) + a3.x;
        v[i].y = (((v[i].y + a0.y) + a1.y) + a2.y) + a3.y;
        v[i].z = (((v[i].z + a0.z) + a1.z) + a2.z) + a3.z;
        v[i].w = (((v[i].w + a0.w) + a1.w) + a2.w) + a3.w;
      }
      for (; p < parts; ++p) {
        const float4 a = __ldg((const float4*)(pp + (size_t)p * part_stride));
        v[i].x += a.x; v[i].y += a.y; v[i].z += a.z; v[i].w += a.w;
      }
      *(float4*)(xr + c) = v[i];
    }
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i)
    sum = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, sum))));
  sum = block_sum(sum, red);
  if (y == nullptr) return;
  const float inv = 1.0f / sqrtf(sum / (float)H + eps);
  TO* yr = y + (size_t)r * H;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = (i * RMS_THREADS + threadIdx.x) * 4;
    if (c >= H) continue;
    float o[4];
    o[0] = to_f32<TW>(w[c]) * (v[i].x * inv);
    o[1] = to_f32<TW>(w[c + 1]) * (v[i].y * inv);
    o[2] = to_f32<TW>(w[c + 2]) * (v[i].z * inv);
    o[3] = to_f32<TW>(w[c + 3]) * (v[i].w * inv);
    if (sizeof(TO) == 4) {
      *(float4*)((float*)yr + c) = make_float4(o[0], o[1], o[2], o[3]);
    } else {
      __nv_bfloat162 h[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
      *(uint2*)((__nv_bfloat16*)yr + c) = *(uint2*)h;
    }
  }
}

template <typename TW, typename TO>
static int rmsnorm_launch(float* x, const float* partial, int parts, size_t part_stride,
                          const void* w, float eps, void* y, const int* rows, int R, int H,
                          cudaStream_t s) {
  const bool aligned = ((uintptr_t)x & 15) == 0 && ((uintptr_t)partial & 15) == 0 &&
                       (part_stride & 3) == 0 && ((uintptr_t)y & 15) == 0;
  if (H % 4 == 0 && H <= 4 * 256 * 16 && aligned) {
    // few rows (a decode step): 1024 threads a row, so that a thread waits for few loads; many
    // rows: 256 threads a row and more rows per SM
#define RMS_GO(V_, T_)                                                                      \
  mb_launch(rmsnorm_vec_kernel<TW, TO, V_, T_>, dim3(R), dim3(T_), 0, s, x, partial, parts, part_stride,         \
                                                      (const TW*)w, eps, (TO*)y, rows, H)
    if (R <= 256 && H > 1024) {
      const int vec = (H + 4 * 1024 - 1) / (4 * 1024);
      if (vec <= 1) RMS_GO(1, 1024);
      else if (vec <= 2) RMS_GO(2, 1024);
      else RMS_GO(4, 1024);
    } else {
      const int vec = (H + 4 * 256 - 1) / (4 * 256);
      if (vec <= 1) RMS_GO(1, 256);
      else if (vec <= 2) RMS_GO(2, 256);
      else if (vec <= 4) RMS_GO(4, 256);
      else if (vec <= 8) RMS_GO(8, 256);
      else RMS_GO(16, 256);
    }
#undef RMS_GO
    MB_CHECK_LAUNCH("mb_rmsnorm");
  }
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  const size_t smem = parts > 0 ? (size_t)H * sizeof(float) : 0;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(rmsnorm_kernel<TW, TO>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) MB_FAIL("mb_rmsnorm: a row of %d values: %s", H, cudaGetErrorString(e));
  }
  mb_launch(rmsnorm_kernel<TW, TO>, dim3(R), dim3(threads), smem, s, x, partial, parts, part_stride,
                                                  (const TW*)w, eps, (TO*)y, rows, H);
  MB_CHECK_LAUNCH("mb_rmsnorm");
}

// y[r,:] = w * x[rows ? rows[r] : r, :] / rms. With parts > 0 (rows must be null) the partial
// products are first added into x. y may be null with parts > 0: only the sum into x is done.
MB_EXPORT int mb_rmsnorm(float* x, const float* partial, int parts, long long part_stride,
                         const void* w, int w_dtype, float eps, void* y, int y_dtype,
                         const int* rows, int R, int H, void* stream) {
  if (R <= 0) return 0;
  if (parts > 0 && rows) MB_FAIL("mb_rmsnorm: partial sums with a row gather");
  if (H > 56 * 1024) MB_FAIL("mb_rmsnorm: a row of %d values is not supported (at most 57344)", H);
  cudaStream_t s = (cudaStream_t)stream;
  if (w_dtype == MB_F32 && y_dtype == MB_F32)
    return rmsnorm_launch<float, float>(x, partial, parts, part_stride, w, eps, y, rows, R, H, s);
  if (w_dtype == MB_F32 && y_dtype == MB_BF16)
    return rmsnorm_launch<float, __nv_bfloat16>(x, partial, parts, part_stride, w, eps, y, rows, R, H, s);
  if (w_dtype == MB_BF16 && y_dtype == MB_F32)
    return rmsnorm_launch<__nv_bfloat16, float>(x, partial, parts, part_stride, w, eps, y, rows, R, H, s);
  return rmsnorm_launch<__nv_bfloat16, __nv_bfloat16>(x, partial, parts, part_stride, w, eps, y, rows, R, H, s);
}

// ------------------------------------------------------------------ SwiGLU
// in [T, 2I]: gate in columns [0, I), up in [I, 2I); out [T, I] = f32(g / (1 + exp(-g))) * u
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ in, T* __restrict__ out, size_t total, int I) {
  mb_grid_wait();
  mb_grid_launch_next();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / I;
    const int c = (int)(i - t * I);
    const float g = to_f32<T>(in[t * 2 * I + c]);
    const float u = to_f32<T>(in[t * 2 * I + I + c]);
    const float b = g / (1.0f + expf(-g));
    out[i] = from_f32<T>(b * u);
  }
}

MB_EXPORT int mb_swiglu(const void* in, void* out, int dtype, int T, int I, void* stream) {
  if (T <= 0) return 0;
  const size_t total = (size_t)T * I;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads
                                                                        : 148 * 16);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == MB_F32)
    mb_launch(swiglu_kernel<float>, dim3(blocks), dim3(threads), 0, s, (const float*)in, (float*)out, total, I);
  else
    mb_launch(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, (const __nv_bfloat16*)in,
                                                             (__nv_bfloat16*)out, total, I);
  MB_CHECK_LAUNCH("mb_swiglu");
}

// ------------------------------------------------------------------ q/k norm + RoPE + cache
// qkv [T, (nh + 2 nkv) hd]: q heads, then k heads, then v heads of a token. One warp per
// (token, head): RMSNorm over the head with q_norm / k_norm (null: no norm), rotate_half over
// the first rot_dim values with angle = f32(inv_freq[i] * pos), q written back in place, k and
// v (when write_kv) stored in the cache at the token's slot and position.
#define QK_WARPS 4
template <typename T, typename TW>
__global__ void qk_norm_rope_store_kernel(
    T* __restrict__ qkv, const TW* __restrict__ q_norm, const TW* __restrict__ k_norm, float eps,
    const float* __restrict__ inv_freq, int rot_dim, const int* __restrict__ tok_seq,
    const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
    const int* __restrict__ page_table, int max_pages, int ring_pages, T* __restrict__ kpool,
    T* __restrict__ vpool, int nh, int nkv, int hd, int write_kv) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ float heads[];  // QK_WARPS x hd
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int head = blockIdx.y * QK_WARPS + warp;
  const int total = nh + 2 * nkv;
  if (head >= total) return;
  const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
  if (!is_q && !write_kv) return;
  T* src = qkv + (size_t)t * total * hd + (size_t)head * hd;
  float* buf = heads + warp * hd;
  const int pos = tok_pos[t];
  T* dst = src;
  if (!is_q) {
    const int g = is_k ? head - nh : head - nh - nkv;
    const size_t row = kv_row(page_table, max_pages, ring_pages, seq_slot[tok_seq[t]], pos, nkv, g);
    dst = (is_k ? kpool : vpool) + row * hd;
    if (!is_k) {  // values are stored as they are
      for (int i = lane; i < hd; i += 32) dst[i] = src[i];
      return;
    }
  }
  const TW* w = is_q ? q_norm : k_norm;
  float sum = 0.f;
  for (int i = lane; i < hd; i += 32) {
    const float v = to_f32<T>(src[i]);
    buf[i] = v;
    sum = fmaf(v, v, sum);
  }
  sum = warp_sum(sum);
  if (w) {
    const float inv = 1.0f / sqrtf(sum / (float)hd + eps);
    for (int i = lane; i < hd; i += 32) buf[i] = to_f32<TW>(w[i]) * (buf[i] * inv);
  }
  __syncwarp();
  const int half = rot_dim >> 1;
  for (int i = lane; i < hd; i += 32) {
    float v = buf[i];
    if (i < rot_dim) {
      const int f = i < half ? i : i - half;
      const float angle = inv_freq[f] * (float)pos;  // float32 product, as the reference
      const float c = cosf(angle), s = sinf(angle);
      v = i < half ? buf[i] * c - buf[i + half] * s : buf[i] * c + buf[i - half] * s;
    }
    dst[i] = from_f32<T>(v);
  }
}


// The same for bfloat16 heads of 64, 128 or 256 values that rotate as a whole, for steps of few
// tokens (as many small warps in flight as possible): one warp per (token, head), every lane holds V = hd / 64 neighbouring values of the first half and their
// rotation partners of the second half, so nothing goes through shared memory. The source is
// the fused qkv row, or (PARTIAL) the float32 partial sums of a split product
// [parts][T][width], which are added up here in split order. q goes to q_out [T, nh * hd] when
// given, else back in place.
template <int V, typename TW, bool PARTIAL>
__global__ void __launch_bounds__(QK_WARPS * 32)
qk_narrow_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ partial, int parts,
               size_t part_stride, __nv_bfloat16* __restrict__ q_out,
               const TW* __restrict__ q_norm, const TW* __restrict__ k_norm, float eps,
               const float* __restrict__ inv_freq, const int* __restrict__ tok_seq,
               const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
               const int* __restrict__ page_table, int max_pages, int ring_pages,
               __nv_bfloat16* __restrict__ kpool, __nv_bfloat16* __restrict__ vpool, int nh,
               int nkv, int write_kv) {
  mb_grid_wait();
  mb_grid_launch_next();
  constexpr int HD = 64 * V, HALF = 32 * V;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int head = blockIdx.y * QK_WARPS + warp;
  const int total = nh + 2 * nkv;
  if (head >= total) return;
  const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
  if (!is_q && !write_kv) return;
  const size_t col = (size_t)head * HD + V * lane;
  float a[V], b[V];
  if (PARTIAL) {
#pragma unroll
    for (int j = 0; j < V; ++j) a[j] = b[j] = 0.f;
    const float* src0 = partial + (size_t)t * total * HD + col;
#pragma unroll 4
    for (int p = 0; p < parts; ++p) {
      const float* src = src0 + (size_t)p * part_stride;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        a[j] += __ldg(src + j);
        b[j] += __ldg(src + HALF + j);
      }
    }
  } else {
    const __nv_bfloat16* src = qkv + (size_t)t * total * HD + col;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      a[j] = __bfloat162float(src[j]);
      b[j] = __bfloat162float(src[HALF + j]);
    }
  }
  const int pos = tok_pos[t];
  __nv_bfloat16* dst;
  if (is_q) {
    dst = q_out ? q_out + (size_t)t * nh * HD + col : qkv + (size_t)t * total * HD + col;
  } else {
    const int g = is_k ? head - nh : head - nh - nkv;
    const size_t row = kv_row(page_table, max_pages, ring_pages, seq_slot[tok_seq[t]], pos, nkv, g);
    dst = (is_k ? kpool : vpool) + row * HD + V * lane;
  }
  if (is_q || is_k) {
    const TW* w = is_q ? q_norm : k_norm;
    if (w) {
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < V; ++j) sum = fmaf(a[j], a[j], fmaf(b[j], b[j], sum));
      sum = warp_sum(sum);
      const float inv = 1.0f / sqrtf(sum / (float)HD + eps);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        a[j] = to_f32<TW>(w[V * lane + j]) * (a[j] * inv);
        b[j] = to_f32<TW>(w[HALF + V * lane + j]) * (b[j] * inv);
      }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float angle = inv_freq[V * lane + j] * (float)pos;  // float32 product
      float sn, cs;
      sincosf(angle, &sn, &cs);
      const float ra = a[j] * cs - b[j] * sn, rb = b[j] * cs + a[j] * sn;
      a[j] = ra;
      b[j] = rb;
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) {
    dst[j] = __float2bfloat16_rn(a[j]);
    dst[HALF + j] = __float2bfloat16_rn(b[j]);
  }
}

// And for steps of many tokens, with 16-byte accesses: hd / 16 neighbouring lanes share a head, each holds eight neighbouring values of
// the first half and their rotation partners of the second half, so nothing goes through
// shared memory and a warp works on 512 / hd heads at once. A warp takes `passes` such groups
// of heads of its token one after another and forms the sines and cosines once. The source is
// the fused qkv row, or (PARTIAL) the float32 partial sums of a split product
// [parts][T][width], which are added up here in split order. q goes to q_out [T, nh * hd] when
// given, else back in place.
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

template <int HD, typename TW, bool PARTIAL>
__global__ void __launch_bounds__(QK_WARPS * 32)
qk_wide_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ partial, int parts,
               size_t part_stride, __nv_bfloat16* __restrict__ q_out,
               const TW* __restrict__ q_norm, const TW* __restrict__ k_norm, float eps,
               const float* __restrict__ inv_freq, const int* __restrict__ tok_seq,
               const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
               const int* __restrict__ page_table, int max_pages, int ring_pages,
               __nv_bfloat16* __restrict__ kpool, __nv_bfloat16* __restrict__ vpool, int nh,
               int nkv, int write_kv, int passes) {
  mb_grid_wait();
  mb_grid_launch_next();
  constexpr int HALF = HD / 2, L = HALF / 8, HPP = 32 / L;  // lanes a head, heads a pass
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sl = lane % L, hl = lane / L;
  const int t = blockIdx.x;
  const int total = nh + 2 * nkv;
  const int pos = tok_pos[t];
  const int group0 = (blockIdx.y * (blockDim.x >> 5) + warp) * passes;
  float cs[8], sn[8];
  bool have_angles = false;
  for (int i = 0; i < passes; ++i) {
    const int head0 = (group0 + i) * HPP;
    if (head0 >= total) break;  // the whole warp
    const int head = head0 + hl;
    const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
    const bool live = head < total && (is_q || write_kv);
    const size_t col = (size_t)head * HD + 8 * sl;
    float a[8], b[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = b[j] = 0.f;
    if (live) {
      if (PARTIAL) {
        const float* src0 = partial + (size_t)t * total * HD + col;
#pragma unroll 2
        for (int p = 0; p < parts; ++p) {
          const float4* sa = reinterpret_cast<const float4*>(src0 + (size_t)p * part_stride);
          const float4* sb = reinterpret_cast<const float4*>(src0 + (size_t)p * part_stride + HALF);
          const float4 a0 = __ldg(sa), a1 = __ldg(sa + 1), b0 = __ldg(sb), b1 = __ldg(sb + 1);
          a[0] += a0.x; a[1] += a0.y; a[2] += a0.z; a[3] += a0.w;
          a[4] += a1.x; a[5] += a1.y; a[6] += a1.z; a[7] += a1.w;
          b[0] += b0.x; b[1] += b0.y; b[2] += b0.z; b[3] += b0.w;
          b[4] += b1.x; b[5] += b1.y; b[6] += b1.z; b[7] += b1.w;
        }
      } else {
        const __nv_bfloat16* src = qkv + (size_t)t * total * HD + col;
        unpack8(*reinterpret_cast<const uint4*>(src), a);
        unpack8(*reinterpret_cast<const uint4*>(src + HALF), b);
      }
    }
    if (head0 < nh + nkv) {  // some head of this pass is a q or k head (uniform over the warp)
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) sum = fmaf(a[j], a[j], fmaf(b[j], b[j], sum));
#pragma unroll
      for (int o = L / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (!have_angles) {
        // the lanes that hold the same eight columns of different heads share the work: each
        // forms 8 / HPP of the eight sines and cosines and hands them round
        constexpr int PER = 8 / HPP;
        float my_sn[PER], my_cs[PER];
#pragma unroll
        for (int r = 0; r < PER; ++r) {
          const float angle = inv_freq[8 * sl + hl * PER + r] * (float)pos;  // float32 product
          sincosf(angle, &my_sn[r], &my_cs[r]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          sn[j] = __shfl_sync(0xffffffffu, my_sn[j % PER], (j / PER) * L + sl);
          cs[j] = __shfl_sync(0xffffffffu, my_cs[j % PER], (j / PER) * L + sl);
        }
        have_angles = true;
      }
      if (live && (is_q || is_k)) {
        const TW* w = is_q ? q_norm : k_norm;
        if (w) {
          const float inv = 1.0f / sqrtf(sum / (float)HD + eps);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            a[j] = to_f32<TW>(w[8 * sl + j]) * (a[j] * inv);
            b[j] = to_f32<TW>(w[HALF + 8 * sl + j]) * (b[j] * inv);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float ra = a[j] * cs[j] - b[j] * sn[j], rb = b[j] * cs[j] + a[j] * sn[j];
          a[j] = ra;
          b[j] = rb;
        }
      }
    }
    if (!live) continue;
    __nv_bfloat16* dst;
    if (is_q) {
      dst = q_out ? q_out + (size_t)t * nh * HD + col : qkv + (size_t)t * total * HD + col;
    } else {
      const int g = is_k ? head - nh : head - nh - nkv;
      const size_t row =
          kv_row(page_table, max_pages, ring_pages, seq_slot[tok_seq[t]], pos, nkv, g);
      dst = (is_k ? kpool : vpool) + row * HD + 8 * sl;
    }
    *reinterpret_cast<uint4*>(dst) = pack8(a);
    *reinterpret_cast<uint4*>(dst + HALF) = pack8(b);
  }
}

// `partial` (may be null): float32 [parts][T][(nh + 2 nkv) hd] partial sums that stand for qkv
// (bfloat16 heads of 64/128/256 values that rotate as a whole only); `q_out` (may be null):
// where q goes instead of back into qkv, [T, nh * hd].
MB_EXPORT int mb_qk_norm_rope_store(void* qkv, const float* partial, int parts,
                                    long long part_stride, void* q_out, int dtype,
                                    const void* q_norm, const void* k_norm,
                                    int w_dtype, float eps, const float* inv_freq, int rot_dim,
                                    const int* tok_seq, const int* tok_pos, const int* seq_slot,
                                    const int* page_table, int max_pages, int ring_pages,
                                    void* kpool, void* vpool, int T, int nh, int nkv, int hd,
                                    int write_kv, void* stream) {
  if (T <= 0) return 0;
  if (rot_dim < 0 || rot_dim > hd || (rot_dim & 1))
    MB_FAIL("mb_qk_norm_rope_store: %d of %d values rotate", rot_dim, hd);
  if (hd <= 0 || hd > 1024) MB_FAIL("mb_qk_norm_rope_store: heads of %d", hd);
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(T, (nh + 2 * nkv + QK_WARPS - 1) / QK_WARPS);
  const bool aligned = !(((uintptr_t)qkv | (uintptr_t)partial | (uintptr_t)q_out |
                          (uintptr_t)kpool | (uintptr_t)vpool) & 15) && (part_stride & 3) == 0;
  const bool fast = dtype == MB_BF16 && rot_dim == hd && (hd == 64 || hd == 128 || hd == 256) &&
                    aligned;
  if ((partial || q_out) && !fast)
    MB_FAIL("mb_qk_norm_rope_store: partial sums or a separate q for heads of %d values "
            "(%d rotate)%s are not supported", hd, rot_dim, aligned ? "" : ", not 16-byte aligned,");
  if (fast) {
    typedef __nv_bfloat16 bf;
    if (T < 512) {
#define QKN(V_, TW_, P_)                                                                       \
  mb_launch(qk_narrow_kernel<V_, TW_, P_>, grid, dim3(QK_WARPS * 32), 0, s,                    \
      (bf*)qkv, partial, parts, (size_t)part_stride, (bf*)q_out, (const TW_*)q_norm,           \
      (const TW_*)k_norm, eps, inv_freq, tok_seq, tok_pos, seq_slot, page_table, max_pages,    \
      ring_pages, (bf*)kpool, (bf*)vpool, nh, nkv, write_kv)
#define QKN_V(TW_, P_)                                                                         \
  if (hd == 64) QKN(1, TW_, P_); else if (hd == 128) QKN(2, TW_, P_); else QKN(4, TW_, P_)
      if (w_dtype == MB_F32) { if (partial) { QKN_V(float, true); } else { QKN_V(float, false); } }
      else { if (partial) { QKN_V(bf, true); } else { QKN_V(bf, false); } }
#undef QKN_V
#undef QKN
      MB_CHECK_LAUNCH("mb_qk_norm_rope_store");
    }
    // groups of 512 / hd heads: blocks of four warps that take three groups each
    const int groups = ((nh + 2 * nkv) * hd + 511) / 512;
    const int warps = QK_WARPS, passes = 3;
    dim3 fgrid(T, (groups + warps * passes - 1) / (warps * passes));
#define QKF(HD_, TW_, P_)                                                                      \
  mb_launch(qk_wide_kernel<HD_, TW_, P_>, fgrid, dim3(warps * 32), 0, s,                       \
      (bf*)qkv, partial, parts, (size_t)part_stride, (bf*)q_out, (const TW_*)q_norm,           \
      (const TW_*)k_norm, eps, inv_freq, tok_seq, tok_pos, seq_slot, page_table, max_pages,    \
      ring_pages, (bf*)kpool, (bf*)vpool, nh, nkv, write_kv, passes)
#define QKF_V(TW_, P_)                                                                         \
  if (hd == 64) QKF(64, TW_, P_); else if (hd == 128) QKF(128, TW_, P_); else QKF(256, TW_, P_)
    if (w_dtype == MB_F32) { if (partial) { QKF_V(float, true); } else { QKF_V(float, false); } }
    else { if (partial) { QKF_V(bf, true); } else { QKF_V(bf, false); } }
#undef QKF_V
#undef QKF
    MB_CHECK_LAUNCH("mb_qk_norm_rope_store");
  }
  const size_t smem = (size_t)QK_WARPS * hd * sizeof(float);
#define QK_LAUNCH(T_, TW_)                                                                     \
  mb_launch(qk_norm_rope_store_kernel<T_, TW_>, dim3(grid), dim3(QK_WARPS * 32), smem, s,                         \
      (T_*)qkv, (const TW_*)q_norm, (const TW_*)k_norm, eps, inv_freq, rot_dim, tok_seq,       \
      tok_pos, seq_slot, page_table, max_pages, ring_pages, (T_*)kpool, (T_*)vpool, nh, nkv,   \
      hd, write_kv)
  if (dtype == MB_F32 && w_dtype == MB_F32) QK_LAUNCH(float, float);
  else if (dtype == MB_F32) QK_LAUNCH(float, __nv_bfloat16);
  else if (w_dtype == MB_F32) QK_LAUNCH(__nv_bfloat16, float);
  else QK_LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef QK_LAUNCH
  MB_CHECK_LAUNCH("mb_qk_norm_rope_store");
}

// ------------------------------------------------------------------ decode without the host
// Between two decode steps that run without a host round trip: the tokens just chosen become
// the next step's input ids and every position moves on by one.
__global__ void advance_decode_kernel(int* __restrict__ tok_ids, int* __restrict__ tok_pos,
                                      const int* __restrict__ chosen, int* __restrict__ history,
                                      int B) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int t = chosen[b];
  tok_ids[b] = t;
  tok_pos[b] += 1;
  if (history) history[b] = t;
}

MB_EXPORT int mb_advance_decode(int* tok_ids, int* tok_pos, const int* chosen, int* history,
                                int B, void* stream) {
  if (B <= 0) return 0;
  mb_launch(advance_decode_kernel, dim3((B + 127) / 128), dim3(128), 0, (cudaStream_t)stream, tok_ids, tok_pos,
                                                                          chosen, history, B);
  MB_CHECK_LAUNCH("mb_advance_decode");
}
