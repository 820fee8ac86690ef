// Bandwidth-bound kernels around the matrix products: embedding rows, RMSNorm (plain, and
// fused with the sum of split partial products into the residual), SwiGLU, and the step from
// one decode step to the next on the device. One file for float32 and bfloat16 activations;
// sums, norms and the residual are float32 in both.
//
// Formulas as the reference computes them (paths within the reference project):
//   RMSNorm   src/infer/mormot.ai.infer.backend.cpu.pas:1769-1795, tools/cuda/ops.cu:116-150
//   SwiGLU    src/infer/mormot.ai.infer.backend.cpu.pas:1827-1833, tools/cuda/ops.cu:155-178
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
template <typename TO, int VEC, int RMS_THREADS, bool PARTIAL>
__global__ void __launch_bounds__(RMS_THREADS)
rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ partial, int parts,
                   size_t part_stride, const void* __restrict__ w, int w_bf16, float eps,
                   TO* __restrict__ y, const int* __restrict__ rows, int H) {
  MB_TRACE_BEGIN();
  __shared__ float red[33];
  const int r = blockIdx.x;
  // Before the wait for the kernel before: what does not depend on it. The row index and the
  // norm's weights were settled by kernels further back (complete once this kernel runs: every
  // kernel of the stream waits for the one before it ahead of letting its successor start).
  // With PARTIAL the kernel before is the matrix product that left its split sums, which
  // wrote nothing else: the residual row itself can be asked for before the wait too, and
  // only the split sums come after it.
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * H;
  float wv[VEC][4];
  if (y != nullptr) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RMS_THREADS + threadIdx.x) * 4;
      if (c >= H) continue;
      if (w_bf16) {  // four weights with one load (c is a multiple of 4)
        const uint2 raw = *(const uint2*)((const __nv_bfloat16*)w + c);
        const float2 lo = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x);
        const float2 hi = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
        wv[i][0] = lo.x; wv[i][1] = lo.y; wv[i][2] = hi.x; wv[i][3] = hi.y;
      } else {
        const float4 raw = *(const float4*)((const float*)w + c);
        wv[i][0] = raw.x; wv[i][1] = raw.y; wv[i][2] = raw.z; wv[i][3] = raw.w;
      }
    }
  }
  float4 v[VEC];
  float sum = 0.f;
  if (PARTIAL) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RMS_THREADS + threadIdx.x) * 4;
      v[i] = c < H ? *(const float4*)(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  mb_grid_wait();
  mb_grid_launch_next();
  if (!PARTIAL) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RMS_THREADS + threadIdx.x) * 4;
      v[i] = c < H ? *(const float4*)(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  if (PARTIAL) {  // a kernel of its own: the loads in flight below cost registers
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RMS_THREADS + threadIdx.x) * 4;
      if (c >= H) continue;
      const float* pp = partial + (size_t)src * H + c;
      // up to eight loads in flight at once, then added in split order
      for (int p0 = 0; p0 < parts; p0 += 8) {
        float4 a[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (p0 + j < parts) a[j] = __ldg((const float4*)(pp + (size_t)(p0 + j) * part_stride));
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (p0 + j < parts) {
            v[i].x += a[j].x; v[i].y += a[j].y; v[i].z += a[j].z; v[i].w += a[j].w;
          }
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
    o[0] = wv[i][0] * (v[i].x * inv);
    o[1] = wv[i][1] * (v[i].y * inv);
    o[2] = wv[i][2] * (v[i].z * inv);
    o[3] = wv[i][3] * (v[i].w * inv);
    if (sizeof(TO) == 4) {
      *(float4*)((float*)yr + c) = make_float4(o[0], o[1], o[2], o[3]);
    } else {
      __nv_bfloat162 h[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
      *(uint2*)((__nv_bfloat16*)yr + c) = *(uint2*)h;
    }
  }
  MB_TRACE_END(2);
}

template <typename TW, typename TO>
static int rmsnorm_launch(float* x, const float* partial, int parts, size_t part_stride,
                          const void* w, float eps, void* y, const int* rows, int R, int H,
                          cudaStream_t s) {
  const bool aligned = ((uintptr_t)x & 15) == 0 && ((uintptr_t)partial & 15) == 0 &&
                       (part_stride & 3) == 0 && ((uintptr_t)y & 15) == 0;
  if (H % 4 == 0 && H <= 4 * 1024 * 4 && aligned && ((uintptr_t)w & 15) == 0) {
    // few rows (a decode step) or wide rows: 1024 threads a row, so that a thread waits for few
    // loads; many rows: 256 threads a row and more rows per SM
    const int w_bf16 = sizeof(TW) == 2;
#define RMS_GO(V_, T_)                                                                      \
  if (parts > 0)                                                                            \
    mb_launch(rmsnorm_vec_kernel<TO, V_, T_, true>, dim3(R), dim3(T_), 0, s, x, partial,    \
              parts, part_stride, w, w_bf16, eps, (TO*)y, rows, H);                         \
  else                                                                                      \
    mb_launch(rmsnorm_vec_kernel<TO, V_, T_, false>, dim3(R), dim3(T_), 0, s, x, partial,   \
              parts, part_stride, w, w_bf16, eps, (TO*)y, rows, H)
    if ((R <= 256 && H > 1024) || H > 4 * 256 * 4) {
      const int vec = (H + 4 * 1024 - 1) / (4 * 1024);
      if (vec <= 1) { RMS_GO(1, 1024); }
      else if (vec <= 2) { RMS_GO(2, 1024); }
      else { RMS_GO(4, 1024); }
    } else {
      const int vec = (H + 4 * 256 - 1) / (4 * 256);
      if (vec <= 1) { RMS_GO(1, 256); }
      else if (vec <= 2) { RMS_GO(2, 256); }
      else { RMS_GO(4, 256); }
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
