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
    embed_kernel<float><<<T, threads, 0, s>>>((const float*)table, ids, x, H, V);
  else
    embed_kernel<__nv_bfloat16><<<T, threads, 0, s>>>((const __nv_bfloat16*)table, ids, x, H, V);
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

template <typename TW, typename TO>
static int rmsnorm_launch(float* x, const float* partial, int parts, size_t part_stride,
                          const void* w, float eps, void* y, const int* rows, int R, int H,
                          cudaStream_t s) {
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  const size_t smem = parts > 0 ? (size_t)H * sizeof(float) : 0;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(rmsnorm_kernel<TW, TO>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) MB_FAIL("mb_rmsnorm: a row of %d values: %s", H, cudaGetErrorString(e));
  }
  rmsnorm_kernel<TW, TO><<<R, threads, smem, s>>>(x, partial, parts, part_stride,
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
    swiglu_kernel<float><<<blocks, threads, 0, s>>>((const float*)in, (float*)out, total, I);
  else
    swiglu_kernel<__nv_bfloat16><<<blocks, threads, 0, s>>>((const __nv_bfloat16*)in,
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

MB_EXPORT int mb_qk_norm_rope_store(void* qkv, int dtype, const void* q_norm, const void* k_norm,
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
  const size_t smem = (size_t)QK_WARPS * hd * sizeof(float);
#define QK_LAUNCH(T_, TW_)                                                                     \
  qk_norm_rope_store_kernel<T_, TW_><<<grid, QK_WARPS * 32, smem, s>>>(                        \
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
  advance_decode_kernel<<<(B + 127) / 128, 128, 0, (cudaStream_t)stream>>>(tok_ids, tok_pos,
                                                                          chosen, history, B);
  MB_CHECK_LAUNCH("mb_advance_decode");
}
