// Per-head RMSNorm of q and k, rotary position encoding, and the write of k and v into the
// paged cache, in one kernel after the fused q/k/v product, for float32 and bfloat16
// activations; sums, norms and angles are float32 in both.
//
// Formulas as the reference computes them (paths within the reference project):
//   q/k norm + RoPE + cache store   tools/cuda/ops.cu:211-314,
//             angles src/infer/mormot.ai.infer.decoder.pas:2539-2561
#include "common.cuh"

MB_DEFINE_LAST_ERROR

// a norm weight that is float32 or bfloat16 (the two fast kernels take either at run time)
__device__ __forceinline__ float norm_w(const void* w, int w_bf16, int i) {
  return w_bf16 ? __bfloat162float(((const __nv_bfloat16*)w)[i]) : ((const float*)w)[i];
}

// qkv [T, (nh + 2 nkv) hd]: q heads, then k heads, then v heads of a token. One warp per
// (token, head): RMSNorm over the head with q_norm / k_norm (null: no norm), rotate_half over
// the first rot_dim values with angle = f32(inv_freq[i] * pos), q written back in place, k and
// v (when write_kv) stored in the cache at the token's slot and position.
#define QK_WARPS 4
template <typename T, typename TW>
__global__ void qk_norm_rope_store_kernel(
    T* __restrict__ qkv, const TW* __restrict__ q_norm, const TW* __restrict__ k_norm, float eps,
    const float* __restrict__ inv_freq, int rot_dim, const int* __restrict__ tok_slot,
    const int* __restrict__ tok_pos,
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
    const size_t row = kv_row(page_table, max_pages, ring_pages, tok_slot[t], pos, nkv, g);
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
template <int V, bool PARTIAL>
__global__ void __launch_bounds__(QK_WARPS * 32)
qk_narrow_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ partial, int parts,
               size_t part_stride, __nv_bfloat16* __restrict__ q_out,
               const void* __restrict__ q_norm, const void* __restrict__ k_norm, int w_bf16,
               float eps,
               const float* __restrict__ inv_freq, const int* __restrict__ tok_slot,
               const int* __restrict__ tok_pos,
               const int* __restrict__ page_table, int max_pages, int ring_pages,
               __nv_bfloat16* __restrict__ kpool, __nv_bfloat16* __restrict__ vpool, int nh,
               int nkv, int write_kv) {
  MB_TRACE_BEGIN();
  constexpr int HD = 64 * V, HALF = 32 * V;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int head = blockIdx.y * QK_WARPS + warp;
  const int total = nh + 2 * nkv;
  const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
  const bool live = head < total && (is_q || write_kv);
  const size_t col = (size_t)head * HD + V * lane;
  // Before the wait for the kernel before (which wrote the values of q, k and v, nothing
  // else): everything that does not depend on them. The token's position and slot, the page
  // table, the norm weights and the frequencies were settled by kernels further back, which
  // are complete once this kernel runs (every kernel of the stream waits for the one before it
  // ahead of letting its successor start). So the only loads after the wait are the values.
  __nv_bfloat16* dst = nullptr;
  float wa[V], wb[V], sn[V], cs[V];
  bool normed = false;
  if (live) {
    const int pos = tok_pos[t];
    if (is_q) {
      dst = q_out ? q_out + (size_t)t * nh * HD + col : qkv + (size_t)t * total * HD + col;
    } else {
      const int g = is_k ? head - nh : head - nh - nkv;
      const size_t row = kv_row(page_table, max_pages, ring_pages, tok_slot[t], pos, nkv, g);
      dst = (is_k ? kpool : vpool) + row * HD + V * lane;
    }
    if (is_q || is_k) {
      const void* w = is_q ? q_norm : k_norm;
      normed = w != nullptr;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        wa[j] = normed ? norm_w(w, w_bf16, V * lane + j) : 1.f;
        wb[j] = normed ? norm_w(w, w_bf16, HALF + V * lane + j) : 1.f;
        const float angle = inv_freq[V * lane + j] * (float)pos;  // float32 product
        sincosf(angle, &sn[j], &cs[j]);
      }
    }
  }
  mb_grid_wait();
  mb_grid_launch_next();
  if (!live) return;
  float a[V], b[V];
  if (PARTIAL) {
    const float* src0 = partial + (size_t)t * total * HD + col;
    // up to eight parts asked for at once, then added in split order
#pragma unroll
    for (int j = 0; j < V; ++j) a[j] = b[j] = 0.f;
    for (int p0 = 0; p0 < parts; p0 += 8) {
      float pa[8][V], pb[8][V];
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        const float* src = src0 + (size_t)(p0 + p) * part_stride;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          pa[p][j] = p0 + p < parts ? __ldg(src + j) : 0.f;
          pb[p][j] = p0 + p < parts ? __ldg(src + HALF + j) : 0.f;
        }
      }
#pragma unroll
      for (int p = 0; p < 8; ++p)
#pragma unroll
        for (int j = 0; j < V; ++j) {
          a[j] += pa[p][j];
          b[j] += pb[p][j];
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
  if (is_q || is_k) {
    if (normed) {
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < V; ++j) sum = fmaf(a[j], a[j], fmaf(b[j], b[j], sum));
      sum = warp_sum(sum);
      const float inv = 1.0f / sqrtf(sum / (float)HD + eps);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        a[j] = wa[j] * (a[j] * inv);
        b[j] = wb[j] * (b[j] * inv);
      }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float ra = a[j] * cs[j] - b[j] * sn[j], rb = b[j] * cs[j] + a[j] * sn[j];
      a[j] = ra;
      b[j] = rb;
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) {
    dst[j] = __float2bfloat16_rn(a[j]);
    dst[HALF + j] = __float2bfloat16_rn(b[j]);
  }
  MB_TRACE_END(3);  // by thread 0: warp 0's head is a q head, which is always live
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

#define QK_PASSES 3  // groups of heads that a warp of the wide form takes, at most
template <int HD, bool PARTIAL>
__global__ void __launch_bounds__(QK_WARPS * 32)
qk_wide_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ partial, int parts,
               size_t part_stride, __nv_bfloat16* __restrict__ q_out,
               const void* __restrict__ q_norm, const void* __restrict__ k_norm, int w_bf16,
               float eps,
               const float* __restrict__ inv_freq, const int* __restrict__ tok_slot,
               const int* __restrict__ tok_pos,
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
  // every pass's values are asked for before the first pass is worked on: a pass's stores
  // may lie over the next one's source (q is rotated in place), so the compiler would not
  // move the loads up by itself, and three round trips to memory in a row would set the time
  uint4 raw[QK_PASSES][2];
  if (!PARTIAL) {
#pragma unroll
    for (int i = 0; i < QK_PASSES; ++i) {
      const int head = (group0 + i) * HPP + hl;
      raw[i][0] = raw[i][1] = make_uint4(0u, 0u, 0u, 0u);
      if (i < passes && head < total && (head < nh || write_kv)) {
        const __nv_bfloat16* src = qkv + (size_t)t * total * HD + (size_t)head * HD + 8 * sl;
        raw[i][0] = *reinterpret_cast<const uint4*>(src);
        raw[i][1] = *reinterpret_cast<const uint4*>(src + HALF);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < QK_PASSES; ++i) {
    if (i >= passes) break;
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
        unpack8(raw[i][0], a);
        unpack8(raw[i][1], b);
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
        const void* w = is_q ? q_norm : k_norm;
        if (w) {
          const float inv = 1.0f / sqrtf(sum / (float)HD + eps);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            a[j] = norm_w(w, w_bf16, 8 * sl + j) * (a[j] * inv);
            b[j] = norm_w(w, w_bf16, HALF + 8 * sl + j) * (b[j] * inv);
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
          kv_row(page_table, max_pages, ring_pages, tok_slot[t], pos, nkv, g);
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
                                    const int* tok_slot, const int* tok_pos,
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
    const int w_bf16 = w_dtype == MB_BF16;
    if (T < 512) {
#define QKN(V_, P_)                                                                            \
  mb_launch(qk_narrow_kernel<V_, P_>, grid, dim3(QK_WARPS * 32), 0, s, (bf*)qkv, partial,      \
      parts, (size_t)part_stride, (bf*)q_out, q_norm, k_norm, w_bf16, eps, inv_freq, tok_slot, \
      tok_pos, page_table, max_pages, ring_pages, (bf*)kpool, (bf*)vpool, nh, nkv,   \
      write_kv)
#define QKN_V(P_)                                                                              \
  if (hd == 64) QKN(1, P_); else if (hd == 128) QKN(2, P_); else QKN(4, P_)
      if (partial) { QKN_V(true); } else { QKN_V(false); }
#undef QKN_V
#undef QKN
      MB_CHECK_LAUNCH("mb_qk_norm_rope_store");
    }
    // groups of 512 / hd heads: blocks of four warps that take three groups each
    const int groups = ((nh + 2 * nkv) * hd + 511) / 512;
    const int warps = QK_WARPS, passes = QK_PASSES;
    dim3 fgrid(T, (groups + warps * passes - 1) / (warps * passes));
#define QKF(HD_, P_)                                                                           \
  mb_launch(qk_wide_kernel<HD_, P_>, fgrid, dim3(warps * 32), 0, s, (bf*)qkv, partial, parts,  \
      (size_t)part_stride, (bf*)q_out, q_norm, k_norm, w_bf16, eps, inv_freq, tok_slot,        \
      tok_pos, page_table, max_pages, ring_pages, (bf*)kpool, (bf*)vpool, nh, nkv,   \
      write_kv, passes)
#define QKF_V(P_)                                                                              \
  if (hd == 64) QKF(64, P_); else if (hd == 128) QKF(128, P_); else QKF(256, P_)
    if (partial) { QKF_V(true); } else { QKF_V(false); }
#undef QKF_V
#undef QKF
    MB_CHECK_LAUNCH("mb_qk_norm_rope_store");
  }
  const size_t smem = (size_t)QK_WARPS * hd * sizeof(float);
#define QK_LAUNCH(T_, TW_)                                                                     \
  mb_launch(qk_norm_rope_store_kernel<T_, TW_>, dim3(grid), dim3(QK_WARPS * 32), smem, s,                         \
      (T_*)qkv, (const TW_*)q_norm, (const TW_*)k_norm, eps, inv_freq, rot_dim, tok_slot,      \
      tok_pos, page_table, max_pages, ring_pages, (T_*)kpool, (T_*)vpool, nh, nkv,   \
      hd, write_kv)
  if (dtype == MB_F32 && w_dtype == MB_F32) QK_LAUNCH(float, float);
  else if (dtype == MB_F32) QK_LAUNCH(float, __nv_bfloat16);
  else if (w_dtype == MB_F32) QK_LAUNCH(__nv_bfloat16, float);
  else QK_LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef QK_LAUNCH
  MB_CHECK_LAUNCH("mb_qk_norm_rope_store");
}

