// Choosing the next token on the device: arg-max (greedy) and a draw from
// softmax(logits / temperature), one block per sequence or, for wide rows, several.
//
// Semantics of the reference's sampler (paths within the reference project):
//   arg-max   src/infer/mormot.ai.infer.sampler.pas:123-159 — the highest value, the lowest
//             index on ties, a NaN never chosen unless all are NaN, -0 equal to +0;
//   draw      src/infer/mormot.ai.infer.sampler.pas:280-342 — softmax in float64 with the
//             maximum subtracted, NaN and infinities weigh 0, one splitmix64 draw per token
//             (:222-233), the vocabulary walked in id order.
// The walk is done in parallel here (per-thread ranges, then a scan), so a draw that falls
// within rounding of a boundary may pick the neighbouring token.
#include "common.cuh"
#include <math.h>

MB_DEFINE_LAST_ERROR

#define SAMPLE_THREADS 1024
#define SORT_CHUNK 2048  // keys that are sorted in shared memory at a time (16 KB)

struct Best {
  float v;
  int i;
};

// a is better than b: b has no candidate yet, or a is greater, or equal with a lower index
__device__ __forceinline__ bool better(const Best& a, const Best& b) {
  if (a.i < 0) return false;
  if (b.i < 0) return true;
  return a.v > b.v || (a.v == b.v && a.i < b.i);
}

__device__ Best block_argmax(const float* __restrict__ row, int V, Best* sh) {
  Best b = {0.f, -1};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v != v) continue;  // NaN
    const Best c = {v, i};
    if (better(c, b)) b = c;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best c;
    c.v = __shfl_xor_sync(0xffffffffu, b.v, o);
    c.i = __shfl_xor_sync(0xffffffffu, b.i, o);
    if (better(c, b)) b = c;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = b;
  __syncthreads();
  if (warp == 0) {
    b = lane < (int)(blockDim.x >> 5) ? sh[lane] : Best{0.f, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best c;
      c.v = __shfl_xor_sync(0xffffffffu, b.v, o);
      c.i = __shfl_xor_sync(0xffffffffu, b.i, o);
      if (better(c, b)) b = c;
    }
    if (lane == 0) sh[0] = b;
  }
  __syncthreads();
  b = sh[0];
  __syncthreads();
  if (b.i < 0) b.i = 0;  // all NaN
  return b;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, size_t stride, int V, int* __restrict__ out) {
  mb_grid_wait();
  mb_grid_launch_next();
  __shared__ Best sh[32];
  const Best b = block_argmax(logits + blockIdx.x * stride, V, sh);
  if (threadIdx.x == 0) out[blockIdx.x] = b.i;
}

// Two stages for wide rows, so that more than one CTA a row reads the logits: every CTA of
// the first stage finds the best of ARGMAX_CHUNK values, the second stage the best of those
// (the lowest index still wins a tie: chunks are compared in order).
#define ARGMAX_CHUNK 2048
__global__ void __launch_bounds__(256)
argmax_chunks_kernel(const float* __restrict__ logits, size_t stride, int V,
                     Best* __restrict__ partial, int chunks) {
  mb_grid_wait();
  mb_grid_launch_next();
  __shared__ Best sh[32];
  const int i0 = blockIdx.x * ARGMAX_CHUNK;
  const int n = min(ARGMAX_CHUNK, V - i0);
  Best b = block_argmax(logits + blockIdx.y * stride + i0, n, sh);
  if (threadIdx.x == 0) {
    // an all-NaN chunk offers no candidate
    const float v = logits[blockIdx.y * stride + i0 + b.i];
    partial[(size_t)blockIdx.y * chunks + blockIdx.x] = Best{v, v != v ? -1 : i0 + b.i};
  }
}

__global__ void __launch_bounds__(128)
argmax_final_kernel(const Best* __restrict__ partial, int chunks, int* __restrict__ out) {
  mb_grid_wait();
  mb_grid_launch_next();
  __shared__ Best sh[4];
  Best b = {0.f, -1};
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const Best x = partial[(size_t)blockIdx.x * chunks + c];
    if (better(x, b)) b = x;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best c;
    c.v = __shfl_xor_sync(0xffffffffu, b.v, o);
    c.i = __shfl_xor_sync(0xffffffffu, b.i, o);
    if (better(c, b)) b = c;
  }
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = b;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 4; ++w)
      if (better(sh[w], b)) b = sh[w];
    out[blockIdx.x] = b.i < 0 ? 0 : b.i;
  }
}

// bytes of scratch with which mb_argmax uses its two-stage form
MB_EXPORT long long mb_argmax_scratch(int rows, int V) {
  return (long long)rows * ((V + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK) * (long long)sizeof(Best);
}

// out[r] = arg-max of logits[r, 0..V). `scratch` (may be null): mb_argmax_scratch bytes.
MB_EXPORT int mb_argmax(const float* logits, long long stride, int rows, int V, int* out,
                        void* scratch, long long scratch_bytes, void* stream) {
  if (rows <= 0) return 0;
  if (V <= 0) MB_FAIL("mb_argmax: a vocabulary of %d", V);
  cudaStream_t s = (cudaStream_t)stream;
  const int chunks = (V + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
  if (scratch && chunks > 4 && rows <= 65535 && scratch_bytes >= mb_argmax_scratch(rows, V)) {
    mb_launch(argmax_chunks_kernel, dim3(dim3(chunks, rows)), dim3(256), 0, s, logits, (size_t)stride, V,
                                                           (Best*)scratch, chunks);
    mb_launch(argmax_final_kernel, dim3(rows), dim3(128), 0, s, (const Best*)scratch, chunks, out);
  } else {
    mb_launch(argmax_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, s, logits, (size_t)stride, V, out);
  }
  MB_CHECK_LAUNCH("mb_argmax");
}

__device__ __forceinline__ double weight_of(float v, float m, double inv_t) {
  // NaN or an infinity weighs 0 (+Inf as the best is excluded before)
  if ((__float_as_uint(v) & 0x7f800000u) == 0x7f800000u) return 0.0;
  return exp(((double)v - (double)m) * inv_t);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, size_t stride, int V, double inv_t,
              const int* __restrict__ state_index, unsigned long long* __restrict__ states,
              int* __restrict__ out) {
  mb_grid_wait();
  mb_grid_launch_next();
  __shared__ Best sh[32];
  __shared__ double sums[SAMPLE_THREADS];
  __shared__ double target_sh;
  __shared__ int found;
  const float* row = logits + blockIdx.x * stride;
  const Best best = block_argmax(row, V, sh);
  const unsigned bits = __float_as_uint(best.v);
  if ((bits & 0x7f800000u) == 0x7f800000u) {  // no finite best: nothing to draw from
    if (threadIdx.x == 0) out[blockIdx.x] = best.i;
    return;
  }
  // a contiguous range of ids per thread, so that the walk stays in id order
  const int per = (V + blockDim.x - 1) / blockDim.x;
  const int i0 = min(V, (int)threadIdx.x * per), i1 = min(V, i0 + per);
  double mine = 0.0;
  for (int i = i0; i < i1; ++i) mine += weight_of(row[i], best.v, inv_t);
  sums[threadIdx.x] = mine;
  if (threadIdx.x == 0) found = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    // exclusive prefix over the threads' ranges, in order; sums[] becomes the prefix
    double total = 0.0;
    for (int t = 0; t < (int)blockDim.x; ++t) {
      const double v = sums[t];
      sums[t] = total;
      total += v;
    }
    // one splitmix64 draw of this sequence's stream
    unsigned long long* st = states + state_index[blockIdx.x];
    unsigned long long z = (*st += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    const double u = (double)(z >> 11) * (1.0 / 9007199254740992.0);
    target_sh = u * total;
  }
  __syncthreads();
  const double target = target_sh;
  const double before = sums[threadIdx.x];
  if (target >= before && target < before + mine) {
    double cum = before;
    for (int i = i0; i < i1; ++i) {
      const double w = weight_of(row[i], best.v, inv_t);
      cum += w;
      if (w > 0.0 && target < cum) {
        found = i;  // the ranges are disjoint: at most one thread gets here
        break;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) out[blockIdx.x] = found >= 0 ? found : best.i;
}

// ---- the same draw by a cluster of SAMPLE_CTAS CTAs a row (wide vocabularies): each CTA takes
// a contiguous share of the ids, the CTAs exchange their best value, their sum of weights and
// the draw through each other's shared memory, and the CTA whose share holds the drawn point
// walks it. Within a CTA every warp owns a contiguous run of ids and its lanes read it
// interleaved (coalesced); the walk of the run that holds the point is a scan over 32 ids at a
// time.
#define SAMPLE_CTAS 8
#define SAMPLE_CL_THREADS 512

__device__ __forceinline__ uint32_t smp_smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint32_t smp_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void smp_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 8 bytes at `addr` (an address in this CTA's shared memory) as they lie in CTA `rank`
__device__ __forceinline__ unsigned long long smp_peer_u64(uint32_t addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  unsigned long long v;
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(remote) : "memory");
  return v;
}

__global__ void __launch_bounds__(SAMPLE_CL_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, size_t stride, int V, double inv_t,
                      const int* __restrict__ state_index,
                      unsigned long long* __restrict__ states, int* __restrict__ out) {
  mb_grid_wait();
  mb_grid_launch_next();
  constexpr int WARPS = SAMPLE_CL_THREADS / 32;
  __shared__ Best sh[32];
  __shared__ double warp_sums[WARPS];
  __shared__ __align__(8) unsigned long long mine_best;   // value bits << 32 | index
  __shared__ __align__(8) double mine_sum;
  __shared__ int found;
  const int r = blockIdx.x / SAMPLE_CTAS;
  const uint32_t rank = smp_cluster_rank();
  const float* row = logits + r * stride;
  const int share = (V + SAMPLE_CTAS - 1) / SAMPLE_CTAS;
  const int lo = min(V, (int)rank * share), hi = min(V, lo + share);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // 1. the best finite-or-not value of the row: of this share, then of all shares
  Best b = {0.f, -1};
  if (hi > lo) {
    b = block_argmax(row + lo, hi - lo, sh);
    const float v = row[lo + b.i];
    b = Best{v, v != v ? -1 : lo + b.i};  // an all-NaN share offers no candidate
  }
  if (threadIdx.x == 0)
    mine_best = ((unsigned long long)__float_as_uint(b.v) << 32) | (unsigned)b.i;
  smp_cluster_sync();
  Best best = {0.f, -1};
  for (uint32_t k = 0; k < SAMPLE_CTAS; ++k) {  // in share order: the lowest index wins a tie
    const unsigned long long x = smp_peer_u64(smp_smem_u32(&mine_best), k);
    const Best c = {__uint_as_float((unsigned)(x >> 32)), (int)(unsigned)x};
    if (better(c, best)) best = c;
  }
  if (best.i < 0) best.i = 0;  // all NaN
  const unsigned bits = __float_as_uint(best.v);
  const bool no_draw = (bits & 0x7f800000u) == 0x7f800000u || best.i < 0;

  // 2. the weights of this share: a contiguous run of ids per warp, lanes interleaved
  const int per_warp = (hi - lo + WARPS - 1) / WARPS;
  const int w0 = min(hi, lo + warp * per_warp), w1 = min(hi, w0 + per_warp);
  double acc = 0.0;
  if (!no_draw)
    for (int i = w0 + lane; i < w1; i += 32) acc += weight_of(row[i], best.v, inv_t);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) warp_sums[warp] = acc;
  if (threadIdx.x == 0) found = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < WARPS; ++w) t += warp_sums[w];  // in id order
    mine_sum = t;
  }
  smp_cluster_sync();
  double before = 0.0, total = 0.0;
  for (uint32_t k = 0; k < SAMPLE_CTAS; ++k) {
    const double v = __longlong_as_double((long long)smp_peer_u64(smp_smem_u32(&mine_sum), k));
    if (k < rank) before += v;
    total += v;
  }
  // 3. one splitmix64 draw of this sequence's stream: every CTA forms it from the state as it
  // was, the first one stores the state that follows (after all have read it)
  unsigned long long* st = states + state_index[r];
  unsigned long long z = *st + 0x9E3779B97F4A7C15ull;
  const unsigned long long next_state = z;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  const double target = (double)(z >> 11) * (1.0 / 9007199254740992.0) * total;
  smp_cluster_sync();
  if (rank == 0 && threadIdx.x == 0) {
    if (no_draw) out[r] = best.i;  // no finite best: nothing to draw from, the stream stays
    else *st = next_state;
  }
  if (no_draw) return;
  const double mine = mine_sum;
  const bool last = rank == SAMPLE_CTAS - 1;
  if (!(target >= before && (target < before + mine || last))) return;
  // 4. the point lies in this share: the warp whose run holds it walks the run
  double wb = before;
  for (int w = 0; w < warp; ++w) wb += warp_sums[w];
  const double ws = warp_sums[warp];
  if (target >= wb && target < wb + ws) {
    double cum = wb;
    for (int i0 = w0; i0 < w1; i0 += 32) {
      const int i = i0 + lane;
      const double w = i < w1 ? weight_of(row[i], best.v, inv_t) : 0.0;
      double incl = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const double v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      const unsigned hit = __ballot_sync(0xffffffffu, w > 0.0 && target < cum + incl);
      if (hit) {
        if (lane == 0) found = i0 + __ffs(hit) - 1;
        break;
      }
      cum += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = found >= 0 ? found : best.i;
}

// out[r] = a draw from softmax(logits[r] / temperature) with the splitmix64 state
// states[state_index[r]], which advances by one draw.
MB_EXPORT int mb_sample(const float* logits, long long stride, int rows, int V,
                        double temperature, const int* state_index, unsigned long long* states,
                        int* out, void* stream) {
  if (rows <= 0) return 0;
  if (V <= 0) MB_FAIL("mb_sample: a vocabulary of %d", V);
  if (!(temperature >= 1e-30)) MB_FAIL("mb_sample: a temperature of %g is greedy", temperature);
  if (V >= 16384 && rows <= 8192) {  // a wide row: a cluster of CTAs shares it
    mb_launch_clusters(sample_cluster_kernel, dim3(rows * SAMPLE_CTAS), dim3(SAMPLE_CL_THREADS), 0,
                       (cudaStream_t)stream, SAMPLE_CTAS, logits, (size_t)stride, V,
                       1.0 / temperature, state_index, states, out);
    MB_CHECK_LAUNCH("mb_sample");
  }
  mb_launch(sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, 
      logits, (size_t)stride, V, 1.0 / temperature, state_index, states, out);
  MB_CHECK_LAUNCH("mb_sample");
}

// ------------------------------------------------------------------ top-k, top-p, min-p
// The reference's filters (src/infer/mormot.ai.infer.sampler.pas:343-436 of the reference
// project), in its order: the candidates are the tokens at or above a threshold that is
// lowered until it holds all that the filters can keep; they are sorted by logit (higher
// first, lower id on a tie); top-k keeps k and every token tied with the k-th; top-p keeps the
// shortest prefix reaching top_p of the mass that top-k kept; min-p keeps tokens at least
// min_p times as probable as the best; then one draw from what is left.
// `scratch` holds one 64-bit key per candidate: [rows][scratch_stride], scratch_stride a power
// of two >= V. A key orders as the reference ranks: ~(logit as ordered integer) in the upper
// half, the id in the lower half, ascending.
__device__ __forceinline__ unsigned ordered_bits(float v) {
  unsigned b = __float_as_uint(v);
  if ((b << 1) == 0) b = 0;  // -0 as +0
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ double block_sum_double(double v, double* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += sh[w];  // in warp order
    sh[32] = t;
  }
  __syncthreads();
  const double r = sh[32];
  __syncthreads();
  return r;
}

// By a whole block: the sum of w[0 .. n) when `total_only`, else the first index whose running
// sum (in index order) reaches `target` (strict: exceeds it), left in *found (n if none).
// Every thread sums a contiguous run, one thread adds the runs up in order, the thread whose
// run holds the target walks it. `runs` holds SAMPLE_THREADS doubles.
__device__ double block_walk(const double* __restrict__ w, int n, double target, bool strict,
                             bool total_only, double* runs, int* found) {
  const int per = (n + blockDim.x - 1) / blockDim.x;
  const int i0 = min(n, (int)threadIdx.x * per), i1 = min(n, i0 + per);
  double mine = 0.0;
  for (int i = i0; i < i1; ++i) mine += w[i];
  runs[threadIdx.x] = mine;
  if (threadIdx.x == 0) *found = n;
  __syncthreads();
  __shared__ double total_sh;
  if (threadIdx.x == 0) {
    double total = 0.0;
    for (int t = 0; t < (int)blockDim.x; ++t) {
      const double v = runs[t];
      runs[t] = total;
      total += v;
    }
    total_sh = total;
  }
  __syncthreads();
  const double total = total_sh;
  if (!total_only) {
    const double before = runs[threadIdx.x];
    const bool here = strict ? (target >= before && target < before + mine)
                             : (target > before && target <= before + mine);
    if (here) {
      double cum = before;
      for (int i = i0; i < i1; ++i) {
        cum += w[i];
        if (strict ? target < cum : cum >= target) {
          atomicMin(found, i);
          break;
        }
      }
    }
  }
  __syncthreads();
  return total;
}

// The search for the candidates' threshold (on the exponent: log of the weight relative to the
// best). It starts at log(1e-3) and goes down until the candidates are enough for the filters
// (k of them, or top_p of the mass); if they are far more than needed (a flat distribution) it
// goes up again by bisection between a threshold that gave enough and one that did not, since
// the sort that follows grows with their number. It ends right after a pass at the threshold it
// keeps. `may_raise` is off when the threshold itself is the filter (min-p alone).
struct ThreshSearch {
  double log_t, ok, bad;
  bool have_ok, finish_next;
};
__device__ __forceinline__ void thresh_start(ThreshSearch& s, double t) {
  s.log_t = t > 0.0 ? log(t) : -INFINITY;
  s.ok = 0.0;
  s.bad = 0.0;  // a threshold above the best weight keeps nothing
  s.have_ok = false;
  s.finish_next = false;
}
// after a pass at s.log_t that found n candidates (enough or not): true when the search is over
__device__ __forceinline__ bool thresh_step(ThreshSearch& s, bool enough, int n, int cap,
                                            int round, bool may_raise) {
  if (enough) {
    if (!may_raise || s.finish_next || n <= cap || round >= 20) return true;
    s.ok = s.log_t;
    s.have_ok = true;
    const double mid = 0.5 * (s.ok + s.bad);
    if (!(mid > s.ok && mid < s.bad)) return true;
    s.log_t = mid;
    return false;
  }
  if (s.log_t == -INFINITY) return true;  // every finite token is a candidate already
  s.bad = s.log_t;
  if (!s.have_ok) {  // still on the way down
    s.log_t += round < 6 ? -2.302585092994046 : -6.907755278982137;
    if (s.log_t < -690.0) s.log_t = -INFINITY;
    return false;
  }
  const double mid = 0.5 * (s.ok + s.bad);
  if (round >= 20 || !(mid > s.ok && mid < s.bad)) {
    s.log_t = s.ok;  // one more pass at the threshold that is known to be enough
    s.finish_next = true;
  } else {
    s.log_t = mid;
  }
  return false;
}

// The n candidate keys in `keys` sorted ascending (padded to the next power of two with the
// largest key), by one block (PARTS = 1) or by the PARTS CTAs of a cluster, of which this is
// number `part`: every CTA takes every PARTS-th chunk and a PARTS-th of each far step, and they
// meet at the cluster's barrier after each step. Bitonic: steps whose partners lie within
// SORT_CHUNK keys of each other run in shared memory, a chunk at a time and as many steps in a
// row as stay inside the chunk; only the far steps of the upper levels go through global memory.
template <int PARTS>
__device__ void sort_candidates(unsigned long long* __restrict__ keys, int n, int part) {
  __shared__ unsigned long long chunk[SORT_CHUNK];
  auto meet = [&]() {
    if (PARTS == 1) {
      __syncthreads();
    } else {
      __threadfence();
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
  };
  int np = 1;
  while (np < n) np <<= 1;
  for (int i = n + part * blockDim.x + threadIdx.x; i < np; i += PARTS * blockDim.x)
    keys[i] = ~0ull;
  meet();
  const int cn = np < SORT_CHUNK ? np : SORT_CHUNK;
  // levels k_lo .. k_hi of chunk-local steps (all steps of a level when k <= cn, else the last
  // ones, j <= cn / 2) for this CTA's chunks
  auto local_levels = [&](int k_lo, int k_hi) {
    for (int base = part * cn; base < np; base += PARTS * cn) {
      for (int i = threadIdx.x; i < cn; i += blockDim.x) chunk[i] = keys[base + i];
      __syncthreads();
      for (int k = k_lo; k <= k_hi; k <<= 1) {
        for (int j = (k >> 1) < cn ? (k >> 1) : (cn >> 1); j > 0; j >>= 1) {
          for (int i = threadIdx.x; i < cn; i += blockDim.x) {
            const int l = i ^ j;
            if (l > i) {
              const unsigned long long a = chunk[i], b = chunk[l];
              const bool up = ((base + i) & k) == 0;
              if ((a > b) == up) { chunk[i] = b; chunk[l] = a; }
            }
          }
          __syncthreads();
        }
      }
      for (int i = threadIdx.x; i < cn; i += blockDim.x) keys[base + i] = chunk[i];
      __syncthreads();
    }
    meet();
  };
  local_levels(2, cn);
  for (int k = 2 * cn; k <= np; k <<= 1) {
    for (int j = k >> 1; j >= cn; j >>= 1) {
      for (int i = part * blockDim.x + threadIdx.x; i < np; i += PARTS * blockDim.x) {
        const int l = i ^ j;
        if (l > i) {
          const unsigned long long a = keys[i], b = keys[l];
          const bool up = (i & k) == 0;
          if ((a > b) == up) { keys[i] = b; keys[l] = a; }
        }
      }
      meet();
    }
    local_levels(k, k);
  }
}

// The end of a filtered draw, by one whole block: `n` candidate keys lie sorted in `keys`. They
// are cut by top-k, top-p and min-p in the reference's order, and one token is drawn from what
// is left with the stream `state`; *result receives it.
__device__ void filtered_finish(const float* __restrict__ row, const Best best, double inv_t,
                                int top_k, double top_p, double min_p, double sum,
                                unsigned long long* __restrict__ keys, size_t scratch_stride,
                                int n, unsigned long long* __restrict__ state,
                                int* __restrict__ result) {
  __shared__ double dsh[33];
  __shared__ int count_sh;
  __shared__ int result_sh;
  __shared__ double wsum[SAMPLE_THREADS];
  int np = 1;
  while (np < n) np <<= 1;
  // The candidates' weights in sorted order, once, next to the keys (there is room unless more
  // than half of the vocabulary is a candidate: then one thread walks them as they are).
  double* wts = 2 * (size_t)np <= scratch_stride ? (double*)(keys + np) : nullptr;
  if (wts) {
    for (int c = threadIdx.x; c < n; c += blockDim.x)
      wts[c] = weight_of(row[(int)(keys[c] & 0xffffffffull)], best.v, inv_t);
    __syncthreads();
    auto id_of = [&](int c) { return (int)(keys[c] & 0xffffffffull); };
    if (top_k > 0 && n > top_k) {
      if (threadIdx.x == 0) {
        int keep = top_k;
        const float kth = row[id_of(top_k - 1)];
        while (keep < n && row[id_of(keep)] == kth) ++keep;
        count_sh = keep;
      }
      __syncthreads();
      n = count_sh;
      __syncthreads();
    }
    if (top_p < 1.0) {
      const double mass = top_k > 0 ? block_walk(wts, n, 0.0, false, true, wsum, &count_sh) : sum;
      block_walk(wts, n, top_p * mass, false, false, wsum, &count_sh);
      n = min(n, count_sh + 1);
      __syncthreads();
    }
    if (min_p > 0.0) {
      // sorted by logit, so the weights do not rise: the first one below the bound ends the list
      if (threadIdx.x == 0) count_sh = n;
      __syncthreads();
      const double bound = min_p * wts[0];
      int first = n;
      for (int c = 1 + threadIdx.x; c < n; c += blockDim.x)
        if (!(wts[c] >= bound)) { first = c; break; }
      if (first < n) atomicMin(&count_sh, first);
      __syncthreads();
      n = count_sh;
      __syncthreads();
    }
    const double kept = block_walk(wts, n, 0.0, false, true, wsum, &count_sh);
    if (threadIdx.x == 0) {
      unsigned long long* st = state;
      unsigned long long z = (*st += 0x9E3779B97F4A7C15ull);
      z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
      z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
      z = z ^ (z >> 31);
      dsh[0] = (double)(z >> 11) * (1.0 / 9007199254740992.0) * kept;
    }
    __syncthreads();
    const double u = dsh[0];
    __syncthreads();
    block_walk(wts, n, u, true, false, wsum, &count_sh);
    if (threadIdx.x == 0) result_sh = id_of(count_sh < n ? count_sh : 0);
  } else
  if (threadIdx.x == 0) {
    auto id_of = [&](int c) { return (int)(keys[c] & 0xffffffffull); };
    auto w_of = [&](int c) { return weight_of(row[id_of(c)], best.v, inv_t); };
    if (top_k > 0 && n > top_k) {
      int keep = top_k;
      const float kth = row[id_of(top_k - 1)];
      while (keep < n && row[id_of(keep)] == kth) ++keep;
      n = keep;
    }
    if (top_p < 1.0) {
      double mass = sum;
      if (top_k > 0) {
        mass = 0.0;
        for (int c = 0; c < n; ++c) mass += w_of(c);
      }
      double cum = 0.0;
      int keep = n;
      for (int c = 0; c < n; ++c) {
        cum += w_of(c);
        if (cum >= top_p * mass) { keep = c + 1; break; }
      }
      n = keep;
    }
    if (min_p > 0.0) {
      int keep = 1;
      const double w0 = w_of(0);
      while (keep < n && w_of(keep) >= min_p * w0) ++keep;
      n = keep;
    }
    double kept = 0.0;
    for (int c = 0; c < n; ++c) kept += w_of(c);
    unsigned long long* st = state;
    unsigned long long z = (*st += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    const double u = (double)(z >> 11) * (1.0 / 9007199254740992.0) * kept;
    int pick = id_of(0);
    double cum = 0.0;
    for (int c = 0; c < n; ++c) {
      cum += w_of(c);
      if (u < cum) { pick = id_of(c); break; }
    }
    result_sh = pick;
  }
  __syncthreads();
  if (threadIdx.x == 0) *result = result_sh;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_filtered_kernel(const float* __restrict__ logits, size_t stride, int V, double inv_t,
                       int top_k, double top_p, double min_p,
                       const int* __restrict__ state_index, unsigned long long* __restrict__ states,
                       unsigned long long* __restrict__ scratch, size_t scratch_stride,
                       int* __restrict__ out) {
  mb_grid_wait();
  mb_grid_launch_next();
  __shared__ Best sh[32];
  __shared__ double dsh[33];
  __shared__ int count_sh;
  const float* row = logits + blockIdx.x * stride;
  unsigned long long* keys = scratch + blockIdx.x * scratch_stride;
  const Best best = block_argmax(row, V, sh);
  if ((__float_as_uint(best.v) & 0x7f800000u) == 0x7f800000u) {
    if (threadIdx.x == 0) out[blockIdx.x] = best.i;
    return;
  }
  // the sum of all weights (relative to the best one, which weighs 1) is needed only for a
  // top-p over the whole vocabulary: p_i = w_i / sum
  const bool whole_mass = top_p < 1.0 && top_k == 0;
  double sum = 0.0;
  if (whole_mass) {
    double mine = 0.0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mine += weight_of(row[i], best.v, inv_t);
    sum = block_sum_double(mine, dsh);
  }
  // A token is a candidate when its weight is at least the threshold, tested on the exponent
  // (no exp for the many that fail).
  ThreshSearch ts;
  thresh_start(ts, (top_k > 0 || top_p < 1.0) ? 1e-3 : min_p);
  const bool may_raise = top_k > 0 || top_p < 1.0;
  const int cap = top_k > 0 ? max(2 * top_k, 1024) : 4096;
  int n = 0;
  for (int round = 0;; ++round) {
    const double log_t = ts.log_t;
    int cnt = 0;
    double above = 0.0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = row[i];
      const bool finite = (__float_as_uint(v) & 0x7f800000u) != 0x7f800000u;
      const double x = ((double)v - (double)best.v) * inv_t;
      if (finite && x >= log_t) {
        ++cnt;
        if (whole_mass) above += exp(x);
      }
    }
    if (whole_mass) above = block_sum_double(above, dsh);
    n = (int)(block_sum_double((double)cnt, dsh) + 0.5);
    bool enough = true;
    if (top_k > 0) enough = n >= top_k;
    else if (top_p < 1.0) enough = above >= top_p * sum;
    if (thresh_step(ts, enough, n, cap, round, may_raise)) break;
  }
  const double log_t = ts.log_t;
  // gather the candidates' keys, pad to a power of two with the largest key
  if (threadIdx.x == 0) count_sh = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    const bool finite = (__float_as_uint(v) & 0x7f800000u) != 0x7f800000u;
    if (finite && ((double)v - (double)best.v) * inv_t >= log_t) {
      const int at = atomicAdd(&count_sh, 1);
      keys[at] = ((unsigned long long)(~ordered_bits(row[i])) << 32) | (unsigned)i;
    }
  }
  __syncthreads();
  n = count_sh;
  sort_candidates<1>(keys, n, 0);
  filtered_finish(row, best, inv_t, top_k, top_p, min_p, sum, keys, scratch_stride, n,
                  states + state_index[blockIdx.x], out + blockIdx.x);
}

// The filtered draw over a wide row: the passes over the vocabulary (best value, sum, counting
// and gathering the candidates) are shared by a cluster of SAMPLE_CTAS CTAs that exchange their
// counts and sums through each other's shared memory; the first CTA then sorts, filters and
// draws as above. Every CTA takes the same decisions from the same exchanged numbers.
__global__ void __launch_bounds__(SAMPLE_CL_THREADS)
sample_filtered_cluster_kernel(const float* __restrict__ logits, size_t stride, int V,
                               double inv_t, int top_k, double top_p, double min_p,
                               const int* __restrict__ state_index,
                               unsigned long long* __restrict__ states,
                               unsigned long long* __restrict__ scratch, size_t scratch_stride,
                               int* __restrict__ out) {
  mb_grid_wait();
  mb_grid_launch_next();
  __shared__ Best sh[32];
  __shared__ double dsh[33];
  __shared__ __align__(8) unsigned long long mine_best;
  __shared__ __align__(8) unsigned long long mail[2][2];  // [round parity][count, mass bits]
  __shared__ int fill_sh;
  const int r = blockIdx.x / SAMPLE_CTAS;
  const uint32_t rank = smp_cluster_rank();
  const float* row = logits + r * stride;
  unsigned long long* keys = scratch + r * scratch_stride;
  const int share = (V + SAMPLE_CTAS - 1) / SAMPLE_CTAS;
  const int lo = min(V, (int)rank * share), hi = min(V, lo + share);

  Best b = {0.f, -1};
  if (hi > lo) {
    b = block_argmax(row + lo, hi - lo, sh);
    const float v = row[lo + b.i];
    b = Best{v, v != v ? -1 : lo + b.i};
  }
  if (threadIdx.x == 0)
    mine_best = ((unsigned long long)__float_as_uint(b.v) << 32) | (unsigned)b.i;
  smp_cluster_sync();
  Best best = {0.f, -1};
  for (uint32_t k = 0; k < SAMPLE_CTAS; ++k) {
    const unsigned long long x = smp_peer_u64(smp_smem_u32(&mine_best), k);
    const Best c = {__uint_as_float((unsigned)(x >> 32)), (int)(unsigned)x};
    if (better(c, best)) best = c;
  }
  if (best.i < 0) best.i = 0;  // all NaN
  if ((__float_as_uint(best.v) & 0x7f800000u) == 0x7f800000u) {
    if (rank == 0 && threadIdx.x == 0) out[r] = best.i;
    smp_cluster_sync();  // no CTA leaves while another may still read its shared memory
    return;              // the same for the whole cluster
  }
  // one exchange: every CTA leaves (count, mass) in the mailbox of this round's parity and
  // reads all eight; the next round uses the other mailbox, so one barrier a round is enough
  int round_no = 0;
  int my_before = 0;  // candidates in the shares before this one (of the last exchange)
  auto exchange = [&](int cnt, double mass, int& cnt_all, double& mass_all) {
    const int par = round_no & 1;
    ++round_no;
    if (threadIdx.x == 0) {
      mail[par][0] = (unsigned long long)(unsigned)cnt;
      mail[par][1] = (unsigned long long)__double_as_longlong(mass);
    }
    smp_cluster_sync();
    cnt_all = 0;
    mass_all = 0.0;
    my_before = 0;
    for (uint32_t k = 0; k < SAMPLE_CTAS; ++k) {
      const int c = (int)smp_peer_u64(smp_smem_u32(&mail[par][0]), k);
      const double m = __longlong_as_double((long long)smp_peer_u64(smp_smem_u32(&mail[par][1]), k));
      if (k < rank) my_before += c;
      cnt_all += c;
      mass_all += m;
    }
  };
  const bool whole_mass = top_p < 1.0 && top_k == 0;
  double sum = 0.0;
  if (whole_mass) {
    double mine = 0.0;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) mine += weight_of(row[i], best.v, inv_t);
    mine = block_sum_double(mine, dsh);
    int unused;
    exchange(0, mine, unused, sum);
  }
  ThreshSearch ts;
  thresh_start(ts, (top_k > 0 || top_p < 1.0) ? 1e-3 : min_p);
  const bool may_raise = top_k > 0 || top_p < 1.0;
  const int cap = top_k > 0 ? max(2 * top_k, 1024) : 4096;
  int n = 0;
  for (int round = 0;; ++round) {
    const double log_t = ts.log_t;
    int cnt = 0;
    double above = 0.0;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const float v = row[i];
      const bool finite = (__float_as_uint(v) & 0x7f800000u) != 0x7f800000u;
      const double x = ((double)v - (double)best.v) * inv_t;
      if (finite && x >= log_t) {
        ++cnt;
        if (whole_mass) above += exp(x);
      }
    }
    if (whole_mass) above = block_sum_double(above, dsh);
    cnt = (int)(block_sum_double((double)cnt, dsh) + 0.5);
    double above_all;
    exchange(cnt, above, n, above_all);
    bool enough = true;
    if (top_k > 0) enough = n >= top_k;
    else if (top_p < 1.0) enough = above_all >= top_p * sum;
    if (thresh_step(ts, enough, n, cap, round, may_raise)) break;
  }
  const double log_t = ts.log_t;
  // every share's candidates go behind those of the shares before it
  if (threadIdx.x == 0) fill_sh = 0;
  __syncthreads();
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = row[i];
    const bool finite = (__float_as_uint(v) & 0x7f800000u) != 0x7f800000u;
    if (finite && ((double)v - (double)best.v) * inv_t >= log_t) {
      const int at = my_before + atomicAdd(&fill_sh, 1);
      keys[at] = ((unsigned long long)(~ordered_bits(v)) << 32) | (unsigned)i;
    }
  }
  __threadfence();
  smp_cluster_sync();  // all keys are written (and nobody reads a mailbox any more)
  sort_candidates<SAMPLE_CTAS>(keys, n, (int)rank);  // ends at the cluster's barrier
  if (rank != 0) return;
  filtered_finish(row, best, inv_t, top_k, top_p, min_p, sum, keys, scratch_stride, n,
                  states + state_index[r], out + r);
}

// Like mb_sample, with top_k (0: off), top_p (1: off) and min_p (0: off). `scratch`:
// rows * scratch_stride 64-bit words, scratch_stride a power of two >= V.
MB_EXPORT int mb_sample_filtered(const float* logits, long long stride, int rows, int V,
                                 double temperature, int top_k, double top_p, double min_p,
                                 const int* state_index, unsigned long long* states,
                                 unsigned long long* scratch, long long scratch_stride, int* out,
                                 void* stream) {
  if (rows <= 0) return 0;
  if (V <= 0) MB_FAIL("mb_sample_filtered: a vocabulary of %d", V);
  if (!(temperature >= 1e-30)) MB_FAIL("mb_sample_filtered: a temperature of %g is greedy", temperature);
  if (top_k < 0 || !(top_p > 0.0 && top_p <= 1.0) || !(min_p >= 0.0 && min_p < 1.0))
    MB_FAIL("mb_sample_filtered: top_k %d, top_p %g, min_p %g", top_k, top_p, min_p);
  if (scratch_stride < V || (scratch_stride & (scratch_stride - 1)))
    MB_FAIL("mb_sample_filtered: a scratch row of %lld words for %d tokens", scratch_stride, V);
  if (V >= 16384 && rows <= 8192) {  // a wide row: a cluster of CTAs shares the passes over it
    mb_launch_clusters(sample_filtered_cluster_kernel, dim3(rows * SAMPLE_CTAS),
                       dim3(SAMPLE_CL_THREADS), 0, (cudaStream_t)stream, SAMPLE_CTAS, logits,
                       (size_t)stride, V, 1.0 / temperature, top_k, top_p, min_p, state_index,
                       states, scratch, (size_t)scratch_stride, out);
    MB_CHECK_LAUNCH("mb_sample_filtered");
  }
  mb_launch(sample_filtered_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, 
      logits, (size_t)stride, V, 1.0 / temperature, top_k, top_p, min_p, state_index, states,
      scratch, (size_t)scratch_stride, out);
  MB_CHECK_LAUNCH("mb_sample_filtered");
}
