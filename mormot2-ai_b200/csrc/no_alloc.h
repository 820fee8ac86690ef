/* An entry point of this library that allocates nothing. It has no counterpart in the
 * reference project (whose engine sizes and allocates its device buffers itself); it exists
 * for hosts that call these kernels but may not, or cannot, ask CUDA for memory:
 *
 *   - a host that has handed the whole device memory to an arena of its own at start-up and
 *     has nothing left for cudaMalloc to give;
 *   - a host with a fixed memory budget that is reviewed before deployment (every byte of
 *     device memory accounted for up front), where a library call that allocates is a defect;
 *   - a binding from another language that wraps kernel launches only and has no way to hand a
 *     scratch buffer of its own to the library.
 *
 * All other entry points of the library take their scratch memory from the caller
 * (mb_attention_decode, mb_gemm_tc, mb_sample_filtered); this one brings its own.
 */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

/* The most float32 values of scratch that mb_attention_decode_static can use: 4 Mi values,
 * 16 MiB. The array lives in the library's image: every GPU on which the library is loaded
 * holds these 16 MiB from the load until the process exits, whether the function is called or
 * not. */
#define MB_ATTENTION_DECODE_STATIC_FLOATS (4ll * 1024 * 1024)

/* mb_attention_decode (attention of single tokens over the paged cache, the pages of a
 * sequence shared out over `splits` CTAs) with the partial results of the splits kept in a
 * scratch array that is part of the library instead of a buffer from the caller. Inputs and
 * outputs are the caller's, exactly as for mb_attention_decode; the result is the same.
 *
 * It calls no cudaMalloc, cudaFree or any routine that allocates.
 *
 * Limit: tokens * heads * splits * (head_dim + 2) must not exceed
 * MB_ATTENTION_DECODE_STATIC_FLOATS; a larger call is refused (-1, the reason in
 * mb_last_error()) and nothing is launched. With 32 heads of 128 values that is, for
 * instance, 64 tokens with 15 splits, or 8 tokens with 126 splits.
 *
 * The first call on a device looks up the device address of the scratch array (once per
 * device, with that device current). Make this first call before any stream capture begins.
 *
 * Every call on a device uses the same array. Nothing in it has to start at zero: each call
 * writes every value that it later reads, so what the call before left there does not
 * matter. But two calls that run on the GPU at the same time (on two streams, or from two
 * threads) write the same memory and race: keep the calls of one device in one stream, or
 * order them yourself.
 *
 * `error`, as for mb_attention_decode, is a device word of the caller's (it may be null) that
 * receives a code if a bounded wait inside the kernel runs out.
 *
 * Returns 0 after the launch, -1 on refusal. */
int mb_attention_decode_static(const void* q, int q_stride, void* out, int out_stride,
                               const void* kpool, const void* vpool, const int* page_table,
                               int max_pages, int ring_pages, const int* tok_slot,
                               const int* tok_pos, int T, int nh, int nkv,
                               int hd, int window, float scale, int splits, int* error,
                               void* stream);

#ifdef __cplusplus
}
#endif
