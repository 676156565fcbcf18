/* roost_b200 kernel library: the C ABI.
 *
 * Every entry point is a plain C function that takes device pointers, sizes and a CUDA stream, launches on
 * that stream and returns a status; nothing here allocates device memory or synchronises. The reference puts
 * its kernels behind a versioned C ABI with status codes and per-op entry points
 * (kernels/include/roost_kernels.h:55-72,107-164,244-262); this is the same boundary with this engine's own
 * op set. A caller checks roost_abi_version() first.
 *
 * dtype codes: 0 = float32, 1 = bfloat16. All index tables are int32. Matrices are row-major.
 */
#ifndef ROOST_B200_KERNELS_H
#define ROOST_B200_KERNELS_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ROOST_ABI_VERSION 11

#define ROOST_OK 0
#define ROOST_ERR_INVALID 1      /* an argument is out of range or inconsistent; nothing was launched */
#define ROOST_ERR_UNSUPPORTED 2  /* the sizes are valid but no kernel serves them; nothing was launched */
#define ROOST_ERR_CUDA 3         /* the CUDA runtime reported an error at launch */

#define ROOST_F32 0
#define ROOST_BF16 1

typedef void* roost_stream_t;

int roost_abi_version(void);
/* Programmatic dependent launch for the library's kernels (off by default): a kernel may start its preamble, and the
 * weight-streaming product its first loads of weights, while the kernel before it on the stream is finishing.
 * With it on, a kernel reads before it waits for the kernel in front: weights (norm weights, the products' weight
 * matrices), index tables (the `rows` of the norms, the work lists of the attention kernels, q_indptr, kv_lens,
 * kv_indptr, kv_indices) and pages of the cache that hold only tokens of earlier steps. A caller must therefore not
 * have those written by the kernel launched directly before the call that reads them (a copy in between is enough);
 * activations and the pages of the step's own tokens are read after the wait. */
void roost_set_pdl(int on);
/* Message of the last non-OK status on this thread. */
const char* roost_last_error(void);

/* Writes, in stream order and without synchronising, the error words of the kernels that wait with a limit into
 * out[0..2] (the tcgen05 products, the decode attention, the tcgen05 prefill attention; 0: no wait was given up since
 * the words were last cleared by roost_gemm_tcgen05_status() / roost_attention_status()) and 1 into out[3]. out is
 * device memory, or with out_is_host page-locked host memory (refused when the device cannot write it): a caller that
 * copies a step's results to the host anyway learns of a given-up wait with them, at no extra synchronisation. */
int roost_status_snapshot(int32_t* out, int out_is_host, roost_stream_t stream);

/* out[t,:] = table[ids[t],:]; an id outside [0, vocab) gives a zero row. */
int roost_embedding(const void* table, const int32_t* ids, void* out, int tokens, int hidden, int vocab, int dtype,
                    roost_stream_t stream);

/* out[i,:] = x[r,:] / sqrt(mean(x[r,:]^2) + eps) * w, r = rows ? rows[i] : i. w has dtype wdtype. */
int roost_rms_norm(const void* x, const void* w, void* out, const int32_t* rows, int n_out, int hidden, float eps,
                   int dtype, int wdtype, roost_stream_t stream);

/* s = residual[r,:] + x[r,:] rounded to dtype; out[i,:] = rms_norm(s). Without rows, residual[r,:] = s is
 * written back (the running residual stream); with rows the residual is left as it is. */
int roost_add_rms_norm(const void* x, void* residual, const void* w, void* out, const int32_t* rows, int n_out,
                       int hidden, float eps, int dtype, int wdtype, roost_stream_t stream);

/* out[t,i] = silu(gate_i) * up_i, x: [tokens, 2*inter]. block 0: a row of x is [gate | up]; block b > 0: blocks of b gate
 * values followed by their b up values (the layout the fused product below wants its weight rows in). */
int roost_silu_mul(const void* x, void* out, int tokens, int inter, int block, int dtype, roost_stream_t stream);

/* Per token and head: optional RMS norm over head_dim (q heads with q_w, k heads with k_w), NeoX rotation of
 * the first rotary_dim elements by angle position * inv_freq[i] (inv_freq: double[rotary_dim/2]; rotary_dim 0
 * = no rotation), then q to q_out[t, h, :], k and v into their page slot:
 * pool[(page * kv_heads + h) * page_size + offset][:] with slot = page * page_size + offset from slot_mapping
 * (a negative slot is skipped). qkv rows hold [q heads | k heads | v heads] with row stride qkv_stride
 * elements; with write_kv 0 only the q part is read. cos_sin: null, or the table roost_rope_table made for these
 * positions and this inv_freq (tokens x rotary_dim/2 pairs). */
int roost_qk_norm_rope_cache(const void* qkv, int64_t qkv_stride, void* q_out, void* k_pool, void* v_pool,
                             const void* q_w, const void* k_w, const double* inv_freq, const int32_t* positions,
                             const int32_t* slot_mapping, const float* cos_sin, int tokens, int q_heads, int kv_heads,
                             int head_dim, int rotary_dim, float eps, int page_size, int64_t pool_pages, int write_kv,
                             int dtype, int wdtype, roost_stream_t stream);

/* The cosines and sines of a step's rotations: cos_sin[(t * half + i) * 2 + {0, 1}] = (cos, sin)(positions[t] * inv_freq[i])
 * for i < half, the angle formed in 64-bit and reduced to [-pi, pi] before the 32-bit sincosf. They depend on the
 * positions only, so a step computes them once and hands them to roost_qk_norm_rope_cache of every layer (its cos_sin
 * argument; null there computes the same values in place). */
int roost_rope_table(const int32_t* positions, const double* inv_freq, int tokens, int half, float* cos_sin, roost_stream_t stream);

/* Causal grouped-query attention over a paged cache, one query token per block and key/value head; 32-bit
 * arithmetic throughout. Token t belongs to batch row token_row[t] and sits at absolute position
 * positions[t]; it sees keys max(0, pos - window + 1) .. pos (window <= 0: from 0). Row b's pages are
 * kv_indices[kv_indptr[b] ..]; key j lies in page j / page_size. */
int roost_paged_attention_generic(const void* q, void* out, const void* k_pool, const void* v_pool,
                                  const int32_t* positions, const int32_t* token_row, const int32_t* kv_indptr,
                                  const int32_t* kv_indices, int tokens, int q_heads, int kv_heads, int head_dim,
                                  int page_size, float scale, int window, int dtype, roost_stream_t stream);

/* Tensor-core attention for bfloat16 (attention_mma.cu). head_dim must be one roost_attention_mma_supported accepts.
 * q_indptr[b] .. q_indptr[b+1] are row b's tokens, kv_lens[b] its keys after this step.
 * prefill work: int32 pairs (batch row, first packed row of a tile of tile_rows rows; roost_attention_prefill_tile_rows picks 64 or 128),
 * packed row = token * group + head. With 128-row tiles, head size 64 or 128, a power-of-two number of query heads per
 * key/value head, pages of 16, 32, 64, ... rows and K and V in one allocation, prompt portions run the tcgen05 kernel
 * (attention_tc.cu) unless roost_attention_set_prefill_tc(0) was called; q then has `tokens` rows.
 * decode work: int32 quadruples (batch row, first key, one past the last key, partial slot or -1); rows with at most
 * 16 packed rows only; the first key of an item is a multiple of 64. merge_work: quadruples (batch row, first slot,
 * chunks | packed rows << 24, the row's first token) for rows split into several chunks; merge_rows: the most packed
 * rows any of them has.
 * part_o: float[slots * kv_heads * 16 * head_dim], part_ml: float[slots * kv_heads * 16 * 2].
 * pool_pages: pages of k_pool and v_pool; with head size 64 or 128, pages of 8, 16 or a multiple of 32 rows and pools
 * on 128-byte boundaries, decode streams keys and values through the copy engine (TMA) unless
 * roost_attention_set_decode_tma(0) was called; 0 when not known (the cp.async kernel runs). It copies whole pages:
 * every slot of a page a block table names must be readable, whatever it holds.
 * roost_attention_status(): 0, or the code of a wait the copy-engine kernel gave up, or 9 when a work item named a
 * partial slot beyond the workspace of roost_attention_decode_static (read and cleared). */
int roost_attention_mma_supported(int head_dim);
int roost_attention_prefill_tile_rows(int head_dim, int q_heads, int kv_heads, int page_size, long long pool_pages, const void* k_pool,
                                      const void* v_pool, long long packed_rows);
void roost_attention_set_prefill_tc(int on);
int roost_attention_prefill(const void* q, long long tokens, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                            const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work,
                            int items, int tile_rows, int q_heads, int kv_heads, int head_dim, int page_size, long long pool_pages,
                            float scale, int window, roost_stream_t stream);
int roost_attention_decode(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                           const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work,
                           int items, const int32_t* merge_work, int merge_items, int merge_rows, float* part_o, float* part_ml,
                           int q_heads, int kv_heads, int head_dim, int page_size, long long pool_pages, float scale, int window,
                           roost_stream_t stream);
void roost_attention_set_decode_tma(int on);
int roost_attention_status(void);
/* The split decode attention without partial results in memory and without a merge kernel: the grid is thread-block
 * clusters of cluster_chunks (1, 2, 4 or 8) CTAs, one cluster a (row, key/value head). The work list holds exactly
 * cluster_chunks items (batch row, first key, end key, unused) a row, in key order, the row's chunks first and empty
 * items (end key 0) after them; padding rows are cluster_chunks items of batch row -1. CTA r of a cluster takes the
 * row's r-th item and CTA 0 combines the results in that order through distributed shared memory, with the merge
 * kernel's arithmetic: the same bits as roost_attention_decode gives for the same chunks. Served where the copy-engine
 * decode kernel is (roost_attention_decode_cluster_supported). */
int roost_attention_decode_cluster_supported(int head_dim, int page_size, long long pool_pages, int kv_heads, const void* k_pool,
                                             const void* v_pool);
int roost_attention_decode_cluster(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                                   const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work,
                                   int items, int cluster_chunks, int q_heads, int kv_heads, int head_dim, int page_size,
                                   long long pool_pages, float scale, int window, roost_stream_t stream);

/* The split decode attention without a workspace argument. It has no counterpart in the reference: it exists for
 * callers that must not allocate device memory while they run (a host that gave the whole GPU to its own arena at
 * start-up, a loop that may never synchronise the device as cudaMalloc and cudaFree do, a plug-in that may not grow
 * its process's footprint). Same arguments and result as roost_attention_decode, except that the partial results of
 * rows split into several chunks (`slots` of them, as the work lists number them) live in a fixed device array of
 * roost_attention_decode_static_capacity_floats() floats (16 MiB) inside the library, which every process that
 * loads the library holds on each GPU it uses until it exits. It calls no cudaMalloc, cudaFree or other allocating
 * routine. A call whose slots need more than the array holds returns ROOST_ERR_UNSUPPORTED and launches nothing.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device current);
 * make that first call outside any stream capture. All calls share the one array and it keeps what the last call
 * wrote; nothing in it needs clearing, because a call writes every element it later reads. Two calls that overlap
 * on the GPU (different streams, or one stream's call still running when another is launched elsewhere) race on the
 * array: order them on one stream or with events. `slots` must exceed every slot id the work lists name: an item that
 * names a slot at or beyond it is skipped, its output rows stay unwritten and roost_attention_status() returns 9, so that
 * a wrong work list cannot write past the library's array. */
int roost_attention_decode_static_capacity_floats(void);
int roost_attention_decode_static(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                                  const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices,
                                  const int32_t* work, int items, const int32_t* merge_work, int merge_items, int slots,
                                  int q_heads, int kv_heads, int head_dim, int page_size, float scale, int window,
                                  roost_stream_t stream);

/* out[m,n] = sum_k a[m,k] * w[n,k], plain FFMA in 32-bit (no tensor cores, no reduced-precision mode), the
 * sum over k in increasing order for every output, whatever m is. in_dtype/out_dtype: 0 or 1. */
int roost_gemm_simt(const void* a, const void* w, void* out, int m, int n, int k, int64_t lda, int64_t ldw,
                    int64_t ldo, int in_dtype, int out_dtype, roost_stream_t stream);


/* out[m,n] = sum_k a[m,k] * w[n,k], bfloat16 operands, 32-bit accumulation in tensor memory (tcgen05.mma fed by TMA;
 * gemm_tcgen05.cu). k and the row strides must be multiples of 8. out_dtype: 1 bfloat16, 0 float32. Every wait inside
 * the kernel is bounded; roost_gemm_tcgen05_status() returns the code of a wait that was given up since the last call
 * (0: none) and synchronises the device. */
int roost_gemm_tcgen05_supported(int m, int n, int k, int64_t lda, int64_t ldw);
int roost_gemm_tcgen05(const void* a, const void* w, void* out, int m, int n, int k, int64_t lda, int64_t ldw, int64_t ldo,
                       int out_dtype, roost_stream_t stream);
int roost_gemm_tcgen05_status(void);
/* 1 (default): tiles of 256 x 256 on pairs of CTAs (tcgen05 cta_group::2); 0: tiles of 128 x 256 on single CTAs. */
void roost_gemm_tcgen05_set_pairs(int on);
/* The gate/up product with SiLU(gate) * up applied to the accumulator: w [n = 2 * inter, k] with rows in blocks of 128
 * gate rows followed by their 128 up rows; out [m, n / 2] bfloat16. n must be a multiple of 256. */
int roost_gemm_tcgen05_swiglu(const void* a, const void* w, void* out, int m, int n, int k, int64_t lda, int64_t ldw,
                              int64_t ldo, roost_stream_t stream);

/* out[m,n] = sum_k x[m,k] * w[n,k] for 1 <= m <= 64 rows of bfloat16 x: w streamed once by TMA through a persistent
 * CTA per SM, the products on tcgen05 with w's rows as the 128-row operand, the work split into equal contiguous ranges
 * of (128 rows x 64 k) units with a fixed-order fix-up of tiles shared by neighbouring CTAs (gemm_tcgen05.cu).
 * ws: roost_gemm_stream_workspace_floats() floats, flags: roost_gemm_stream_workspace_flags() int32, zero before the first
 * call and left zero by every call. */
int roost_gemm_stream_workspace_floats(void);
int roost_gemm_stream_workspace_flags(void);
int roost_gemm_stream_supported(int m, int n, int k, int64_t ldx, int64_t ldw);
int roost_gemm_stream(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldo,
                      int out_dtype, float* ws, int32_t* flags, roost_stream_t stream);
/* The same product for weights of few 128-row tiles and a long k (an output projection, a down projection): k split
 * over thread-block clusters of up to 8 CTAs, one cluster a tile, the partial sums added up in CTA order through
 * distributed shared memory; no workspace. Supported where roost_gemm_stream is and the tiles are few enough for every
 * cluster to run at once with two CTAs an SM (n up to about 18,900 rows on 148 SMs). */
int roost_gemm_split_supported(int m, int n, int k, int64_t ldx, int64_t ldw);
int roost_gemm_split_preferred(int m, int n, int k, int64_t ldx, int64_t ldw);  /* measured faster than the other products */
int roost_gemm_split(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldo,
                     int out_dtype, roost_stream_t stream);
/* The k-split product with the SwiGLU of the fused product: w's rows in blocks of 256 (128 gate rows, then the 128 up
 * rows of the same outputs), out[m, j] = silu(gate_j) * up_j with n / 2 columns; at most 32 rows of x. */
int roost_gemm_split_swiglu_supported(int m, int n, int k, int64_t ldx, int64_t ldw);
int roost_gemm_split_swiglu(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldo,
                            int out_dtype, roost_stream_t stream);
/* The same with the SwiGLU of the fused product: w's rows in blocks of 256 (128 gate rows, then the 128 up rows of the
 * same outputs), out[m, j] = silu(gate_j) * up_j with n / 2 columns; at most 32 rows of x, n a multiple of 256. */
int roost_gemm_stream_swiglu_supported(int m, int n, int k, int64_t ldx, int64_t ldw);
int roost_gemm_stream_swiglu(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldo,
                             int out_dtype, float* ws, int32_t* flags, roost_stream_t stream);

/* ids[r] = index of the largest logit of row r, ties to the lowest index, NaN never chosen (-1 if none). */
int roost_argmax(const float* logits, int64_t stride, int rows, int vocab, int32_t* ids, roost_stream_t stream);
/* The same result with a row split over `splits` (1 to 32) blocks, for vocabularies that one SM reads too slowly.
 * part_v, part_i: rows * splits entries of scratch; counters: rows words that are zero before the first call (the
 * kernel leaves them zero). */
int roost_argmax_split(const float* logits, int64_t stride, int rows, int vocab, int32_t* ids, int splits, float* part_v,
                       int32_t* part_i, uint32_t* counters, roost_stream_t stream);

/* Temperature / top-k / top-p / min-p sampling with a Philox4x32-10 draw per row; see sampling.cu.
 * workspace: rows * vocab floats. temperature <= 0 is greedy. */
int roost_sample(const float* logits, int64_t stride, int rows, int vocab, const float* temperature,
                 const int32_t* top_k, const float* top_p, const float* min_p, const uint64_t* seeds,
                 const uint64_t* offsets, float* workspace, int32_t* ids, roost_stream_t stream);

/* What the reference's sampler does beside the draw (src/Starlings.Roost.Ops/CpuOps.Sampling.cs:10-46), in its float32 form.
 * roost_sample_penalise: out[r, v] (rows * vocab floats) = logits[r, v] with the repetition, frequency and presence
 * penalties of row r applied for the tokens counted in counts[row_slot[r], :] (int32 [slots, vocab]: the request's output
 * so far) or named by prompt_bits[row_slot[r], :] (bit v % 32 of word v / 32 of (vocab + 31) / 32 words a slot), and
 * then -inf where the token's bit in mask_bits[row_slot[r], :] is 0 (mask_bits may be null: no token is removed); a row
 * with row_slot < 0 is copied. roost_sample_count_tokens: counts[row_slot[r], ids[r]] += 1. roost_sample_prompt_bits: sets
 * the bits of n token ids in one slot's words. roost_sample_logprobs: logprob[r] = log-softmax of the raw logits of row r
 * at ids[r] (-inf for id -1; logprob may be null), and the `top` highest raw logits of the row, ties to the lower index,
 * with their log-softmax (id -1 and -inf where the row has fewer non-NaN logits). */
int roost_sample_penalise(const float* logits, int64_t stride, int rows, int vocab, float* out, const int32_t* counts,
                          const uint32_t* prompt_bits, const uint32_t* mask_bits, const int32_t* row_slot, const float* repetition,
                          const float* presence, const float* frequency, roost_stream_t stream);
int roost_sample_count_tokens(int32_t* counts, int vocab, const int32_t* row_slot, const int32_t* ids, int rows, roost_stream_t stream);
int roost_sample_prompt_bits(uint32_t* bits, const int32_t* ids, int n, int vocab, roost_stream_t stream);
int roost_sample_logprobs(const float* logits, int64_t stride, int rows, int vocab, const int32_t* ids, float* logprob, int top,
                          int32_t* top_ids, float* top_vals, roost_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
