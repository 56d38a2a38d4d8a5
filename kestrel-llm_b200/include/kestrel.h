/* kestrel.h - the C interface of the kestrel-llm_b200 engine.
 *
 * Two shared libraries export it:
 *   libkestrel_host.so  cache manager (kcache_*), scheduler (ksched_*) and the packer of a step's
 *                       description (kbatch_*): plain C++ on the host, no CUDA needed;
 *   libkestrel_cuda.so  the sm_100a kernels (kestrel_<kernel>), the attention dispatcher, the step
 *                       program and the runner behind kestrel_step_raw (kprog_*, krunner_*); it
 *                       links against libkestrel_host.so.
 * The reference's header-level interface is include/model/vllm_safetensors.h:497-670
 * (st_qwen_inference_init, st_qwen_model_forward, st_qwen_model_prefill_batch,
 * st_qwen_model_forward_batch, st_qwen_inference_free); there one state object is one request on
 * the CPU, here one runner serves all live requests of a GPU.
 *
 * Conventions
 *  - Every function is extern "C".  Functions that return int return 0 (or a count, where the
 *    text says so) on success and a negative code on failure; the kernel library keeps the text
 *    of the last failure of the calling thread in kestrel_last_error().
 *  - Kernel entry points take raw device pointers, sizes and a CUDA stream, launch on that
 *    stream and do not synchronise.  Storage type codes: 0 = float32, 1 = bfloat16.
 *  - This file is included by every source file that defines one of these symbols, so a
 *    definition that drifts from its declaration does not compile; the Python bindings take
 *    their argument types from this file too (csrc/cdecl.py).  Keep one declaration per
 *    statement, with parameter names, in the plain types used below.
 */
#ifndef KESTREL_H
#define KESTREL_H

#ifdef __cplusplus
#define KESTREL_API extern "C" __attribute__((visibility("default")))
#else
#define KESTREL_API __attribute__((visibility("default")))
#endif

/* a CUDA stream (cudaStream_t is this same pointer type) */
typedef struct CUstream_st *kestrel_stream_t;

#define KESTREL_F32 0
#define KESTREL_BF16 1

/* ============================================================================================
 * Cache manager (libkestrel_host.so): pages of keys and values per group of layers, a block
 * table per request and group, one state slot per live request.  Host bookkeeping only.
 * ========================================================================================== */
KESTREL_API void *kcache_create(int n_groups, const int *windows, const int *num_pages, int page_size, int max_requests, int max_blocks_per_request);
KESTREL_API void kcache_destroy(void *h);
/* a windowed group also keeps the pages of its requests' first `keep_first` tokens (call before any request is admitted); 0 done, -6 no such group */
KESTREL_API int kcache_set_keep_first(void *h, int group, int keep_first);
/* slot of the new request; -1 no slot free; -2 the id is live already */
KESTREL_API int kcache_admit(void *h, long long id);
/* 1 if kcache_reserve(id, n_new) would succeed, 0 if pages are short, negative on misuse */
KESTREL_API int kcache_can_reserve(void *h, long long id, int n_new);
/* pages for positions [length, length + n_new) in every group: 0 done, -1 pages short (nothing changed), -3 unknown request, -4 longer than the block table */
KESTREL_API int kcache_reserve(void *h, long long id, int n_new);
/* length += n_new (must be reserved); windowed groups give back pages no later query can reach */
KESTREL_API int kcache_commit(void *h, long long id, int n_new);
/* gives back everything the request holds, and its slot */
KESTREL_API int kcache_release(void *h, long long id);
KESTREL_API int kcache_length(void *h, long long id);
KESTREL_API int kcache_slot(void *h, long long id);
KESTREL_API int kcache_num_blocks(void *h, long long id, int group);
KESTREL_API int kcache_block_table(void *h, long long id, int group, int *out, int n);
KESTREL_API int kcache_describe_decode(void *h, const long long *ids, int n, int B, int W, int *pos, int *kv, int *slot, int *tables, int *bad);
KESTREL_API int kcache_free_pages(void *h, int group);
KESTREL_API int kcache_num_pages(void *h, int group);
KESTREL_API int kcache_num_groups(void *h);
KESTREL_API int kcache_page_size(void *h);
KESTREL_API int kcache_max_blocks(void *h);
KESTREL_API int kcache_live_requests(void *h);
KESTREL_API int kcache_free_slots(void *h);
KESTREL_API long long kcache_pages_handed_out(void *h);
KESTREL_API long long kcache_pages_given_back(void *h);
/* ids of the requests admitted since the last call (their state slots are to be cleared); returns how many there were */
KESTREL_API int kcache_take_admitted(void *h, long long *ids, int *slots, int cap);
/* puts the free pages of every group into a pseudo-random order fixed by `seed` (the layout a pool has after long serving) */
KESTREL_API int kcache_shuffle_free(void *h, long long seed);
/* 0 if every page and slot is free exactly once or held exactly once, else a negative code naming the broken invariant */
KESTREL_API int kcache_check(void *h);

/* ============================================================================================
 * Scheduler (libkestrel_host.so): admission, token budget, prompt portions, decode first,
 * preempt-youngest-and-recompute when pages run out.  It counts tokens; values live with the caller.
 * ========================================================================================== */
KESTREL_API void *ksched_create(void *cache, int max_step_tokens, int prefill_chunk, int batch_max, int max_queued, int max_model_len);
KESTREL_API void ksched_destroy(void *h);
/* 0 queued; -1 waiting queue full; -2 longer than max_model_len or the whole pool; -3 empty prompt or duplicate id */
KESTREL_API int ksched_add(void *h, long long id, int prompt_len, int max_new_tokens);
/* builds the next step, pages reserved: entry e runs tokens [starts[e], starts[e] + counts[e]) of ids[e]; wants[e] = 1 if it ends with the request's last known token.  Returns the number of entries. */
KESTREL_API int ksched_schedule(void *h, long long *ids_out, int *starts_out, int *counts_out, int *wants_out, int cap);
KESTREL_API int ksched_preempted(void *h, long long *out, int cap);
KESTREL_API int ksched_step_done(void *h);
/* one more token of the request is known; 1 if it has reached its token limit */
KESTREL_API int ksched_on_token(void *h, long long id);
KESTREL_API int ksched_finish(void *h, long long id);
KESTREL_API int ksched_num_running(void *h);
KESTREL_API int ksched_num_waiting(void *h);
KESTREL_API long long ksched_num_preemptions(void *h);
KESTREL_API int ksched_known(void *h, long long id);

/* ============================================================================================
 * The description of one step (libkestrel_host.so).  A step runs T tokens of n requests: prompt
 * portions beside single decoded tokens.  kbatch_pack writes everything a kernel needs to place
 * a token into ONE int32 buffer (copied to the device in one transfer) and describes it in
 * `layout`, KBATCH_LAYOUT_INTS ints indexed by the KB_* names: counts first, then offsets
 * (in ints) of the sections.
 * ========================================================================================== */
#define KB_NUM_TOKENS 0      /* T */
#define KB_NUM_SEQS 1        /* n */
#define KB_NUM_ROWS 2        /* R: places whose logits are wanted */
#define KB_TABLE_WIDTH 3     /* W: entries per block-table row */
#define KB_NUM_GROUPS 4      /* G */
#define KB_MAX_COUNT 5       /* most tokens of one request in this step */
#define KB_MAX_KV_LEN 6      /* longest request after this step */
#define KB_TOTAL_INTS 7
#define KB_O_TOKEN_IDS 8     /* [T] */
#define KB_O_POSITIONS 9     /* [T] position of each token in its request */
#define KB_O_SEQ_OF_TOKEN 10 /* [T] index of its request in this step */
#define KB_O_CU_SEQLENS 11   /* [n + 1] first token of each request */
#define KB_O_KV_LENS 12      /* [n] request length after this step */
#define KB_O_SLOTS 13        /* [n] state slot */
#define KB_O_ROWS 14         /* [R] token rows whose logits are wanted */
#define KB_O_MAX_KV 15       /* [1] KB_MAX_KV_LEN again, for kernels */
#define KB_O_TABLES 16       /* [G, n, W] pages, -1 where there is none */
#define KBATCH_LAYOUT_INTS 24
/* ints that kbatch_pack will write for these entries (table_width 0: the narrowest multiple of 8 that holds them) */
KESTREL_API int kbatch_ints_needed(void *cache, int n, const long long *ids, const int *counts, int n_wants, int table_width);
/* tokens: the entries' token ids one after the other (NULL leaves the section unwritten: ids that are on the device already);
 * want_counts[e] places of entry e are wanted, listed in `wants` as offsets among the entry's tokens.  Pages must be reserved.
 * Returns the ints written, or -2 bad argument, -3 unknown request, -9 buffer too small. */
KESTREL_API int kbatch_pack(void *cache, int n, const long long *ids, const int *counts, const int *tokens, const int *want_counts, const int *wants, int table_width, int *out, int cap, int *layout);

/* the check of the runner's debug guards, on the host: 0 if every token of the packed description can be placed by the kernels,
 * else (rule << 16) | (token & 0xffff) for the first that cannot (rules: 1 token id, 2 request index, 3 position,
 * 4 block-table column, 5 page id, 6 token outside its request's rows); pages[g] = pages of group g's tensors */
KESTREL_API int kbatch_check(const int *batch, const int *layout, int vocab, int page_size, const int *pages);

/* ============================================================================================
 * Kernel library (libkestrel_cuda.so): runtime
 * ========================================================================================== */
KESTREL_API const char *kestrel_last_error(void);
KESTREL_API int kestrel_device_arch(void);
KESTREL_API int kestrel_sm_count(void);
KESTREL_API void kestrel_set_pdl(int on);
KESTREL_API int kestrel_wait_probe(float *elapsed_ms);
/* 0 if no bounded wait of any kernel has run out since the last call, else which kernels' did (bit 0 product, 1 prompt attention, 2 decode attention); synchronises the device */
KESTREL_API int kestrel_kernel_errors(void);

/* ---- elementwise kernels ---- */
KESTREL_API int kestrel_embed(const void *table, int dtype, const int *ids, float *out, int T, int d, kestrel_stream_t stream);
KESTREL_API void kestrel_set_norm_warp_rows(int rows, int with_slices);   /* rows from which a norm that only reads the stream takes a warp a row (0: the default), and whether one that adds slices does too; for tests of both kernels */
KESTREL_API int kestrel_add_rmsnorm(float *residual, const float *partial, int S, long long slice_stride, const float *bias, const int *rows, const float *w, float eps, void *out, int out_dtype, int R, int d, int write_back, kestrel_stream_t stream);
KESTREL_API int kestrel_swiglu(const float *partial, int S, long long slice_stride, void *out, int out_dtype, int T, int ff, kestrel_stream_t stream);
/* rot_mode: 0 pairs dimension j with j + rot/2 (rotate-half), 1 pairs 2j with 2j + 1 (interleaved); rot_scale multiplies cos and sin */
KESTREL_API int kestrel_attn_prepare(const float *partial, int S, long long slice_stride, const float *bias, const float *q_norm_w, const float *k_norm_w, float norm_eps, const float *inv_freq, int rot, int rot_mode, float rot_scale, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *k_cache, void *v_cache, void *q_out, int dtype, int T, int nq, int nkv, int hd, int write_kv, kestrel_stream_t stream);
KESTREL_API int kestrel_reduce_partials(const float *partial, int S, long long slice_stride, const float *bias, void *out, int out_dtype, int T, int width, kestrel_stream_t stream);

/* ---- kernels around the residual stream for other arrangements than the pre-norm block (stream_ops.cu) ---- */
/* x[t, 2i] += sin(pos[t] freq[i]), x[t, 2i + 1] += cos(pos[t] freq[i]) */
KESTREL_API int kestrel_add_sinusoid(float *x, const int *positions, const float *freq, int T, int d, kestrel_stream_t stream);
/* residual += sum of a's slices + sum of b's slices (b may be NULL); cast = residual in the storage type (may be NULL) */
KESTREL_API int kestrel_add_two(float *residual, const float *a, int Sa, long long stride_a, const float *b, int Sb, long long stride_b, void *cast, int cast_dtype, int T, int d, kestrel_stream_t stream);
/* out[t, i] = gelu_tanh(sum of g's slices at [t, i]) * table[ids[t], col0 + i], i < n; table and out in the storage type */
KESTREL_API int kestrel_gelu_table_mul(const float *g, int S, long long slice_stride, int ld, const void *table, int table_ld, int col0, const int *ids, void *out, int dtype, int T, int n, kestrel_stream_t stream);
/* y = sum of p's slices; residual[t] += y / sqrt(mean(y^2) + eps) * w */
KESTREL_API int kestrel_add_normed(float *residual, const float *p, int S, long long slice_stride, const float *w, float eps, int T, int d, kestrel_stream_t stream);
/* out[t, i] = sum of p's slices at [t, col0 + i], i < n, in the storage type */
KESTREL_API int kestrel_partial_columns(const float *p, int S, long long slice_stride, int ld, int col0, void *out, int dtype, int T, int n, kestrel_stream_t stream);
/* the same with the product's bias (NULL: none; indexed like the product's columns) and an activation on the sum: 0 none, 1 relu squared, 2 tanh, 3 silu, 4 gelu (erf), 5 gelu (tanh form) */
KESTREL_API int kestrel_partial_columns_act(const float *p, int S, long long slice_stride, int ld, int col0, const float *bias, int act, void *out, int dtype, int T, int n, kestrel_stream_t stream);
/* residual += sum of a's + b's + c's slices (b, c may be NULL), (a + b) + c; cast = residual in the storage type (may be NULL) */
KESTREL_API int kestrel_add_three(float *residual, const float *a, int Sa, long long stride_a, const float *b, int Sb, long long stride_b, const float *c, int Sc, long long stride_c, void *cast, int cast_dtype, int T, int d, kestrel_stream_t stream);
/* x[t, i] *= sigmoid(sum of g's slices at [t, col0 + i] + bias[col0 + i]), i < n, in place in the storage type (bias may be NULL) */
KESTREL_API int kestrel_gate_columns_mul(void *x, int dtype, const float *g, int S, long long slice_stride, int ld, int col0, const float *bias, int T, int n, kestrel_stream_t stream);
/* x[t, :] += row[:] */
KESTREL_API int kestrel_add_row(float *x, const float *row, int T, int d, kestrel_stream_t stream);
/* out[t, :] = table[ids[t], :] * scale, float32 */
KESTREL_API int kestrel_embed_scaled(const void *table, int dtype, const int *ids, float *out, int T, int d, float scale, kestrel_stream_t stream);
/* out[t] = mix (a / sqrt(mean(a^2) + eps) wa + b / sqrt(mean(b^2) + eps) wb), a and b the sums of two products' slices, float32 */
KESTREL_API int kestrel_combine_normed(const float *a, int Sa, long long stride_a, const float *wa, const float *b, int Sb, long long stride_b, const float *wb, float eps, float mix, float *out, int T, int d, kestrel_stream_t stream);
/* v = (sum of y's slices + y_bias) * sigmoid(sum of g's slices + g_bias) (g may be NULL: no gate); residual[t] += v / sqrt(mean(v^2) + eps) w; with next_w also next_out[t] = residual[t] / sqrt(mean(residual[t]^2) + eps_next) next_w in the storage type */
KESTREL_API int kestrel_add_gated_normed(float *residual, const float *y, int Sy, long long stride_y, const float *y_bias, const float *g, int Sg, long long stride_g, const float *g_bias, const float *w, float eps, const float *next_w, float eps_next, void *next_out, int next_dtype, int T, int d, kestrel_stream_t stream);
/* x[t] += table[ids[t]] */
KESTREL_API int kestrel_embed_add(const void *table, int dtype, const int *ids, float *x, int T, int d, kestrel_stream_t stream);
/* logits <- logits * scale, then cap tanh(logits / cap) where cap > 0; in place */
KESTREL_API int kestrel_logit_scale_cap(float *logits, long long ld, int R, int V, float scale, float cap, kestrel_stream_t stream);

/* ---- attention without rotation, with values of their own size, kept first tokens and an output gate ---- */
/* product columns [q: nq hd | k: nkv hd | v: nkv vd | gate: nq]; k, v absent if has_kv = 0, gate if gate_out is NULL; qk_norm: q, k / sqrt(mean(x^2) + eps) per head, times q_norm_w / k_norm_w [hd] where given */
KESTREL_API int kestrel_attn_prepare_ex(const float *partial, int S, long long slice_stride, int ld, const float *q_norm_w, const float *k_norm_w, int qk_norm, float norm_eps, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *k_cache, void *v_cache, void *q_out, float *gate_out, int dtype, int T, int nq, int nkv, int hd, int vd, int has_kv, kestrel_stream_t stream);
/* the plain attention with a value size vd, the first keep_first keys of a request visible beyond the window, and head outputs multiplied by gate [T, nq] (may be NULL) */
KESTREL_API int kestrel_attention_plain_ex(const void *q, const void *k_cache, const void *v_cache, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *out, int dtype, int T, int nq, int nkv, int hd, int vd, int window, int keep_first, const float *gate, float scale, kestrel_stream_t stream);
/* the same attention for bfloat16 on the tensor cores (attention_window.cu); head sizes in multiples of 8 up to 256; max_count = the most tokens one request brings in this step */
KESTREL_API int kestrel_attention_window_supported(int hd, int vd, int nq, int nkv);
KESTREL_API int kestrel_attention_window(const void *q, const void *k_cache, const void *v_cache, void *out, const float *gate, const int *cu_seqlens, const int *kv_lens, const int *block_table, int table_stride, int page_size, int nseq, int max_count, int nq, int nkv, int hd, int vd, int window, int keep_first, float scale, kestrel_stream_t stream);

/* ---- options on the scores and on the weighing of keys (attention_score.cuh); all float32 ----
   softcap > 0: s <- softcap tanh(s / softcap); r1, r2 [nq] (both or neither): s <- s - r1[h] ln(1 + r2[h] (i - j));
   weighting 0: softmax; 1: softmax with a valueless extra term exp(sink[h]) in the denominator (sink [nq], or NULL for
   exp(0)); 2: every visible key weighs sigmoid(s + head_bias[h]) (head_bias [nq] or NULL), not normalised over keys */
KESTREL_API int kestrel_attention_plain_scored(const void *q, const void *k_cache, const void *v_cache, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *out, int dtype, int T, int nq, int nkv, int hd, int vd, int window, int keep_first, const float *gate, float scale, float softcap, const float *r1, const float *r2, const float *head_bias, int weighting, const float *sink, kestrel_stream_t stream);
/* the same with rel[bucket[min(i - j, rel_far)], head] added to the scores: rel float32 [buckets, nq], rel_bucket int32 [rel_far + 1] (rel may be NULL); v_ld > 0: the V plane's rows hold v_ld numbers, the first vd of them the value */
KESTREL_API int kestrel_attention_plain_biased(const void *q, const void *k_cache, const void *v_cache, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *out, int dtype, int T, int nq, int nkv, int hd, int vd, int window, int keep_first, const float *gate, float scale, float softcap, const float *r1, const float *r2, const float *head_bias, int weighting, const float *sink, const float *rel, const int *rel_bucket, int rel_far, int v_ld, kestrel_stream_t stream);
KESTREL_API int kestrel_attention_window_scored(const void *q, const void *k_cache, const void *v_cache, void *out, const float *gate, const int *cu_seqlens, const int *kv_lens, const int *block_table, int table_stride, int page_size, int nseq, int max_count, int nq, int nkv, int hd, int vd, int window, int keep_first, float scale, float softcap, const float *r1, const float *r2, const float *head_bias, int weighting, const float *sink, int ksplit, float *scratch, kestrel_stream_t stream);
KESTREL_API int kestrel_attention_window_biased(const void *q, const void *k_cache, const void *v_cache, void *out, const float *gate, const int *cu_seqlens, const int *kv_lens, const int *block_table, int table_stride, int page_size, int nseq, int max_count, int nq, int nkv, int hd, int vd, int window, int keep_first, float scale, float softcap, const float *r1, const float *r2, const float *head_bias, int weighting, const float *sink, const float *rel, const int *rel_bucket, int rel_far, int v_ld, int ksplit, float *scratch, kestrel_stream_t stream);
/* a step of single tokens may cut its key rounds into `ksplit` shares, a CTA each, merged by a second kernel; scratch of kestrel_attention_window_scratch_floats floats */
KESTREL_API int kestrel_attention_window_splits(int nseq, int max_count, int nq, int nkv, int hd, int vd, int window, int max_kv_len);
KESTREL_API long long kestrel_attention_window_scratch_floats(int nseq, int max_count, int nq, int nkv, int hd, int vd, int ksplit);
KESTREL_API int kestrel_attention_tc_scored(const void *q, const void *k_cache, const void *v_cache, void *out, float *part_o, float *part_ml, const int *tile_seq, const int *tile_row0, int tiles, int rows_per_tile, const int *cu_seqlens, const int *kv_lens, const int *block_table, int table_width, int table_stride, int page_size, int cache_pages, int T, int nq, int nkv, int hd, int window, int slices, int slice_len, const int *max_kv_ptr, float scale, float softcap, const float *r1, const float *r2, const float *head_bias, int weighting, const float *sink, kestrel_stream_t stream);
KESTREL_API int kestrel_attention_tc_biased(const void *q, const void *k_cache, const void *v_cache, void *out, float *part_o, float *part_ml, const int *tile_seq, const int *tile_row0, int tiles, int rows_per_tile, const int *cu_seqlens, const int *kv_lens, const int *block_table, int table_width, int table_stride, int page_size, int cache_pages, int T, int nq, int nkv, int hd, int window, int slices, int slice_len, const int *max_kv_ptr, float scale, float softcap, const float *r1, const float *r2, const float *head_bias, int weighting, const float *sink, const float *rel, const int *rel_bucket, int rel_far, kestrel_stream_t stream);
/* attn_prepare_ex with a bias per product column (NULL: none); qk_norm 0: none, 1: per head (weights [hd] or NULL), 2: over the whole q and the whole k projection (weights [nq hd], [nkv hd]); v_norm: v / sqrt(mean(v^2) + eps) per head */
KESTREL_API int kestrel_attn_prepare_normed(const float *partial, int S, long long slice_stride, int ld, const float *bias, const float *q_norm_w, const float *k_norm_w, int qk_norm, int v_norm, float norm_eps, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *k_cache, void *v_cache, void *q_out, float *gate_out, int dtype, int T, int nq, int nkv, int hd, int vd, int has_kv, kestrel_stream_t stream);
/* attn_prepare_normed, then q and k turned by position where inv_freq is given: pair j of a head's first `rot` dimensions by position * inv_freq[j]; rot_mode 0 pairs j with j + rot / 2, 1 pairs 2j with 2j + 1; rot_scale multiplies cos and sin */
KESTREL_API int kestrel_attn_prepare_rotated(const float *partial, int S, long long slice_stride, int ld, const float *bias, const float *q_norm_w, const float *k_norm_w, int qk_norm, int v_norm, float norm_eps, const float *inv_freq, int rot, int rot_mode, float rot_scale, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *k_cache, void *v_cache, void *q_out, float *gate_out, int dtype, int T, int nq, int nkv, int hd, int vd, int has_kv, kestrel_stream_t stream);
/* the same with a query temperature: q times 1 + q_temp_coef ln(floor((position + 1) / q_temp_every) + 1); q_temp_every = 0: none */
KESTREL_API int kestrel_attn_prepare_tempered(const float *partial, int S, long long slice_stride, int ld, const float *bias, const float *q_norm_w, const float *k_norm_w, int qk_norm, int v_norm, float norm_eps, const float *inv_freq, int rot, int rot_mode, float rot_scale, float q_temp_coef, int q_temp_every, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *k_cache, void *v_cache, void *q_out, float *gate_out, int dtype, int T, int nq, int nkv, int hd, int vd, int has_kv, kestrel_stream_t stream);

/* ---- attention over cached latents (attention_latent.cu) ---- */
/* product columns [q latent: q_rank | kv latent: kv_rank | gate: n_gate]: both latents RMS-normed with their weights; the query latent to q_out [T, q_rank], the kv latent into the token's slot of latent_cache [pages, 1, page_size, kv_rank], sigmoid of the gate columns to gate_out [T, n_gate]; kv_out (may be NULL) receives the kv latents as rows [T, kv_rank] too */
KESTREL_API int kestrel_latent_prepare(const float *partial, int S, long long slice_stride, int ld, const float *q_norm_w, const float *kv_norm_w, float norm_eps, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *latent_cache, void *q_out, float *gate_out, void *kv_out, int dtype, int T, int q_rank, int kv_rank, int n_gate, kestrel_stream_t stream);
/* the same with rot_cols more columns between the kv latent and the gates: a key part shared by all heads, not normed, its first `rot` dimensions turned by position (rot_mode 0 halves, 1 neighbours; rot_scale on cos and sin); a cache row is [latent | key part] */
KESTREL_API int kestrel_latent_prepare_rotated(const float *partial, int S, long long slice_stride, int ld, const float *q_norm_w, const float *kv_norm_w, float norm_eps, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *latent_cache, void *q_out, float *gate_out, void *kv_out, int dtype, int T, int q_rank, int kv_rank, int n_gate, int rot_cols, const float *inv_freq, int rot, int rot_mode, float rot_scale, kestrel_stream_t stream);
/* q_lat[t, h out_head_stride + col0 + i] = column d + i of head h of q (head_stride columns a head), i < rot_cols, the first `rot` turned by position */
KESTREL_API int kestrel_latent_rotate_queries(const void *q, int ldq, int head_stride, int d, void *q_lat, int ldo, int out_head_stride, int col0, const int *positions, int dtype, int T, int H, int rot_cols, const float *inv_freq, int rot, int rot_mode, float rot_scale, kestrel_stream_t stream);
/* x[t, h, :] *= gate[t, h] in place, x [T, heads d] in the storage type */
KESTREL_API int kestrel_head_scale(void *x, const float *gate, int dtype, int T, int heads, int d, kestrel_stream_t stream);
/* out[t, h N + n] = sum_k x[t, h K + k] w_h[n, k]; w_kn = 0: w_h = rows [h N, (h + 1) N) of w [H N, K]; w_kn = 1: w_h[n, k] = w[h K + k, n] of w [H K, N]; all in the storage type, float32 sums */
KESTREL_API int kestrel_head_gemm(const void *x, int ldx, const void *w, int ldw, int w_kn, void *out, int ldo, int dtype, int T, int H, int N, int K, kestrel_stream_t stream);
/* the same with head h's input at x[t, h hsx + k] and its output at out[t, h hso + n], float32 output if out_f32 */
KESTREL_API int kestrel_head_gemm_strided(const void *x, int ldx, int hsx, const void *w, int ldw, int w_kn, void *out, int ldo, int hso, int out_f32, int dtype, int T, int H, int N, int K, kestrel_stream_t stream);
KESTREL_API void kestrel_head_gemm_set_plain(int on);   /* 1: bfloat16 head-wise products take the CUDA-core kernel too; for tests of both */

/* ---- gated delta rule with a decay per key channel (delta_rule.cu); state slot = [S: H d dv | tail: (taps - 1) C] float32 ---- */
KESTREL_API int kestrel_delta_conv_silu(const float *partial, int S, long long slice_stride, int ld, const float *w, int taps, float *state, long long state_stride, long long tail_off, const int *seq_of_token, const int *cu_seqlens, const int *slots, float *out, int T, int nseq, int C, kestrel_stream_t stream);
KESTREL_API int kestrel_delta_gates(const float *act, int C, const float *partial, int S, long long slice_stride, int ld, int col_beta, const float *a_part, int Sa, long long a_stride, const float *A_log, const float *dt_bias, float *qn, float *kn, float *decay, float *beta, int T, int H, int G, int d, kestrel_stream_t stream);
KESTREL_API int kestrel_delta_scan(const float *qn, const float *kn, const float *decay, const float *act, int C, int col_v, const float *beta, float *state, long long state_stride, const int *cu_seqlens, const int *slots, float *out, int nseq, int H, int G, int d, int dv, kestrel_stream_t stream);
KESTREL_API int kestrel_delta_out(const float *o, const float *w, float eps, const float *g_part, int Sg, long long g_stride, void *out, int dtype, int T, int H, int dv, kestrel_stream_t stream);

/* ---- a diagonal recurrence with gates made from its own input (rglru.cu); state slot = [S: C | tail: (taps - 1) C] float32 ---- */
KESTREL_API int kestrel_rglru_branches(const float *partial, int S, long long slice_stride, int ld, const float *bias, const float *conv_w, const float *conv_b, int taps, float *state, long long state_stride, long long tail_off, const int *seq_of_token, const int *cu_seqlens, const int *slots, float *y_out, float *u_out, void *u_st, int dtype, int T, int nseq, int C, kestrel_stream_t stream);
KESTREL_API int kestrel_rglru_scan(const float *y, const float *u, const float *gr, const float *gi, const float *r_bias, const float *i_bias, const float *lam, float rate, float *state, long long state_stride, const int *cu_seqlens, const int *slots, void *out, int dtype, int nseq, int C, kestrel_stream_t stream);
/* the same in chunks of `chunk` tokens (a multiple of 8) for steps that bring a request many tokens: two kernels, a thread a (request, chunk, channel); scratch float32 [nseq * ceil(max_count / chunk) * 2 * C] */
KESTREL_API int kestrel_rglru_scan_chunked(const float *y, const float *u, const float *gr, const float *gi, const float *r_bias, const float *i_bias, const float *lam, float rate, float *state, long long state_stride, const int *cu_seqlens, const int *slots, void *out, int dtype, int nseq, int max_count, int chunk, float *scratch, int C, kestrel_stream_t stream);

/* ---- linear recurrences S_t = diag(w) S + a (b^T S) + k v^T, o = S^T r per head (linear_recurrence.cu); S [H, d, dv] float32 at state_off of the request's state slot ---- */
/* product columns q, f [n = H d] and v [nv = H dv]: r = silu(q), w = lower + (1 - lower) sigmoid(f + f_bias), k = 1 - w, v as it is; all float32 [T, .] */
KESTREL_API int kestrel_forget_gates(const float *partial, int S, long long slice_stride, int ld, int col_q, int col_f, int col_v, const float *f_bias, const float *lower, float *r_out, float *w_out, float *k_out, float *v_out, int T, int n, int nv, kestrel_stream_t stream);
/* product columns r, k, v, rate logits [H d each]; wz a second product [T, H d]: u = k / sqrt(sum k^2 + 1e-6) per head, w = exp(-decay_rate sigmoid(wz + w_bias)), a = -(sigmoid(rate + a_bias) u), b = u */
KESTREL_API int kestrel_removal_gates(const float *partial, int S, long long slice_stride, int ld, int col_r, int col_k, int col_v, int col_a, const float *a_bias, const float *wz, int Sw, long long w_stride, const float *w_bias, float decay_rate, float *r_out, float *k_out, float *v_out, float *w_out, float *a_out, float *b_out, int T, int H, int d, kestrel_stream_t stream);
/* r, w, k, a, b [T, H d], v and out [T, H dv], float32; a and b both NULL: no correction */
KESTREL_API int kestrel_recurrence_scan(const float *r, const float *w, const float *k, const float *v, const float *a, const float *b, float *state, long long state_stride, long long state_off, const int *cu_seqlens, const int *slots, float *out, int nseq, int H, int d, int dv, kestrel_stream_t stream);
/* out = o / sqrt(mean(o^2) + eps) per head, times w[h w_stride + i] (w_stride 0: one weight [dv] for all heads, dv: one per head), times sigmoid of the gate product's columns g_col0 + h dv + i where g_part is given; storage type */
KESTREL_API int kestrel_head_norm_gate(const float *o, const float *w, int w_stride, float eps, const float *g_part, int Sg, long long g_stride, int g_ld, int g_col0, void *out, int dtype, int T, int H, int dv, kestrel_stream_t stream);

/* ---- routed feed-forward (moe.cu) ---- */
KESTREL_API int kestrel_moe_route(const float *z_part, int S, long long slice_stride, const float *bias, int *ids, float *weights, int T, int E, int top, kestrel_stream_t stream);
/* scores sigmoid(z); chosen by score + correction[e] (may be NULL) among the experts of the `keep` best of `n_groups` groups of neighbours (a group's score: the sum of its two largest choice scores); weights = chosen scores / (their sum + 1e-20) * scale */
KESTREL_API int kestrel_moe_route_sigmoid(const float *z_part, int S, long long slice_stride, const float *correction, int n_groups, int keep, float scale, int *ids, float *weights, int T, int E, int top, kestrel_stream_t stream);
KESTREL_API int kestrel_moe_max_tiles(int P, int E, int rows_per_tile);
KESTREL_API void kestrel_moe_set_plain(int on);   /* 1: the bfloat16 grouped products take the CUDA-core kernel instead of the tensor-core one; for tests of both */
KESTREL_API int kestrel_moe_group(const int *ids, int P, int E, int rows_per_tile, int *offsets, int *row_pair, int *pair_row, int *tile_expert, int *tile_row0, int *n_tiles, kestrel_stream_t stream);
KESTREL_API int kestrel_moe_gate_up(const void *x, long long ldx, const void *w, const int *offsets, const int *row_pair, const int *tile_expert, const int *tile_row0, const int *n_tiles, int max_tiles, int top, float limit, void *act, int dtype, int ff, int K, kestrel_stream_t stream);
KESTREL_API int kestrel_moe_down(const void *act, const void *w, const int *offsets, const int *row_pair, const int *tile_expert, const int *tile_row0, const int *n_tiles, int max_tiles, const float *pair_weight, float *y, int dtype, int N, int ff, kestrel_stream_t stream);
/* experts without a gate: act [P, ff] = activation(W_up[e] xs), xs [P, K] the pairs' input rows in sorted order, w [E, ff, K]; act_kind 1 gelu (erf), 2 gelu (tanh form), 3 silu, 4 relu squared */
KESTREL_API int kestrel_moe_up_act(const void *xs, const void *w, const int *offsets, const int *row_pair, const int *tile_expert, const int *tile_row0, const int *n_tiles, int max_tiles, int act_kind, void *act, int dtype, int ff, int K, kestrel_stream_t stream);
KESTREL_API int kestrel_moe_gather_rows_any(const void *x, long long ldx, const int *row_pair, int top, void *xs, int dtype, int P, int K, kestrel_stream_t stream);
/* the grouped products of many tokens on tcgen05 (moe_tcgen05.cu): tiles of kestrel_moe_tc_tile_rows() rows; xs = the pairs' input rows gathered in sorted order */
KESTREL_API int kestrel_moe_tc_tile_rows(void);
KESTREL_API int kestrel_moe_tc_supported(const void *xs, const void *act, const void *w_gate_up, const void *w_down, int ff, int K);
KESTREL_API int kestrel_moe_gather_rows(const void *x, long long ldx, const int *row_pair, int top, void *xs, int P, int K, kestrel_stream_t stream);
KESTREL_API int kestrel_moe_gate_up_tc(const void *xs, const void *w, const int *offsets, const int *tile_expert, const int *tile_row0, const int *n_tiles, int max_tiles, float limit, void *act, int P, int E, int ff, int K, kestrel_stream_t stream);
KESTREL_API int kestrel_moe_down_tc(const void *act, const void *w, const int *offsets, const int *row_pair, const int *tile_expert, const int *tile_row0, const int *n_tiles, int max_tiles, const float *pair_weight, float *y, int P, int E, int N, int ff, kestrel_stream_t stream);
KESTREL_API int kestrel_moe_up_act_tc(const void *xs, const void *w, const int *offsets, const int *tile_expert, const int *tile_row0, const int *n_tiles, int max_tiles, int act_kind, void *act, int P, int E, int ff, int K, kestrel_stream_t stream);
KESTREL_API int kestrel_moe_tc_error(void);
KESTREL_API void kestrel_moe_tc_set_ring_kb(int kb);   /* shared memory of a CTA's stages in KB: 104 (default) lets two CTAs share an SM, 200 gives one all of it; for measurements */
KESTREL_API int kestrel_moe_combine(const float *y, const int *pair_row, int top, float *out, int T, int N, kestrel_stream_t stream);

/* ---- matrix products ---- */
KESTREL_API int kestrel_gemm_plain(const void *x, const void *w, float *out, int dtype, int T, int N, int K, long long ldx, long long ldw, long long ldo, kestrel_stream_t stream);
KESTREL_API int kestrel_gemm_tc_supported(const void *x, const void *w, int T, int N, int K, long long ldx, long long ldw);
KESTREL_API int kestrel_gemm_tc_splits(int T, int N, int K);
KESTREL_API int kestrel_gemm_tc_plan(const void *x, const void *w, int T, int N, int K, long long ldx, long long ldw);
KESTREL_API int kestrel_gemm_tc_w(const void *x, const void *w, float *out, int T, int N, int K, long long ldx, long long ldw, long long ldo, int splits, long long slice_stride, int weights_static, kestrel_stream_t stream);
KESTREL_API int kestrel_gemm_tc(const void *x, const void *w, float *out, int T, int N, int K, long long ldx, long long ldw, long long ldo, int splits, long long slice_stride, kestrel_stream_t stream);
KESTREL_API int kestrel_gemm_tc_add(const void *x, const void *w, float *residual, int T, int N, int K, long long ldx, long long ldw, long long ldo, kestrel_stream_t stream);
KESTREL_API int kestrel_gemm_tc_act(const void *x, const void *w, void *out, int act, int T, int N, int K, long long ldx, long long ldw, long long ldo, kestrel_stream_t stream);
KESTREL_API int kestrel_gemm_tc_swiglu_w(const void *x, const void *w, void *out, int T, int ff, int K, long long ldx, long long ldw, long long ldo, int weights_static, kestrel_stream_t stream);
KESTREL_API int kestrel_gemm_tc_swiglu(const void *x, const void *w, void *out, int T, int ff, int K, long long ldx, long long ldw, long long ldo, kestrel_stream_t stream);
/* the q, k, v product of many tokens with the prepare kernel's work in its epilogue (head size 128, rotate-half over the whole head); 0 done, 1 this form does not apply and nothing ran */
KESTREL_API int kestrel_gemm_tc_qkv_prepare(const void *x, const void *w, int T, int K, long long ldx, long long ldw, const float *bias, const float *q_norm_w, const float *k_norm_w, float norm_eps, const float *inv_freq, int rot, int rot_mode, float rot_scale, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *k_cache, void *v_cache, void *q_out, int nq, int nkv, int hd, int write_kv, kestrel_stream_t stream);
KESTREL_API void kestrel_gemm_tc_set_qkv_fused(int mode);   /* 0 never, 1 where the product is not cut along K (default), 2 wherever the kernel takes the sizes */
KESTREL_API int kestrel_gemm_tc_error(void);
KESTREL_API int kestrel_linear_bf16_noalloc(const void *x, const void *w, const float *bias, void *out, int out_dtype, int T, int N, int K, long long ldx, long long ldw, kestrel_stream_t stream);
/* tuning and test hooks of the products */
KESTREL_API void kestrel_gemm_tc_set_persistent(int on);
KESTREL_API void kestrel_gemm_tc_set_pairs(int on);
KESTREL_API void kestrel_gemm_tc_set_swiglu_tile(int bn);
/* the SwiGLU product on CTA pairs with the tokens as the M operand: 0 never, 1 where its finer tiles save a round (the default), 2 always */
KESTREL_API void kestrel_gemm_tc_set_swiglu_swapped(int mode);
KESTREL_API void kestrel_gemm_tc_set_pair_tuning(int min_tokens, int overhead_kb);
KESTREL_API void kestrel_gemm_tc_set_tuning(int overhead_kb, int ctas_per_sm);
KESTREL_API void kestrel_gemm_tc_set_wide(int on, int more_than_tokens);

/* ---- attention kernels (tile lists: request and first row of each tile).  max_kv_ptr, if not
 * NULL, points to the longest request's length on the device; the slice length is then
 * ceil(that / slices) rounded up to a multiple of 128 instead of slice_len (a captured launch
 * follows the context that way). ---- */
KESTREL_API int kestrel_attention_plain(const void *q, const void *k_cache, const void *v_cache, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *out, int dtype, int T, int nq, int nkv, int hd, int window, float scale, kestrel_stream_t stream);
KESTREL_API int kestrel_attention_mma(const void *q, const void *k_cache, const void *v_cache, void *out, float *part_o, float *part_ml, const int *tile_seq, const int *tile_row0, int tiles, int rows_per_tile, const int *cu_seqlens, const int *kv_lens, const int *block_table, int table_stride, int page_size, int T, int nq, int nkv, int hd, int window, int slices, int slice_len, const int *max_kv_ptr, float scale, kestrel_stream_t stream);
KESTREL_API int kestrel_attention_mma_rows_per_tile(int hd);
KESTREL_API int kestrel_attention_mma_slots(int hd);
KESTREL_API int kestrel_attention_merge(const float *part_o, const float *part_ml, void *out, const int *tile_seq, const int *tile_row0, int tiles, int rows_per_tile, const int *cu_seqlens, int slices, int hd, int nq, int nkv, const float *sink, kestrel_stream_t stream);
KESTREL_API int kestrel_attention_tc(const void *q, const void *k_cache, const void *v_cache, void *out, float *part_o, float *part_ml, const int *tile_seq, const int *tile_row0, int tiles, int rows_per_tile, const int *cu_seqlens, const int *kv_lens, const int *block_table, int table_width, int table_stride, int page_size, int cache_pages, int T, int nq, int nkv, int hd, int window, int slices, int slice_len, const int *max_kv_ptr, float scale, kestrel_stream_t stream);
KESTREL_API int kestrel_attention_tc_supported(int hd, int page_size);
KESTREL_API int kestrel_attention_tc_slots(void);
KESTREL_API int kestrel_attention_tc_error(void);
KESTREL_API int kestrel_attention_decode(const void *q, const void *k_cache, const void *v_cache, void *out, float *part_o, float *part_ml, const int *tile_seq, const int *tile_row0, int tiles, const int *cu_seqlens, const int *kv_lens, const int *block_table, int table_width, int table_stride, int page_size, int cache_pages, int T, int nq, int nkv, int hd, int window, int slices, int slice_len, const int *max_kv_ptr, float scale, kestrel_stream_t stream);
KESTREL_API int kestrel_attention_decode_supported(int hd, int page_size);
KESTREL_API int kestrel_attention_decode_slots(int hd);
KESTREL_API int kestrel_attention_decode_cluster_slices(void);
KESTREL_API int kestrel_attention_decode_error(void);

/* ---- attention of a whole step: picks kernels, tiles the step's rows, cuts key ranges ----
 * A planner belongs to the mixers of one model.  It keeps the tile lists of the current step on
 * the device (built once per step from the step's host description and copied in one small
 * transfer; steps of one token per request need none) and scratch for key-range slices.
 * `batch_host` / `batch_dev` are the packed step description (kbatch_pack) on the host and on
 * the device, `layout` its layout; `step_serial` changes with every step.  captured != 0: the
 * launch is being recorded for replay with other contents, so the number of slices follows
 * layout[KB_MAX_KV_LEN] (a nominal context) and their length is read on the device. */
/* short prompt portions on the kernel for decode tokens: the key limits in per cent of the defaults (0: never, negative: the default); for tests and tuning */
KESTREL_API void kestrel_attention_set_small_portions(int per_cent);
KESTREL_API void *kestrel_attn_planner_create(int max_tokens, int max_seqs);
KESTREL_API void kestrel_attn_planner_destroy(void *planner);
KESTREL_API int kestrel_attention(void *planner, long long step_serial, const int *batch_host, const int *batch_dev, const int *layout, int group, int captured, const void *q, const void *k_cache, const void *v_cache, void *out, int dtype, int cache_pages, int page_size, int nq, int nkv, int hd, int window, float scale, kestrel_stream_t stream);
/* kernels launched by the planner's last kestrel_attention call */
KESTREL_API int kestrel_attn_planner_last_launches(void *planner);

/* ---- sampling ---- */
KESTREL_API int kestrel_argmax(const float *logits, long long ld, int R, int V, int *out, float *cand_v, int *cand_i, kestrel_stream_t stream);
KESTREL_API int kestrel_argmax_chunks(int V);
KESTREL_API int kestrel_repetition_penalty(float *logits, long long ld, int R, int V, const int *history, int width, const int *counts, const float *penalty, kestrel_stream_t stream);
KESTREL_API void kestrel_sample_set_cluster(int on);
KESTREL_API int kestrel_sample(const float *logits, long long ld, int R, int V, const float *temperature, const int *top_k, const float *top_p, const float *min_p, const float *uniform, int *out, kestrel_stream_t stream);

/* ============================================================================================
 * The step program (libkestrel_cuda.so): a model as a list of kernel-level operations, written
 * once when the model is built and run natively for every step, so that a step costs the host
 * one call.  Operations read and write "registers": activations of the step, allocated by the
 * runner from its workspace.  kprog_* functions that make a value return its register (>= 0)
 * or a negative code.  `tag` names the phase an operation is timed under when profiling
 * (KPH_*).  Weights and cache tensors are device pointers that stay valid while the program
 * lives.  `dtype` arguments are storage type codes.
 * ========================================================================================== */
#define KPH_OTHER 0
#define KPH_NORM 1
#define KPH_QKV 2
#define KPH_ROPE 3
#define KPH_ATTN 4
#define KPH_O 5
#define KPH_GATE_UP 6
#define KPH_DOWN 7
#define KPH_LM_HEAD 8
#define KPH_EMBED 9
#define KPH_COUNT 10
KESTREL_API void *kprog_create(int dtype);
KESTREL_API void kprog_destroy(void *prog);
/* marks the start of a layer call: registers made in the call before it stay readable during this one, older ones do not */
KESTREL_API int kprog_begin_call(void *prog);
/* float32 residual stream [T, width] = table[token ids] */
KESTREL_API int kprog_embed(void *prog, const void *table, int table_dtype, int width);
/* residual += delta (a product register, or -1); result = rmsnorm(residual) * w in out_dtype; logit_rows != 0: only the wanted rows, nothing written back */
KESTREL_API int kprog_add_rmsnorm(void *prog, int residual, int delta, const float *w, float eps, int width, int out_dtype, int logit_rows, int tag);
/* x w^T (+ bias later, by the consumer) as float32 slices; add_to >= 0: the product may add itself to that float32 register in its epilogue, its own register is then empty */
KESTREL_API int kprog_linear(void *prog, int x, const void *w, long long ldw, int N, int K, const float *bias, int add_to, int tag);
/* silu(x Wg^T) * (x Wu^T), gate rows first in w [2 ff, K] */
KESTREL_API int kprog_gate_up_swiglu(void *prog, int x, const void *w, long long ldw, int ff, int K, int tag);
/* bias, per-head RMSNorm (weights may be NULL), rotation, K and V into their pages; returns the query register [T, nq * hd] */
KESTREL_API int kprog_attn_prepare(void *prog, int qkv, const float *q_norm_w, const float *k_norm_w, float norm_eps, const float *inv_freq, int rot, int rot_mode, float rot_scale, int group, int page_size, void *k_cache, void *v_cache, int nq, int nkv, int hd, int write_kv, int tag);
/* causal attention of the step's queries over their requests' pages */
KESTREL_API int kprog_attention(void *prog, int q, void *planner, int group, int page_size, int cache_pages, const void *k_cache, const void *v_cache, int nq, int nkv, int hd, int window, float scale, int tag);
/* float32 logits [R, V] = x w^T for the wanted rows: the program's result */
KESTREL_API int kprog_logits(void *prog, int x, const void *w, long long ldw, int V, int K, int tag);
KESTREL_API int kprog_num_ops(void *prog);

/* ---- the runner: a program, a cache manager, buffers for the step description and a workspace ---- */
KESTREL_API void *krunner_create(void *prog, void *cache, int max_tokens, int max_seqs);
KESTREL_API void krunner_destroy(void *runner);
/* flags of kestrel_step_raw */
#define KSTEP_RESERVED 1     /* the caller has reserved the pages already */
#define KSTEP_NO_COMMIT 2    /* the caller commits the cache manager itself */
#define KSTEP_PROFILE 4      /* time the phases of this step with CUDA events (synchronises) */
/* Runs one step: entry e brings counts[e] next tokens of request ids[e] (`tokens`: all entries' ids one after the other);
 * want_counts / wants as in kbatch_pack.  Reserves pages (unless KSTEP_RESERVED), packs and copies the description, runs the
 * program on `stream`, writes float32 logits [R, ld_logits] to `logits` (device memory; may be NULL if R = 0) and commits the
 * requests' new lengths (unless KSTEP_NO_COMMIT).  Nothing is synchronised.  Returns the number of kernels launched, or
 * -1 pages short (nothing ran, nothing changed), other negative codes on errors. */
KESTREL_API int kestrel_step_raw(void *runner, int n, const long long *ids, const int *counts, const int *tokens, const int *want_counts, const int *wants, float *logits, long long ld_logits, int flags, kestrel_stream_t stream);
/* host-to-device bytes of the last step's description */
KESTREL_API long long krunner_last_h2d_bytes(void *runner);
/* milliseconds per phase (KPH_COUNT floats) of the last step run with KSTEP_PROFILE */
KESTREL_API int krunner_phase_ms(void *runner, float *out);
/* bytes of workspace the runner holds */
KESTREL_API long long krunner_workspace_bytes(void *runner);
/* debug checks: nonzero makes every step write guard words behind each register and check them (synchronises); returns the old value */
KESTREL_API int krunner_set_guards(void *runner, int on);
/* registers whose guard words were found damaged since the runner was made */
KESTREL_API int krunner_guard_failures(void *runner);

#endif /* KESTREL_H */
