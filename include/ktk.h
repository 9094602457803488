/*
 * ktk.h -- C ABI of the block top-k paged decode attention library (libktk.so).
 *
 * Hand-written sm_100a CUDA kernels behind plain C entry points: raw device
 * pointers, explicit sizes, a cudaStream_t passed as void*.  No torch types,
 * no exceptions.  Every call only enqueues work on `stream`; none of them
 * synchronises or allocates device memory.
 *
 * Each entry point names the interface of the reference project
 * (Infini-AI-Lab/Kinetics) that it replaces, as file:line inside that project.
 *
 * Data model (all row-major, innermost dimension last):
 *   kv_cache   [num_pages, 2, page_size, Hkv, D]   dtype   (2 = K then V; the
 *              "NHD" paged layout of benchmark/blocktopk_decoder.py:161-164)
 *   summaries  [B, Hkv, summary_stride, D]         dtype   per-page mean key,
 *              indexed by the LOGICAL page number of sequence b
 *              (benchmark/blocktopk_decoder.py:166-168 `compressed_key_cache`)
 *   page table in CSR form, exactly as the reference hands it to flashinfer
 *              (benchmark/blocktopk_decoder.py:141-149):
 *              kv_indices[int32], kv_indptr[int32, B+1], kv_last_page_len[int32, B]
 *              sequence b owns physical pages kv_indices[kv_indptr[b] .. kv_indptr[b+1]),
 *              its last page holds kv_last_page_len[b] in [1, page_size] tokens.
 *   q, o       [B, Hq, D]                          dtype,  Hq = Hkv * G
 *
 * Only D = 128 and page_size = 16 are built; anything else returns
 * KTK_ERR_UNSUPPORTED.
 */
#ifndef KTK_H_
#define KTK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define KTK_API __attribute__((visibility("default")))
#else
#define KTK_API
#endif

/* element types of q / k / v / kv_cache / summaries / o */
#define KTK_F32 0
#define KTK_BF16 1

/* return codes (host side, detected before anything is enqueued) */
#define KTK_OK 0
#define KTK_ERR_ARG (-1)         /* null pointer, negative size, bad enum     */
#define KTK_ERR_UNSUPPORTED (-2) /* head_dim / page_size / group size not built */
#define KTK_ERR_WORKSPACE (-3)   /* workspace too small for the split count    */
#define KTK_ERR_CUDA (-4)        /* a CUDA runtime call failed; see ktk_last_error */
#define KTK_ERR_TOO_LARGE (-5)   /* size beyond a stated maximum                */

/* device-side status word values (written to `status[0]`, first fault wins;
 * the offending access is skipped, the kernel never traps) */
#define KTK_STATUS_OK 0
#define KTK_STATUS_BAD_PAGE 1    /* physical page id outside [0, num_pages)      */
#define KTK_STATUS_BAD_TABLE 2   /* kv_indptr not monotone / last_page_len out of range */
#define KTK_STATUS_TIMEOUT 3     /* a bounded wait on an asynchronous copy gave up       */
#define KTK_STATUS_INTERNAL 4    /* a kernel's own consistency check failed              */

/* decode kernel variants (ktk_sparse_decode / ktk_dense_decode `variant`) */
#define KTK_VARIANT_AUTO 0
#define KTK_VARIANT_SIMT 1       /* fp32 FMA path (the only one for KTK_F32)     */
#define KTK_VARIANT_MMA 2        /* bf16 tensor-core path with TMA-staged pages  */
#define KTK_VARIANT_UMMA 3       /* prefill only: bf16 on tcgen05 with accumulators in tensor memory */

/* num_splits value: cut the concatenated page lists evenly over one CTA per resident slot
 * (bf16 tensor-core path only); see ktk_decode_num_splits */
#define KTK_SPLITS_BALANCED (-1)

typedef struct ktk_shape {
    int32_t batch;          /* B: sequences in this step                         */
    int32_t num_kv_heads;   /* Hkv, local to this GPU                            */
    int32_t group_size;     /* G = Hq / Hkv                                      */
    int32_t head_dim;       /* D, must be 128                                    */
    int32_t page_size;      /* P, must be 16                                     */
    int32_t dtype;          /* KTK_F32 or KTK_BF16                               */
    int64_t num_pages;      /* physical pages in kv_cache (bounds check)         */
} ktk_shape;

/*
 * Optional view of a sequence's pages, for callers whose block grid does not start at token 0
 * or who keep more than the newest page always attended -- the LiteSys semantics of
 * LiteSys/litesys/attention/sparsity_utils.py:24-47 (sink = 4 tokens, `attn_local` newest tokens,
 * 16-token blocks counted from the end of the sink).  A null view means {0, 1, NULL, NULL}: the
 * semantics of benchmark/blocktopk_decoder.py (every full page before the one being filled is
 * scored, that last page is always attended).
 *   sink_tokens  0..15.  When > 0, logical page 0 of every sequence holds only the first
 *                sink_tokens tokens (slots 0..sink_tokens-1); it is never scored and always
 *                attended.  Token t >= sink_tokens lives in logical page 1 + (t - sink_tokens) / 16.
 *   local_tokens L >= 0.  Scored pages are the full pages whose tokens all lie more than L tokens
 *                behind the end: n_dyn = max(0, tokens_after_sink - L) / 16 pages, right after
 *                the sink page; every later page is always attended.
 *   page_count   nullable int32[B]: number of pages of sequence b.  kv_indptr[b] is then only
 *                the start of its list in kv_indices (lists need not be packed), and kv_indptr
 *                needs B entries.
 *   slot_index   nullable int32[B]: row of `summaries` that belongs to sequence b (default b).
 *   seq_order    nullable int32[B], read by ktk_select_v only: a permutation of 0..B-1, the sequences from the
 *                longest to the shortest.  The persistent CTAs then take the sequences in that order, every other
 *                round of CTAs in reverse, so that a ragged batch loads them evenly; results do not depend on it.
 *                An entry outside [0, B) reports KTK_STATUS_BAD_TABLE and leaves that row at -1.
 * Selected-page rows then hold [sink page][<= topk picks][always-attended tail pages], at most
 * ktk_view_row_width(topk, view) entries.
 */
typedef struct ktk_view {
    int32_t sink_tokens;
    int32_t local_tokens;
    const int32_t* page_count;
    const int32_t* slot_index;
    const int32_t* seq_order;
} ktk_view;

/* Entries per (sequence, kv head) row of a selected-page table under `view` (topk + 1 for a null view). */
KTK_API int32_t ktk_view_row_width(int32_t topk, const ktk_view* view);

/* Human-readable text of the last error on the calling thread ("" if none). */
KTK_API const char* ktk_last_error(void);
/* Library version, "major.minor". */
KTK_API const char* ktk_version(void);

/*
 * Paged KV append + page-summary maintenance (decode, one token per sequence).
 * Replaces: torch op mylib::update_kv -> flashinfer.append_paged_kv_cache
 *   (benchmark/blocktopk_decoder.py:23-46, call site :209-213; dense twin
 *   benchmark/dense_decoder.py:21-44) and LiteSys copy_to_cache
 *   (LiteSys/litesys/attention/cache_utils.py:5-51, batch_cache.py:76-84).
 * The page table must already describe the state AFTER the append (flashinfer
 * convention): the token goes to page kv_indices[kv_indptr[b+1]-1], slot
 * kv_last_page_len[b]-1.  If `summaries` is non-null the summary of that
 * (last) logical page is rewritten as the mean of the page's filled keys:
 * fp32 sequential sum over slots 0..c-1, divided by c, rounded to dtype.
 *   k, v: [B, Hkv, D]
 */
KTK_API int ktk_append(const void* k, const void* v, void* kv_cache, void* summaries,
               int64_t summary_stride, const int32_t* kv_indices,
               const int32_t* kv_indptr, const int32_t* kv_last_page_len,
               const ktk_shape* shape, int32_t* status, void* stream);

/*
 * Rebuild the summaries of every page of every sequence from the cache (bulk
 * initialisation after a prefill).  The reference fills `compressed_key_cache`
 * with random numbers (benchmark/blocktopk_decoder.py:166-168); the mean-of-keys
 * definition follows LiteSys/litesys/attention/sparsity_utils.py:37.
 */
KTK_API int ktk_build_summaries(const void* kv_cache, void* summaries, int64_t summary_stride,
                        const int32_t* kv_indices, const int32_t* kv_indptr,
                        const int32_t* kv_last_page_len, const ktk_shape* shape,
                        int32_t* status, void* stream);

/*
 * GQA query x page-summary scoring fused with top-k page selection.
 * Replaces: benchmark/blocktopk_decoder.py:216-221 (einsum + mean, torch.topk,
 *   logical->physical map, always-on last page, int32 cast) and the selection
 *   inside LiteSys/litesys/attention/sparsity_utils.py:24-47.
 * For each (b, kv head): scored pages are the logical pages 0 .. n_pages-2 (every
 * page but the one being filled); score = dot(mean_g q[b, h*G+g, :], summary) in
 * fp32 in a fixed summation order; if their number <= topk all are taken in index
 * order, else the topk largest, descending score, ties to the LOWEST page index;
 * the last page is appended.  Writes cnt = min(topk, n_pages-1) + 1 entries, the
 * rest of the row is -1.
 *   out_pages   [B, Hkv, topk+1] int32  physical page ids        (required)
 *   out_logical [B, Hkv, topk+1] int32  logical page numbers     (nullable)
 *   out_scores  [B, Hkv, summary_stride] fp32 raw scores         (nullable)
 */
KTK_API int ktk_select(const void* q, const void* summaries, int64_t summary_stride,
               const int32_t* kv_indices, const int32_t* kv_indptr,
               const int32_t* kv_last_page_len, int32_t topk, int32_t* out_pages,
               int32_t* out_logical, float* out_scores, const ktk_shape* shape,
               int32_t* status, void* stream);

/*
 * Split count the decode kernels use when the caller passes num_splits = 0, and
 * the workspace size that count needs.  `max_entries` = largest number of pages
 * one (sequence, kv head) attends (topk+1 for sparse, max pages per sequence
 * for dense).  Host-only, no CUDA call except a cached device-attribute query.
 * For bf16 the answer is KTK_SPLITS_BALANCED: the grid is one CTA per resident slot
 * and the concatenation of all page lists (each padded to `max_entries`) is cut into
 * equal chunks, so that every SM finishes at the same time whatever the batch size;
 * a list that crosses a cut is merged by a second small launch.  Its workspace is a
 * few MB (two partial slots per CTA) and does not depend on the batch.  For fp32 the
 * answer is a per-list split count >= 1.
 * flashinfer's analogue is the 128 MB workspace + plan()
 * (benchmark/blocktopk_decoder.py:152, :255-265).
 */
KTK_API int32_t ktk_decode_num_splits(const ktk_shape* shape, int32_t max_entries);
KTK_API size_t ktk_decode_workspace_bytes(const ktk_shape* shape, int32_t num_splits);

/*
 * Flash-decode attention over the selected pages only.
 * Replaces: mylib::decode -> BatchDecodeWithPagedKVCacheWrapper.run
 *   (benchmark/blocktopk_decoder.py:153-160, :171-184, :223-225) and, restricted
 *   to the selected pages, LiteSys qk / softmax / sv
 *   (LiteSys/litesys/attention/cache_utils.py:54-93, :97-130, :135-169).
 * o[b, h*G+g, :] = softmax_s(q . K_s * sm_scale) . V_s over the tokens of the
 * pages listed in sel_pages[b, h, 0..cnt), cnt = min(topk, n_pages-1) + 1; the last
 * listed page is masked to kv_last_page_len[b] tokens.  fp32 accumulation.
 *   num_splits 0 = ktk_decode_num_splits(); > 1 (that many CTAs per list) and
 *   KTK_SPLITS_BALANCED need `workspace` of ktk_decode_workspace_bytes() bytes
 *   (partials + a second combine launch); 1 needs none.
 */
KTK_API int ktk_sparse_decode(const void* q, const void* kv_cache, const int32_t* sel_pages,
                      int32_t topk, const int32_t* kv_indptr,
                      const int32_t* kv_last_page_len, float sm_scale, void* o,
                      void* workspace, size_t workspace_bytes, int32_t num_splits,
                      int32_t variant, const ktk_shape* shape, int32_t* status,
                      void* stream);

/*
 * ktk_sparse_decode for callers that can neither pass a workspace nor let the library
 * allocate one.  No counterpart in the reference: flashinfer takes a caller-allocated
 * 128 MB workspace, and nothing in the reference runs without one.
 *
 * Who needs it: an engine that gave all device memory to its own page pool when it
 * started, so that an allocation made on its behalf would fail or shrink the pool; or a
 * decode loop in which the device-wide synchronisation of cudaMalloc is not acceptable.
 *
 * Same arguments (num_splits = 0 and KTK_SPLITS_BALANCED included) and results as
 * ktk_sparse_decode, minus `workspace`.  The partial results of a split decode go to a
 * 16 MiB array that is part of the library image (ktk_noalloc_scratch_bytes()); every GPU
 * that loads the library keeps that array until the process ends.  What a call needs is
 * ktk_decode_workspace_bytes(): for KTK_SPLITS_BALANCED (what num_splits = 0 means for
 * bf16) a fixed 2 to 4 MB whatever the batch -- two partial slots per resident CTA -- so
 * that case always fits; for an explicit split count batch * Hq * num_splits * 520 bytes,
 * and a call that needs more than the array holds returns KTK_ERR_TOO_LARGE and launches
 * nothing.  The call itself performs no cudaMalloc / cudaFree and uses no allocating
 * library routine.
 *
 * The first call on a device looks up the array's device address (one runtime query, no
 * allocation); make that first call outside any stream capture.  All calls on a device
 * share the one array: two calls whose kernels may overlap on the GPU (different
 * streams) race on it -- keep them on one stream or order them with events.  Nothing in
 * the array has to be cleared between calls.
 */
KTK_API size_t ktk_noalloc_scratch_bytes(void);
KTK_API int ktk_sparse_decode_noalloc(const void* q, const void* kv_cache, const int32_t* sel_pages,
                                      int32_t topk, const int32_t* kv_indptr,
                                      const int32_t* kv_last_page_len, float sm_scale, void* o,
                                      int32_t num_splits, int32_t variant, const ktk_shape* shape,
                                      int32_t* status, void* stream);

/*
 * Dense paged decode over all pages of each sequence (the baseline the sparse
 * path is compared with).  max_pages_per_seq must be >= every sequence's page count
 * (a longer list is clipped and flagged KTK_STATUS_BAD_TABLE by the balanced partition).
 * Replaces: benchmark/dense_decoder.py:149-156, :168-170, :178-189.
 */
KTK_API int ktk_dense_decode(const void* q, const void* kv_cache, const int32_t* kv_indices,
                     const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                     int32_t max_pages_per_seq, float sm_scale, void* o, void* workspace,
                     size_t workspace_bytes, int32_t num_splits, int32_t variant,
                     const ktk_shape* shape, int32_t* status, void* stream);

/*
 * RMSNorm over the last dimension: out = x * rsqrt(mean(x^2) + eps) * w, fp32
 * arithmetic, result in dtype.  x, out: [rows, cols]; w: [cols].
 * Replaces: mylib::layer_norm / mylib::qk_norm -> flashinfer.rmsnorm
 *   (benchmark/model_utils.py:4-25, benchmark/blocktopk_decoder.py:61-85).
 */
KTK_API int ktk_rmsnorm(const void* x, const void* w, float eps, void* out, int64_t rows,
                int32_t cols, int32_t dtype, void* stream);

/*
 * Residual add + RMSNorm in one pass: s = x + residual (rounded to dtype, stored to out_sum when
 * that is non-null), out_norm = s * rsqrt(mean(s^2) + eps) * w.  residual may be null (plain RMSNorm).
 * cols a multiple of 8, at most 8192; pointers 16-byte aligned.
 * Replaces `hidden_states = residual + hidden_states` followed by mylib::layer_norm
 * (benchmark/blocktopk_decoder.py:229-231); flashinfer's own fused form is
 * benchmark/model_utils.py:27-41 (fused_add_rmsnorm, unused by the reference layer).
 */
KTK_API int ktk_add_rmsnorm(const void* x, const void* residual, const void* w, float eps, void* out_sum,
                            void* out_norm, int64_t rows, int32_t cols, int32_t dtype, void* stream);

/*
 * Split of the fused QKV projection with q-norm and k-norm applied on the way:
 * proj [B, (Hq + 2 Hkv) * 128] -> q [B, Hq, 128] (RMSNorm, wq), k [B, Hkv, 128] (RMSNorm, wk),
 * v [B, Hkv, 128] (copied).  Replaces the split / view / contiguous / mylib::qk_norm sequence of
 * benchmark/blocktopk_decoder.py:197-207.
 */
KTK_API int ktk_qkv_norm(const void* proj, const void* wq, const void* wk, float eps, void* q, void* k,
                         void* v, int64_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t dtype,
                         void* stream);

/*
 * The same with the rotary position embedding applied to the normalised query and key heads:
 * x * cos[pos] + rotate_half(x) * sin[pos], rotate_half(x) = (-x[64:], x[:64]), pos = position_ids[b]
 * (clamped to the table).  cos_table / sin_table: [max_positions, 128] in `dtype`; one token per row.
 * Replaces qk_norm + apply_rotary_pos_emb of the LiteSys decode step
 * (LiteSys/litesys/models/qwen3.py:96-102, models/model_utils.py:17-50).
 */
KTK_API int ktk_qkv_norm_rope(const void* proj, const void* wq, const void* wk, float eps, const void* cos_table,
                              const void* sin_table, const int64_t* position_ids, int64_t max_positions, void* q,
                              void* k, void* v, int64_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                              int32_t dtype, void* stream);

/*
 * o_proj all-reduce + residual add + RMSNorm in one kernel over NVLink (bf16).
 * Replaces `dist.all_reduce(hidden_states)` followed by the residual add and the layer norm
 * (LiteSys/litesys/models/qwen3_dist.py:111-114).
 * Every rank holds its partial o_proj output [rows, cols] in a buffer the others can reach, and a
 * `sum` buffer of the same shape.  Two forms, chosen by `mode`:
 *   KTK_ALLREDUCE_MULTICAST  the buffers are bound to NVSwitch multicast objects; the switch adds the
 *                            partials (multimem.ld_reduce) and replicates the sums (multimem.st).
 *                            Needs x_multicast, sum_multicast.
 *   KTK_ALLREDUCE_PEER       plain peer loads and stores; needs x_peer_ptrs, sum_peer_ptrs: device
 *                            arrays of `world` pointers to every rank's buffer (own included).
 *                            Built for 2 and 4 ranks.
 *   KTK_ALLREDUCE_AUTO       peer form at 2 and 4 ranks (a rank's own share would otherwise cross the
 *                            switch and come back), multicast form above, given the pointers each needs.
 *   residual, w      local [rows, cols] (identical on all ranks), [cols]
 *   sum_local        this rank's own `sum` buffer: receives residual + sum of the partials, all rows
 *   norm_local       local [rows, cols]: receives RMSNorm of that sum (computed on every rank)
 *   flag_ptrs        device array of `world` pointers: rank p's flag words, uint32[grid * world],
 *                    zero before the first launch, reachable from every rank (peer memory)
 *   launch_count     local uint32[grid], zero before the first launch (kept by the kernel)
 * grid = ktk_allreduce_grid(rows, world).  rows must divide by world; cols a multiple of 8, <= 8192.
 * Rank r reduces rows [r*rows/world, (r+1)*rows/world) and sends their sum to every rank; every rank
 * normalises all rows into its own `norm_local`.  The ranks meet in bounded flag waits before the
 * reduction and after the sums were sent (expiry: KTK_STATUS_TIMEOUT in `status`).
 * All ranks must launch it the same number of times with the same shape and mode.
 */
#define KTK_ALLREDUCE_AUTO 0
#define KTK_ALLREDUCE_MULTICAST 1
#define KTK_ALLREDUCE_PEER 2
KTK_API int32_t ktk_allreduce_grid(int64_t rows, int32_t world);
KTK_API int ktk_allreduce_add_rmsnorm(const void* x_multicast, const void* x_peer_ptrs, const void* residual,
                                      const void* w, void* sum_multicast, const void* sum_peer_ptrs,
                                      const void* sum_local, void* norm_local, const void* flag_ptrs,
                                      void* launch_count, int32_t rank, int32_t world, int64_t rows,
                                      int32_t cols, float eps, int32_t mode, int32_t* status, void* stream);

/*
 * Both exchanges of the tensor-parallel layer, row-pipelined (the loads of a CTA's next row are in
 * flight while it sends the sums of the current one, and rows received from the other ranks are
 * normalised as their flags arrive).  Same buffers, pointer tables and rank/row ownership as
 * ktk_allreduce_add_rmsnorm; `result` chooses what every rank ends up with:
 *   KTK_EXCHANGE_ALLREDUCE_NORM  out_local = residual + sum of the partials (all rows, `out_local` is this
 *                                rank's own `sum` buffer), norm_local = its RMSNorm.  Replaces
 *                                dist.all_reduce + residual add + layer_norm
 *                                (LiteSys/litesys/models/qwen3_dist.py:111-114); between stacked layers also the
 *                                down_proj all-reduce + residual add (:120-122) followed by the next layer's
 *                                input layer_norm (:91).
 *   KTK_EXCHANGE_ALLREDUCE       the same without the norm (w, norm_local may be null): the down_proj
 *                                all-reduce + residual add (:120-122).
 *   KTK_EXCHANGE_SCATTER         reduce-scatter: out_local (any local [rows, cols] buffer) receives
 *                                residual + sum for the rows [rank*rows/world, (rank+1)*rows/world) only;
 *                                nothing is sent back.  sum_multicast / sum_peer_ptrs may be null.
 * flag_ptrs: rank p's flag words, uint32[ktk_exchange_grid() * world], zero before the first launch;
 * launch_count: local uint32[ktk_exchange_grid()], zero before the first launch (ktk_exchange_grid is an
 * upper bound of the CTAs any form launches).  A set of flags belongs
 * to one (shape, mode, result) for its whole life.  cols a multiple of 8, <= 8192.
 */
#define KTK_EXCHANGE_ALLREDUCE_NORM 0
#define KTK_EXCHANGE_ALLREDUCE 1
#define KTK_EXCHANGE_SCATTER 2
KTK_API int32_t ktk_exchange_grid(int64_t rows, int32_t world);
KTK_API int ktk_exchange_rows(const void* x_multicast, const void* x_peer_ptrs, const void* residual,
                              const void* w, void* sum_multicast, const void* sum_peer_ptrs, void* out_local,
                              void* norm_local, const void* flag_ptrs, void* launch_count, int32_t rank,
                              int32_t world, int64_t rows, int32_t cols, float eps, int32_t mode,
                              int32_t result, int32_t* status, void* stream);

/*
 * A barrier of the ranks as a one-CTA kernel in `stream`: work enqueued after it on any rank starts only
 * when every rank's stream has reached its own barrier launch (and that rank's earlier writes, peer
 * copies included, are visible).  For host-side pipelines that hand buffers between ranks with copy
 * engines; the layer kernels carry their own flags.  No reference counterpart (the reference's ranks
 * meet inside NCCL collectives, LiteSys/litesys/models/qwen3_dist.py:112,121).
 *   flag_ptrs     device array of `world` pointers: rank p's uint32[world] flag words, zero before the
 *                 first launch, reachable from every rank
 *   launch_count  local uint32[1], zero before the first launch
 * The wait is bounded (about a second): on expiry KTK_STATUS_TIMEOUT goes to `status` and the kernel returns.
 */
KTK_API int ktk_rank_barrier(const void* flag_ptrs, void* launch_count, int32_t rank, int32_t world,
                             int32_t* status, void* stream);

/*
 * SwiGLU gate: out = silu(gate) * up, elementwise, fp32 arithmetic.
 * Replaces the activation + multiply of benchmark/blocktopk_decoder.py:235-236.
 */
KTK_API int ktk_silu_mul(const void* gate, const void* up, void* out, int64_t n, int32_t dtype,
                 void* stream);
/*
 * The same over [rows, cols] operands whose rows lie in_row_stride elements apart -- the two halves of ONE GEMM
 * output [rows, 2 * cols] when gate_proj and up_proj (benchmark/blocktopk_decoder.py:235, LiteSys qwen3.py:81-83)
 * are multiplied as one stacked weight.  `out` is contiguous [rows, cols]; cols a multiple of 8, rows 16-byte aligned.
 */
KTK_API int ktk_silu_mul_rows(const void* gate, const void* up, void* out, int64_t rows, int64_t cols,
                              int64_t in_row_stride, int32_t dtype, void* stream);

/*
 * The same four operations under a ktk_view (null view = the plain entry points above).
 * Replace, in the LiteSys decode path: copy_to_cache + kv_offset update
 * (LiteSys/litesys/attention/batch_cache.py:76-84), the selection inside blockwise_topk_sparsity
 * (sparsity_utils.py:24-47, reached through attn_logits_processor :217-249), and qk / softmax / sv
 * (cache_utils.py:173-226) restricted to the kept tokens; dense when the view keeps everything
 * (layers listed in attn_layer_skip, sparsity_utils.py:211,221-222).
 * `out_pages` / `sel_pages` rows are `row_width` ints wide (>= ktk_view_row_width()).
 */
KTK_API int ktk_append_v(const void* k, const void* v, void* kv_cache, void* summaries,
                         int64_t summary_stride, const int32_t* kv_indices, const int32_t* kv_indptr,
                         const int32_t* kv_last_page_len, const ktk_view* view, const ktk_shape* shape,
                         int32_t* status, void* stream);
/*
 * Append several tokens per sequence (prefill, chunked append) and refresh the summaries of the
 * pages they touch.  k, v: [total_tokens, Hkv, D] packed by sequence; append_indptr int32[B+1] gives
 * each sequence's range, exactly the `kv_append_indptr` argument of mylib::update_kv ->
 * flashinfer.append_paged_kv_cache (benchmark/blocktopk_decoder.py:23-46); the page table describes
 * the state after the append.  Also the write half of the LiteSys prefill
 * (LiteSys/litesys/attention/batch_cache.py:123-127).  `view` may be null.
 */
KTK_API int ktk_append_tokens(const void* k, const void* v, const int32_t* append_indptr, int64_t total_tokens,
                              void* kv_cache, void* summaries, int64_t summary_stride,
                              const int32_t* kv_indices, const int32_t* kv_indptr,
                              const int32_t* kv_last_page_len, const ktk_view* view, const ktk_shape* shape,
                              int32_t* status, void* stream);
/*
 * Chunked causal prefill attention over the paged cache: the new tokens of every sequence (already in their
 * pages, see ktk_append_tokens) attend their sequence's history up to their own position.
 * Replaces flashinfer.single_prefill_with_kv_cache(q, k_cache[:total], v_cache[:total], causal=True)
 * (LiteSys/litesys/attention/batch_cache.py:129-145), which the reference calls for one sequence at a time on a
 * contiguous cache; here the pages are read through the table where they lie and one launch serves the batch.
 *   q, o             [total_new_tokens, Hq, D] packed by sequence; q_indptr int32[B+1] gives each sequence's
 *                    range (the append_indptr of ktk_append_tokens); shape->batch = B
 *   max_new_tokens   an upper bound of the new tokens of any one sequence (sizes the grid; host value)
 *   page table       the state AFTER the append: sequence b holds n tokens in all, its new tokens are the
 *                    last q_indptr[b+1] - q_indptr[b] of them.  `view` as for the other entry points (sink page,
 *                    page_count); local_tokens plays no part, every visible token is attended.
 *   variant          KTK_VARIANT_AUTO: tensor cores for bf16 with a group size of 1, 2, 4 or 8 -- the tcgen05
 *                    kernel (KTK_VARIANT_UMMA: one CTA per sequence, kv head and tile of 128 / G tokens, history
 *                    in blocks of 64 keys, S and O accumulated in tensor memory); KTK_VARIANT_MMA asks for the
 *                    earlier mma.sync kernel (tiles of 32 / G tokens, each page staged once per tile by TMA);
 *                    otherwise, and for KTK_VARIANT_SIMT, every new token runs as one row of the dense paged
 *                    decode with its own horizon, which needs `workspace` of ktk_prefill_workspace_bytes()
 *                    bytes (three ints per new token).
 */
KTK_API size_t ktk_prefill_workspace_bytes(int64_t total_new_tokens, int32_t dtype, int32_t variant);
KTK_API int ktk_prefill_attention(const void* q, const int32_t* q_indptr, int64_t total_new_tokens,
                                  int32_t max_new_tokens, const void* kv_cache, const int32_t* kv_indices,
                                  const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                                  const ktk_view* view, float sm_scale, void* o, void* workspace,
                                  size_t workspace_bytes, int32_t variant, const ktk_shape* shape,
                                  int32_t* status, void* stream);
KTK_API int ktk_build_summaries_v(const void* kv_cache, void* summaries, int64_t summary_stride,
                                  const int32_t* kv_indices, const int32_t* kv_indptr,
                                  const int32_t* kv_last_page_len, const ktk_view* view,
                                  const ktk_shape* shape, int32_t* status, void* stream);
KTK_API int ktk_select_v(const void* q, const void* summaries, int64_t summary_stride,
                         const int32_t* kv_indices, const int32_t* kv_indptr,
                         const int32_t* kv_last_page_len, int32_t topk, const ktk_view* view,
                         int32_t row_width, int32_t* out_pages, int32_t* out_logical, float* out_scores,
                         const ktk_shape* shape, int32_t* status, void* stream);
KTK_API int ktk_sparse_decode_v(const void* q, const void* kv_cache, const int32_t* sel_pages,
                                int32_t topk, const ktk_view* view, int32_t row_width,
                                const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                                float sm_scale, void* o, void* workspace, size_t workspace_bytes,
                                int32_t num_splits, int32_t variant, const ktk_shape* shape,
                                int32_t* status, void* stream);
KTK_API int ktk_dense_decode_v(const void* q, const void* kv_cache, const int32_t* kv_indices,
                               const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                               const ktk_view* view, int32_t max_pages_per_seq, float sm_scale, void* o,
                               void* workspace, size_t workspace_bytes, int32_t num_splits,
                               int32_t variant, const ktk_shape* shape, int32_t* status, void* stream);

/*
 * The LiteSys decode chain function by function, on its own layout: unpaged key / value caches
 * [max_batch, Hkv, max_len, D] and an fp32 logits buffer [rows, Hq, max_len] handed from step to step.
 * For code written against those functions; they read every key and value of a sequence, which the
 * paged kernels above avoid.  `offset` is indexed by the row of the active batch, the cache slot is
 * batch_idx[row], exactly as in the reference kernels (cache_utils.py:67,106,149).
 *   ktk_copy_to_cache    copy_to_cache (LiteSys/litesys/attention/cache_utils.py:5-51): src row `row`, head h
 *                        (strides in elements) -> cache[batch_id[row], h, offset[row], :]
 *   ktk_qk               qk (:54-93, :173-190): logits[row, hq, s] = q . K[s] / sqrt(D) for s < offset[row],
 *                        -inf up to the end of the last block of `block_seq` positions it touches
 *   ktk_block_topk_mask  blockwise_topk_sparsity (sparsity_utils.py:24-47), block size 16: rows longer than
 *                        ceil16(sink + local + 16 * topk_block) keep the sink, the topk_block best blocks of the
 *                        region behind it (mean logit over the query group and the block; ties to the lower
 *                        block) and the tail; the rest of the region becomes -inf
 *   ktk_softmax_rows     softmax (cache_utils.py:97-130, :216-226): in place over s < offset[row]
 *   ktk_sv               sv (:135-169, :193-212): out[row, hq, :] = sum_s p[row, hq, s] * V[s, :], in the cache dtype
 * A slot or position outside the cache sets KTK_STATUS_BAD_TABLE and skips the access.
 */
KTK_API int ktk_copy_to_cache(void* cache, const void* src, const int64_t* batch_id, const int32_t* offset,
                              int32_t rows, int32_t num_kv_heads, int64_t max_batch, int64_t max_len,
                              int32_t head_dim, int64_t src_row_stride, int64_t src_head_stride, int32_t dtype,
                              int32_t* status, void* stream);
KTK_API int ktk_qk(const void* q, const void* key_cache, const int64_t* batch_idx, const int32_t* offset,
                   float* logits, int32_t rows, int32_t num_q_heads, int32_t num_kv_heads, int64_t max_batch,
                   int64_t max_len, int32_t head_dim, int32_t block_seq, int32_t dtype, int32_t* status,
                   void* stream);
KTK_API int ktk_block_topk_mask(float* logits, const int32_t* offset, int32_t rows, int32_t num_q_heads,
                                int32_t num_kv_heads, int64_t max_len, int32_t topk_block, int32_t local,
                                int32_t sink, int32_t* status, void* stream);
KTK_API int ktk_softmax_rows(float* logits, const int32_t* offset, int32_t rows, int32_t num_q_heads,
                             int64_t max_len, void* stream);
KTK_API int ktk_sv(const void* value_cache, const int64_t* batch_idx, const int32_t* offset, const float* probs,
                   void* out, int32_t rows, int32_t num_q_heads, int32_t num_kv_heads, int64_t max_batch,
                   int64_t max_len, int32_t head_dim, int32_t dtype, int32_t* status, void* stream);

/*
 * Token-level top-k sparsity and the paged forms of the steps around it (the LiteSys decode chain with
 * attn_topk instead of attn_block_topk, LiteSys/litesys/attention/batch_cache.py:154-168).
 *   ktk_token_topk_mask  topk_sparsity (sparsity_utils.py:6-21): rows longer than sink + topk + local keep the
 *                        sink, the `local` newest tokens and the topk tokens of the region between them with the
 *                        largest logit averaged over the query group (ties to the lower position); the rest of
 *                        that region becomes -inf for every head of the group.  logits fp32 [rows, Hq, max_len],
 *                        offset[row] = tokens of the row.  max_len - sink - local <= 49152.
 *   ktk_paged_qk         qk (cache_utils.py:173-190) over a paged cache: logits[row, hq, s] = sm_scale * q . K[s]
 *                        for s < tokens(row), the keys read through the page table (and `view`: sink page,
 *                        page_count).  Positions behind the row's length are left as they are.
 *   ktk_paged_sv         sv (cache_utils.py:193-212) over a paged cache: out[row, hq, :] = sum_s p[row, hq, s] * V[s];
 *                        value rows whose probability is zero for the whole query group are not read.
 * Between them ktk_softmax_rows applies unchanged.
 */
KTK_API int ktk_token_topk_mask(float* logits, const int32_t* offset, int32_t rows, int32_t num_q_heads,
                                int32_t num_kv_heads, int64_t max_len, int32_t topk, int32_t local, int32_t sink,
                                int32_t* status, void* stream);
KTK_API int ktk_paged_qk(const void* q, const void* kv_cache, const int32_t* kv_indices, const int32_t* kv_indptr,
                         const int32_t* kv_last_page_len, const ktk_view* view, float sm_scale, float* logits,
                         int64_t max_len, const ktk_shape* shape, int32_t* status, void* stream);
KTK_API int ktk_paged_sv(const void* kv_cache, const int32_t* kv_indices, const int32_t* kv_indptr,
                         const int32_t* kv_last_page_len, const ktk_view* view, const float* probs, int64_t max_len,
                         void* out, const ktk_shape* shape, int32_t* status, void* stream);

/*
 * Host-side page pool for continuous batching.  No CUDA call, no device memory: the pool decides
 * which physical pages of the KV cache a sequence slot owns and writes the CSR arrays the kernels
 * read.  The reference has no counterpart: its benchmark uses one static interleaved table
 * (benchmark/blocktopk_decoder.py:141) and its engine reserves max_seq_len tokens of cache per slot
 * (LiteSys/litesys/attention/batch_cache.py:32-40); the engine loop it serves is
 * LiteSys/litesys/engine/engine.py:167-242.
 *   admit    slot takes ceil(n_tokens / page) pages now and is promised ceil(max_total_tokens / page):
 *            pages promised to one sequence are not handed to another, so `extend` inside the promise
 *            cannot fail.  KTK_ERR_TOO_LARGE (nothing changed) when the pool cannot promise that much.
 *   extend   every listed slot grows by tokens_each tokens (a decode step: 1), taking a new page when it
 *            crosses a page boundary; all or nothing.
 *   release  the slot's pages go back to the pool.
 *   export   for the listed slots, in that order: kv_indices (their pages, concatenated), kv_indptr
 *            [n + 1], kv_last_page_len [n] into host memory of the caller; returns the number of
 *            entries written to kv_indices, or a negative error.
 * Not thread-safe: one pool, one scheduling thread.
 */
typedef struct ktk_pool ktk_pool;
KTK_API ktk_pool* ktk_pool_create(int64_t num_pages, int32_t max_slots, int32_t page_size);
KTK_API void ktk_pool_destroy(ktk_pool* pool);
KTK_API int64_t ktk_pool_free_pages(const ktk_pool* pool);               /* free and not promised */
KTK_API int64_t ktk_pool_slot_tokens(const ktk_pool* pool, int32_t slot);  /* -1: slot not in use */
KTK_API int64_t ktk_pool_slot_pages(const ktk_pool* pool, int32_t slot);
KTK_API int ktk_pool_admit(ktk_pool* pool, int32_t slot, int64_t n_tokens, int64_t max_total_tokens);
KTK_API int ktk_pool_extend(ktk_pool* pool, const int32_t* slots, int32_t n, int32_t tokens_each);
KTK_API int ktk_pool_release(ktk_pool* pool, int32_t slot);
KTK_API int64_t ktk_pool_export(const ktk_pool* pool, const int32_t* slots, int32_t n, int32_t* kv_indices,
                                int64_t indices_capacity, int32_t* kv_indptr, int32_t* kv_last_page_len);

#ifdef __cplusplus
}
#endif
#endif /* KTK_H_ */
