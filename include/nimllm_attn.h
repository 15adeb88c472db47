/* nimllm_attn.h -- C ABI of the B200 (sm_100a) grouped-query attention path for nimllm.
 *
 * This is the boundary the Nim host code binds with {.importc, cdecl.}, the way
 * src/gpu.nim:219-328 binds src/kernels.cu today.  Conventions follow the
 * reference: raw device pointers, runtime int shapes, no structs, the caller owns
 * every buffer, nothing is allocated per call, no host synchronisation inside.
 * Unlike the reference's void launchers every new entry point returns an int
 * status (0 = ok) that Nim may `discard`; nimllm_attn_last_error() explains it.
 * `stream` is a cudaStream_t passed as void*; NULL is the legacy default stream
 * the reference launches everything on (src/gpu.nim:166-175).
 *
 * Stream order: every entry point behaves as a plain stream-ordered launch.  Internally the decode and
 * projection kernels are launched with programmatic stream serialization and wait on the device for the
 * kernel before them before they read an input or write an output, so that back-to-back calls of this
 * library overlap their launch latencies; nothing is required of the caller.
 *
 * Tensor layouts are the reference's: activations are row-major [tokens, heads*D]
 * with heads as column blocks of width D (src/model.nim:487-497); a KV head of
 * the cache is a dense row-major [rows, D] block with K stored AFTER RoPE and V
 * raw (src/model.nim:797-815); query head h reads KV head h / (Hq/Hkv)
 * (src/kernels.cu:447, src/model.nim:823).
 */
#ifndef NIMLLM_ATTN_H
#define NIMLLM_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of activations / cache */
#define NIMLLM_F32 0
#define NIMLLM_BF16 1

/* status codes */
#define NIMLLM_OK 0
#define NIMLLM_ERR_ARG 1         /* null pointer, bad shape */
#define NIMLLM_ERR_UNSUPPORTED 2 /* head_dim / dtype / group size without a kernel */
#define NIMLLM_ERR_WORKSPACE 3   /* caller-provided workspace too small */
#define NIMLLM_ERR_CUDA 4        /* launch or runtime error; see last_error */

/* Message for the calling thread's most recent non-zero status ("" if none). */
const char *nimllm_attn_last_error(void);
int nimllm_attn_version(void);

/* ---- RoPE tables -----------------------------------------------------------
 * Replaces the host loop of src/model.nim:153-163: cos/sin [max_pos, D/2] fp32,
 * theta = float(pos) / powf(base, 2f/D), filled on the HOST (upload them the way
 * initModel does).  base is a run-time value (the reference bakes ropeTheta in
 * at compile time, src/model.nim:22). */
int nimllm_rope_tables_host(float *cos_tab, float *sin_tab, int max_pos, int head_dim, float base);

/* ---- KV cache: contiguous layout ---------------------------------------------
 * Replaces KvCache / initKvCache / resetKvCache (src/model.nim:70-73,729-746).
 * The reference makes 2*nLayer*nKvHead separate cudaMallocs of [blockSize, D]
 * fp32.  Here K and V are ONE allocation each, [n_layer][n_seq][Hkv][max_seq][D]
 * of `dtype`, zero-filled; a (layer, sequence, KV head) block is the same dense
 * [max_seq, D] rows the reference's per-head buffer is.  The handle also keeps
 * the host-side `pos` of the reference's KvCache.  create/destroy allocate and
 * free and are set-up calls, not hot-path calls. */
typedef struct nimllm_kvcache nimllm_kvcache;
nimllm_kvcache *nimllm_kvcache_create(int n_layer, int n_seq, int n_kv_head, int max_seq,
                                      int head_dim, int dtype);
void nimllm_kvcache_destroy(nimllm_kvcache *kv);
int nimllm_kvcache_reset(nimllm_kvcache *kv, void *stream); /* zero-fill, pos = 0 */
void *nimllm_kvcache_k(const nimllm_kvcache *kv, int layer); /* [n_seq][Hkv][max_seq][D] */
void *nimllm_kvcache_v(const nimllm_kvcache *kv, int layer);
int nimllm_kvcache_pos(const nimllm_kvcache *kv);
void nimllm_kvcache_set_pos(nimllm_kvcache *kv, int pos);
int64_t nimllm_kvcache_seq_stride(const nimllm_kvcache *kv);  /* elements: Hkv*max_seq*D */
int64_t nimllm_kvcache_head_stride(const nimllm_kvcache *kv); /* elements: max_seq*D */

/* ---- fused RoPE + cast + cache append ------------------------------------------
 * Replaces, in one launch, ropeFwd(q) and ropeFwd(kNew) (src/model.nim:796-797 via
 * src/kernels.cu:399-423) and the per-KV-head append of src/model.nim:799-815
 * (2*Hkv cudaMemcpy D2D for one token, gpu_extract_kv_head for several).
 *
 *   q      [B, n, Hq*D] act_dtype, rotated IN PLACE (NULL: skip)
 *   k_new  [B, n, Hkv*D] act_dtype; rotated copy goes to the cache; it is also
 *          written back in place when write_back_k != 0 (the reference always
 *          rotates in place)
 *   v_new  [B, n, Hkv*D] act_dtype, copied raw
 *   rope_cos / rope_sin  full tables [>= max position + 1, D/2]; both NULL: no rotation
 *   seq_pos  DEVICE int32 [B], absolute position of each sequence's first new
 *          token, or NULL: every sequence starts at pos0 (the reference's kv.pos)
 *   k_cache / v_cache  cache_dtype; sequence b's block starts at element
 *          kv_off[b] (DEVICE int64 [B]) or, with kv_off NULL, at b*seq_stride;
 *          KV head h follows at h*head_stride; cache row = position - cache_row0;
 *          rows outside [0, max_seq) are not stored (a KV-sequence shard keeps only
 *          its own rows).  Both NULL: rotate only.
 */
int nimllm_rope_append(void *q, int n_head, void *k_new, const void *v_new, int act_dtype,
                       int write_back_k, const float *rope_cos, const float *rope_sin,
                       const int32_t *seq_pos, int pos0, void *k_cache, void *v_cache,
                       int cache_dtype, const int64_t *kv_off, int64_t seq_stride,
                       int64_t head_stride, int cache_row0, int max_seq, int batch, int n,
                       int n_kv_head, int head_dim, void *stream);

/* ---- GQA decode -----------------------------------------------------------------
 * Replaces the per-query-head loop of src/model.nim:822-840 (cublasSgemm_v2 [1,D]x
 * [L,D]^T, gpu_scale, gpu_softmax_fwd, cublasSgemm_v2 [1,L]x[L,D]; 4 launches per
 * query head) for a whole batch of sequences: each KV head is read once for all of
 * its Hq/Hkv query heads, the KV sequence is split into chunks whose partial
 * (max, sum, output) triples are merged by log-sum-exp.
 *
 *   q        [B, Hq*D] q_dtype, already rotated
 *   seq_len  DEVICE int32 [B], rows to attend (the reference's pos + 1), or NULL:
 *            every sequence attends max_len rows
 *   max_len  host upper bound of seq_len (sizes the grid and the workspace)
 *   out      [B, Hq*D] out_dtype (may be NULL when partials_out is given)
 *   partials_out  optional fp32 [B*Hq, D+4] records {o[D] normalised, m, l, 0, 0}
 *            with m = max of the scaled scores and l = sum exp(s - m): what a
 *            KV-sequence shard hands to nimllm_attn_combine
 *   chunk_rows  KV rows per split; 0 = choose
 *   workspace   nimllm_attn_decode_workspace_bytes(...) bytes, 256-byte aligned
 *   Cache rows are read 16 bytes at a time: k_cache / v_cache, seq_stride, head_stride and every
 *   kv_off[b] must be multiples of 16 bytes (8 bf16 or 4 fp32 elements); the host-visible ones are
 *   checked (NIMLLM_ERR_ARG), the device array kv_off cannot be.
 */
size_t nimllm_attn_decode_workspace_bytes(int batch, int n_head, int n_kv_head, int head_dim,
                                          int max_len, int chunk_rows);
int nimllm_attn_decode(const void *q, int q_dtype, const void *k_cache, const void *v_cache,
                       int cache_dtype, const int64_t *kv_off, int64_t seq_stride,
                       int64_t head_stride, const int32_t *seq_len, int max_len, void *out,
                       int out_dtype, float *partials_out, int batch, int n_head,
                       int n_kv_head, int head_dim, float scale, int chunk_rows,
                       void *workspace, size_t workspace_bytes, void *stream);

/* How the library's own split (chunk_rows = 0, bf16 cache) would cut a batch, computed on the
 * host with the arithmetic the kernels use; no GPU involved.  The batch is one list of row units
 * (`unit` rows: 32 at head_dim 64, 16 at 128) ordered by sequence, KV head, row, cut into equal
 * spans for `warps` workers.  segs_out receives 6 ints per segment (worker, sequence, KV head,
 * first unit, end unit, record slot or -1 when the worker covers the whole (sequence, KV head)
 * pair), pairs_out (optional) 3 ints per pair (first worker, pieces, slot of the first piece).
 * Returns the number of segments, or -1 when max_segs is too small or an argument is bad.
 * No counterpart in the reference. */
int nimllm_attn_decode_plan(const int32_t *lens, int batch, int n_kv_head, int unit, int warps,
                            int32_t *segs_out, int max_segs, int32_t *pairs_out);

/* ---- decode over a paged KV cache ---------------------------------------------------------
 * No counterpart in the reference, whose cache is one buffer per (layer, KV head)
 * (src/model.nim:729-739); this is the block-managed cache its chat loop's multi-turn reuse
 * asks for (src/chat.nim:57,86-91).  K and V live in pages of page_rows rows:
 *   k_pages, v_pages  bf16 [n_pages][n_kv_head][page_rows][head_dim]
 *   page_table        device int32 [batch, max_pages]: rows r*page_rows .. of sequence b are in
 *                     page page_table[b][r] (entries past the sequence's length are not read)
 *   page_rows         a power of two >= 32
 * Everything else as nimllm_attn_decode with chunk_rows = 0 (the library's own split of the
 * batch); workspace of nimllm_attn_decode_workspace_bytes(batch, n_head, n_kv_head, head_dim,
 * max_len, 0) bytes.  New rows are appended with nimllm_rope_append_paged below.
 */
int nimllm_attn_decode_paged(const void *q, int q_dtype, const void *k_pages, const void *v_pages,
                             const int32_t *page_table, int max_pages, int page_rows,
                             const int32_t *seq_len, int max_len, void *out, int out_dtype,
                             float *partials_out, int batch, int n_head, int n_kv_head, int head_dim,
                             float scale, void *workspace, size_t workspace_bytes, void *stream);

/* ---- fused RoPE + cast + append into a paged KV cache --------------------------------------
 * No counterpart in the reference (see above).  nimllm_rope_append with the cache given as
 * pages: the row at position p of sequence b goes to row p % page_rows of page
 * page_table[b][p / page_rows], so an append of several tokens may cross page boundaries.
 * Positions at or past max_pages * page_rows, table entries < 0 and pages >= n_pages (the size
 * of the pool) are not stored -- nothing is ever written outside the pool.
 *   k_pages, v_pages  cache_dtype [n_pages][n_kv_head][page_rows][head_dim]
 *   page_rows         a power of two (>= 32 for nimllm_attn_decode_paged)
 * q, k_new, v_new, the tables, seq_pos / pos0, write_back_k as in nimllm_rope_append. */
int nimllm_rope_append_paged(void *q, int n_head, void *k_new, const void *v_new, int act_dtype,
                             int write_back_k, const float *rope_cos, const float *rope_sin,
                             const int32_t *seq_pos, int pos0, void *k_pages, void *v_pages, int cache_dtype,
                             const int32_t *page_table, int max_pages, int page_rows, int n_pages, int batch,
                             int n, int n_kv_head, int head_dim, void *stream);

/* ---- block manager of the paged KV cache ----------------------------------------------------
 * Replaces the reference's cache policy: one conversation, one [blockSize, D] buffer per
 * (layer, KV head), everything dropped when the next turn would not fit (src/chat.nim:86-91,
 * resetKvCache at src/model.nim:741-743).  A pool owns n_pages pages per layer, shared by up to
 * max_seqs sequences; a sequence holds ceil(rows / page_rows) of them, a finished one gives them
 * back, and a request that does not fit is refused alone (NIMLLM_ERR_WORKSPACE, nothing changed)
 * so the caller can release a sequence of its choosing.  All layers of a sequence use the same
 * page numbers, so there is ONE table.  Host bookkeeping only, no kernel of its own:
 *   create(..., on_device)   on_device = 1 allocates K and V pages (zero-filled) and the device
 *                            table; 0 keeps only the host table (callers that own the memory, and
 *                            machines without a GPU) -- k(), v() and table() then return NULL
 *   reserve(seq, rows_total) pages for rows 0 .. rows_total-1 of sequence slot `seq`; never shrinks
 *   release(seq)             all pages of the slot back to the free list
 *   sync(stream)             uploads the table rows changed since the last sync, on `stream`,
 *                            before the launches that read them
 *   table(first_seq)         device int32 [max_seqs - first_seq][max_pages]: the page_table
 *                            argument of the two paged entry points for the batch of sequence
 *                            slots first_seq, first_seq+1, ...  (entries without a page are -1)
 *   k(layer), v(layer)       [n_pages][n_kv_head][page_rows][head_dim] of that layer
 * Not thread-safe: one pool, one calling thread at a time. */
typedef struct nimllm_kvpool nimllm_kvpool;
nimllm_kvpool *nimllm_kvpool_create(int n_layer, int n_pages, int page_rows, int n_kv_head, int head_dim,
                                    int dtype, int max_seqs, int max_pages_per_seq, int on_device);
void nimllm_kvpool_destroy(nimllm_kvpool *pool);
int nimllm_kvpool_reserve(nimllm_kvpool *pool, int seq, int rows_total);
int nimllm_kvpool_release(nimllm_kvpool *pool, int seq);
int nimllm_kvpool_sync(nimllm_kvpool *pool, void *stream);
int nimllm_kvpool_free_pages(const nimllm_kvpool *pool);
int nimllm_kvpool_seq_pages(const nimllm_kvpool *pool, int seq);
int nimllm_kvpool_seq_rows(const nimllm_kvpool *pool, int seq);
const int32_t *nimllm_kvpool_table_host(const nimllm_kvpool *pool);
const int32_t *nimllm_kvpool_table(const nimllm_kvpool *pool, int first_seq);
void *nimllm_kvpool_k(const nimllm_kvpool *pool, int layer);
void *nimllm_kvpool_v(const nimllm_kvpool *pool, int layer);

/* ---- GQA decode for callers that cannot allocate ------------------------------------
 * No counterpart in the reference.  Same computation and arguments as nimllm_attn_decode,
 * minus the workspace: the chunk records of split sequences go to a fixed 8 MiB array that
 * lives inside the library (every GPU that loads the library carries it until the process
 * exits).  It exists for host code that has no device memory to hand over when the call is
 * made: nimllm sizes its scratch arena once at start-up and bump-allocates from it
 * (src/autograd.nim:16-65), so a decode step that arrives when the arena is exhausted, or a
 * caller that must not touch cudaMalloc because it synchronises the device, can still run.
 * The function itself never allocates or frees.
 *   - A call is refused with NIMLLM_ERR_WORKSPACE only when its records fit the array under
 *     neither kernel.  With chunk_rows = 0, a bf16 cache and Hq/Hkv <= 8 the library's own split
 *     of the batch keeps a fixed number of records that depends on the head shape alone
 *     (about 2 MB at 9q/3kv heads of 64, 5 MB at 32q/8kv heads of 128, 10 MB -- too much -- at
 *     Hq/Hkv = 8 with heads of 128).  If that does not fit, or chunk_rows > 0, the chunk grid
 *     runs and needs ceil(max_len / chunk_rows) * batch * n_head * (head_dim + 4) * 4 bytes
 *     (nothing when no sequence is split; with chunk_rows = 0 the library picks the chunk length).
 *     nimllm_attn_decode_noalloc_max_bytes() is the size of the array (8 MiB).
 *   - The first call on each device looks the array's device address up
 *     (cudaGetSymbolAddress); make that first call outside any stream capture.
 *   - All calls on a device share the array, and it keeps what the last call left there
 *     (nothing in it needs clearing: every record is written before it is read).  Two calls
 *     that may overlap on the GPU -- different streams, no ordering between them -- race on
 *     it; give such calls their own workspace through nimllm_attn_decode instead. */
size_t nimllm_attn_decode_noalloc_max_bytes(void);
int nimllm_attn_decode_noalloc(const void *q, int q_dtype, const void *k_cache, const void *v_cache,
                               int cache_dtype, const int64_t *kv_off, int64_t seq_stride,
                               int64_t head_stride, const int32_t *seq_len, int max_len, void *out,
                               int out_dtype, float *partials_out, int batch, int n_head,
                               int n_kv_head, int head_dim, float scale, int chunk_rows, void *stream);

/* ---- the steps either side of decode attention (one new token per sequence) -----------------
 * Weight matrices are row-major [out, in] as the reference stores them (gpuSgemm op 2 multiplies
 * by the transpose, src/gpu.nim:185-207).  w_type: */
#define NIMLLM_W_F32 0  /* float rows */
#define NIMLLM_W_BF16 1 /* bf16 rows */
#define NIMLLM_W_Q8_0 2 /* blocks {half d; int8 qs[32]}, 34 bytes per 32 weights (src/kernels.cu:1013-1016) */
#define NIMLLM_W_Q4_0 3 /* blocks {half d; uint8 qs[16]}, 18 bytes per 32 weights (src/kernels.cu:898-901) */

/* Replaces, in one launch, the q / k / v projections, ropeFwd on q and kNew and the per-KV-head
 * append of forwardCached (src/model.nim:775-815: three quantMatvec or gpuSgemm calls, two
 * gpu_rope_fwd launches, 2*nKvHead cudaMemcpy): q, k and v are computed from x_norm and the three
 * weight matrices, q and k are rotated at each sequence's position, and rotated K / raw V go
 * straight into the cache row -- they are never written to and re-read from activation buffers.
 *   x_norm [batch, n_embd] fp32 (the output of the layer's RMSNorm)
 *   wq [n_head*head_dim, n_embd], wk, wv [n_kv_head*head_dim, n_embd] of w_type, 16-byte aligned
 *   q_out  [batch, n_head*head_dim] fp32, rotated: what nimllm_attn_decode takes as q
 *   k_out, v_out  optional [batch, n_kv_head*head_dim] fp32 copies (rotated K, raw V); NULL: cache only
 *   rope tables, seq_pos / pos0, caches, kv_off, strides, cache_row0, max_seq: as nimllm_rope_append
 * A weight byte is fetched once per 8 sequences (larger batches re-read the weights per group of 8:
 * a decode batch that large wants a GEMM, which this entry point is not). */
int nimllm_qkv_rope_append(const float *x_norm, const void *wq, const void *wk, const void *wv, int w_type, float *q_out,
                           float *k_out, float *v_out, const float *rope_cos, const float *rope_sin,
                           const int32_t *seq_pos, int pos0, void *k_cache, void *v_cache, int cache_dtype,
                           const int64_t *kv_off, int64_t seq_stride, int64_t head_stride, int cache_row0, int max_seq,
                           int batch, int n_embd, int n_head, int n_kv_head, int head_dim, void *stream);

/* Replaces the output projection and the residual add after attention (src/model.nim:843-849:
 * quantMatvec or gpuSgemm, then gpu_add): x_out[b] = x_resid[b] + wo attn_out[b].
 *   attn_out [batch, n_in] fp32, wo [n_embd, n_in] of w_type, x_resid / x_out [batch, n_embd] fp32 */
int nimllm_wo_residual(const float *attn_out, const void *wo, int w_type, const float *x_resid, float *x_out, int batch,
                       int n_embd, int n_in, void *stream);

/* y[b] = w x[b] (+ residual[b]) for any of the weight types: the general form of the two entry
 * points above and of the reference's quantMatvec (src/model.nim:445-450).  x [batch, cols],
 * y and residual (optional) [batch, rows], fp32. */
int nimllm_matvec(const void *w, int w_type, const float *x, const float *residual, float *y, int batch, int rows,
                  int cols, void *stream);
/* The staged form of the projection kernels (eight input vectors per tile) waits for its weight copies
 * with a bound (about 2 s without progress); a launch in which a wait gave up leaves incomplete results
 * and raises a per-device status word that stays raised until it is cleared.  Returns 0, 1 (raised) or
 * a negative NIMLLM_ERR_* code; reset != 0 clears the word.  Synchronises the device: call it where the
 * host waits for results anyway.  No counterpart in the reference. */
int nimllm_matvec_status(int reset);

/* ---- merge of (max, sum, output) partials ----------------------------------------
 * No counterpart in the reference (it never splits a softmax row, src/kernels.cu:
 * 267-303 sees the whole row).  parts [n_parts, rows, rec_stride] fp32 records
 * {o[D], m, l, ...}; out [rows, D].  Used after gathering the shards of a
 * KV-sequence-sharded decode. partials_out (optional) receives the merged records. */
int nimllm_attn_combine(const float *parts, int n_parts, int rows, int head_dim, int rec_stride,
                        void *out, int out_dtype, float *partials_out, void *stream);

/* ---- exchange and merge of KV-sequence shards over peer memory ------------------------
 * No counterpart in the reference (single GPU).  One process per GPU of a box; every rank's
 * decode has produced records [rows, D+4] (partials_out above) for ITS rows of the KV sequence.
 * nimllm_attn_combine_peers stores them into every peer's exchange buffer over NVLink (plain
 * peer stores, then a per-rank flag), waits -- up to the wait limit, then *status_dev = 1 --
 * for all peers' records, and merges them: the all-gather and the merge of
 * nimllm_attn_combine in two small launches with no collective library on the path.
 * Set-up: create a buffer per rank, pass every rank's 64-byte export handle to every other rank
 * (any host transport), import them, then ready().  All ranks must call combine_peers the same
 * number of times, in the same order. */
typedef struct nimllm_peer_exchange nimllm_peer_exchange;
nimllm_peer_exchange *nimllm_peer_exchange_create(int rank, int world, int rows_max, int head_dim);
int nimllm_peer_exchange_export(nimllm_peer_exchange *x, void *handle_out_64_bytes);
int nimllm_peer_exchange_import(nimllm_peer_exchange *x, int peer_rank, const void *handle_64_bytes);
/* a peer that lives in the same process on the same device (several ranks driven by one process,
 * tests on one GPU): its buffer is used directly, without a handle */
int nimllm_peer_exchange_import_local(nimllm_peer_exchange *x, int peer_rank, nimllm_peer_exchange *peer);
int nimllm_peer_exchange_ready(nimllm_peer_exchange *x);
/* how long the wait for the peers' records may last before it gives up and sets *status_dev = 1
 * (default 1000 ms); a rank that stopped calling leaves the others with that status, not a hang */
int nimllm_peer_exchange_set_wait_limit(nimllm_peer_exchange *x, int milliseconds);
void nimllm_peer_exchange_destroy(nimllm_peer_exchange *x);
int nimllm_attn_combine_peers(nimllm_peer_exchange *x, const float *rec_local, int rows, void *out, int out_dtype,
                              int *status_dev, void *stream);

/* The same exchange fused into the shard's decode (bf16 cache, Hq/Hkv <= 8, head_dim 64 or 128):
 * nimllm_attn_decode_push runs this rank's decode over its rows of the KV sequence (arguments as
 * nimllm_attn_decode with chunk_rows = 0) and its merge launch stores every finished record straight
 * into every peer's buffer -- no separate copy of the records, no extra launch; nimllm_attn_wait_combine
 * then waits (bounded) for all ranks' records of this call and merges them into out [batch*n_head, D].
 * Every rank calls the pair once per step, in the same order; both launches may be captured in a graph. */
size_t nimllm_attn_decode_push_workspace_bytes(int batch, int n_head, int n_kv_head, int head_dim, int max_len);
int nimllm_attn_decode_push(nimllm_peer_exchange *x, const void *q, int q_dtype, const void *k_cache,
                            const void *v_cache, const int64_t *kv_off, int64_t seq_stride, int64_t head_stride,
                            const int32_t *seq_len, int max_len, int batch, int n_head, int n_kv_head, int head_dim,
                            float scale, void *workspace, size_t workspace_bytes, void *stream);
int nimllm_attn_wait_combine(nimllm_peer_exchange *x, int rows, void *out, int out_dtype, int *status_dev, void *stream);

/* ---- causal prefill ----------------------------------------------------------------
 * Replaces the attention block of forward(), src/model.nim:469-475,494-508: RoPE on
 * q and k, then per query head gather / cublasSgemm_v2 QK^T / gpu_causal_mask /
 * gpu_softmax_fwd / cublasSgemm_v2 PV / scatter (2 + 8*Hq launches, two S x S fp32
 * matrices per head) -- as one flash-style kernel (plus one RoPE/append pre-pass).
 *
 *   q [B,S,Hq*D], k, v [B,S,Hkv*D], out [B,S,Hq*D], all `dtype`
 *   rope tables as above (NULL: inputs are already rotated); token i of every
 *   sequence sits at position pos0 + i
 *   save_cache  the reference's forward(saveCache) flag (src/model.nim:454-457,534):
 *            non-zero guarantees q and k hold their post-RoPE values on return, as
 *            backward() expects (src/model.nim:656-685).  k is rotated in place in
 *            either case; with 0 the contents of q afterwards are unspecified.
 *   k_cache / v_cache (optional) receive rows pos0..pos0+S-1, as in rope_append
 *   lse      optional fp32 [B, Hq, S]: log-sum-exp of the scaled scores per row
 *   dtype F32 runs on the CUDA cores in fp32 (the <= 1e-4 parity path); BF16 runs
 *   QK^T and PV on the tcgen05 tensor cores with fp32 accumulation.
 *   workspace: nimllm_attn_prefill_workspace_bytes(...) bytes (currently 0: NULL is accepted)
 *
 * The bf16 kernel's internal waits are bounded (about 2 s without progress); a launch in which
 * one gave up leaves incomplete results in out / lse and raises a per-device status word that
 * stays raised until it is cleared:
 *   nimllm_attn_prefill_status(reset)  returns 0 (every bf16 prefill since the last reset ran to
 *            completion), 1 (one did not), or a negative NIMLLM_ERR_* code; reset != 0 clears the
 *            word.  It synchronises the device, so call it where the host waits for results anyway
 *            (after a forward pass, before sampling), not per layer.
 */
size_t nimllm_attn_prefill_workspace_bytes(int batch, int seq_len, int n_head, int n_kv_head,
                                           int head_dim, int dtype);
int nimllm_attn_prefill_status(int reset);
int nimllm_attn_prefill(void *q, void *k, const void *v, int dtype, const float *rope_cos,
                        const float *rope_sin, int pos0, void *out, int batch, int seq_len,
                        int n_head, int n_kv_head, int head_dim, float scale, int save_cache,
                        void *k_cache, void *v_cache, int cache_dtype, const int64_t *kv_off,
                        int64_t seq_stride, int64_t head_stride, int max_seq, float *lse,
                        void *workspace, size_t workspace_bytes, void *stream);

/* ---- backward of the causal prefill (training with saveCache) -------------------------
 * Replaces the attention block of backward(), src/model.nim:639-685 (per query head: recompute
 * scores and probabilities, dWeights, softmax_bwd src/kernels.cu:305-328, dq / dk / dv products,
 * accumulation of dk and dv over the query heads of a KV head with atomics
 * src/kernels.cu:451-461) followed by ropeBwd on dq and dk (src/kernels.cu:425-431).  fp32.
 *   q_rot, k_rot  the post-RoPE activations the forward left behind (save_cache = 1)
 *   v, out        V as given to the forward, and the forward's output
 *   dout          gradient of out, [B, S, Hq*D]
 *   lse           [B, Hq, S] as written by nimllm_attn_prefill (required)
 *   rope_cos/sin  the forward's tables: dq and dk come back in the pre-RoPE space, as ropeBwd
 *                 leaves them (NULL: no rotation is undone)
 *   dq [B, S, Hq*D], dk, dv [B, S, Hkv*D] are overwritten (the reference accumulates into
 *                 zero-initialised buffers); sums run in a fixed order, results repeat bit for bit
 *   workspace     nimllm_attn_prefill_bwd_workspace_bytes(batch, seq_len, n_head, head_dim) bytes
 */
size_t nimllm_attn_prefill_bwd_workspace_bytes(int batch, int seq_len, int n_head, int head_dim);
int nimllm_attn_prefill_bwd(const float *q_rot, const float *k_rot, const float *v, const float *out,
                            const float *dout, const float *lse, const float *rope_cos,
                            const float *rope_sin, int pos0, float *dq, float *dk, float *dv,
                            int batch, int seq_len, int n_head, int n_kv_head, int head_dim,
                            float scale, void *workspace, size_t workspace_bytes, void *stream);

/* ---- the reference's own attention-path launchers, same names and arguments -------
 * Kept so that callers that still use the unfused sequence (backward(), the test
 * programs) link against this library alone.  All launch on the legacy default
 * stream and return void like the originals. */
/* src/kernels.cu:417-423 */
void gpu_rope_fwd(float *data, const float *cos_tab, const float *sin_tab, int seq_len,
                  int n_embd, int n_head, int head_dim);
/* src/kernels.cu:376-381 */
void gpu_extract_head(const float *src, float *dst, int h, int seq_len, int n_embd, int head_dim);
/* src/kernels.cu:383-388 */
void gpu_insert_head(const float *src, float *dst, int h, int seq_len, int n_embd, int head_dim);
/* src/kernels.cu:463-469 */
void gpu_extract_kv_head(const float *src, float *dst, int qHead, int kvRepeat, int seq_len,
                         int n_kv_dim, int head_dim);
/* src/kernels.cu:260-263 */
void gpu_causal_mask(float *scores, float scale, int seq_len);
/* src/kernels.cu:159-161 */
void gpu_scale(const float *x, float s, float *y, int n);
/* src/kernels.cu:336-339 */
void gpu_softmax_fwd(const float *x, float *y, int rows, int cols);
/* src/kernels.cu:750-755 (bound in src/gpu.nim:309-311, no caller): single-head fused
 * attention on dense [S, hd] fp32 buffers */
void gpu_flash_attn_fwd(const float *Q, const float *K, const float *V, float *O, int S, int hd,
                        float scale, int causal);
/* src/kernels.cu:996-1003 and :1053-1059: y[rows] = A[rows, cols] x[cols] with A in Q4_0 / Q8_0 blocks */
void gpu_matvec_q4_0(const void *A, const float *x, float *y, int rows, int cols);
void gpu_matvec_q8_0(const void *A, const float *x, float *y, int rows, int cols);

#ifdef __cplusplus
}
#endif
#endif /* NIMLLM_ATTN_H */
