/*
 * bonsai_kv.h - C ABI of the B200 KV-cache path (libbonsai_kv.so).
 *
 * Scope: the KV-cache hot path of the qwen35 full-attention layers of
 * herlangga72/ternary-bonsai-inference: per-token append (IMROPE on K, then
 * store K/V as f32, f16 or the rotated Lloyd-Max "planar" format) and GQA
 * decode attention over that cache.  Everything below runs on the GPU (CUDA,
 * sm_100a); there is no CPU fallback.  Each entry point names the reference
 * interface it replaces (paths inside the reference project).
 *
 * Conventions
 *  - Every function returns a bk_status; bk_last_error() gives the text of the
 *    last failure on a context (the reference returns Result<_, String>).
 *  - A bk_ctx owns one CUDA stream and is NOT thread-safe: one in-order stream
 *    per context, as the reference decodes on one thread.  Use one context per
 *    host thread / per GPU.
 *  - Pointers named *_dev are device pointers valid on the context's device and
 *    the call is asynchronous on the context's stream.  Pointers named *_host
 *    are host pointers and the call returns after the result is in host memory.
 *  - The caller owns q/k/v/out buffers; the library owns caches and tables.
 *  - Kernels of one context overlap at their edges: a kernel begins its set-up
 *    while the one before it on the stream is finishing, and reads what earlier
 *    calls produced (q, k, v, the cache) only after that kernel has completed.
 *    Weights are read during the set-up: the norm weights given to
 *    bk_attn_layer_step and the payloads given to bk_pq2_matvec* must be
 *    complete in device memory before the PRECEDING call on the context is
 *    issued, and must not be rewritten while calls are in flight (upload them
 *    once with bk_memcpy_h2d + bk_synchronize).
 *  - Every wait inside a kernel is bounded.  A wait that runs out (a peer of the
 *    context split never sent its rows) sets an error word; every call that
 *    blocks the host (bk_synchronize, the *_host forms, downloads, snapshots,
 *    bk_event_elapsed_ms) then returns BK_ERR_CUDA with the reason, the step
 *    in flight is void, and the context stays usable.
 *  - Layouts follow the reference: token-major [pos][kv_head][...].
 */
#ifndef BONSAI_KV_H
#define BONSAI_KV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define BK_API __attribute__((visibility("default")))
#else
#define BK_API
#endif

typedef struct bk_ctx bk_ctx;
typedef struct bk_cache bk_cache;
typedef struct bk_event bk_event;

typedef enum bk_status {
    BK_OK = 0,
    BK_ERR_INVALID = 1,     /* bad argument (null pointer, size mismatch, bits outside 1..8) */
    BK_ERR_CUDA = 2,        /* a CUDA runtime call failed or a kernel gave up a bounded wait; text in bk_last_error */
    BK_ERR_OOM = 3,         /* device or host allocation failed */
    BK_ERR_RANGE = 4,       /* position beyond the allocated context (src/gdev.rs:907-912) */
    BK_ERR_UNSUPPORTED = 5  /* geometry this build has no kernel for (src/gdev.rs:274-282) */
} bk_status;

/* KvMode, src/kvquant.rs:486-493. */
enum { BK_MODE_F32 = 0, BK_MODE_F16 = 1, BK_MODE_PLANAR = 2 };
typedef struct bk_kv_mode {
    int32_t kind;    /* BK_MODE_* */
    int32_t bits;    /* 1..8 for BK_MODE_PLANAR, else 0 */
    int32_t v_quant; /* planar only: 1 = V quantized too, 0 = K only (V stays f32) */
} bk_kv_mode;

/* Geometry of a cache.  bk_default_config fills the qwen35 constants of
 * src/gdev.rs:21-37: 24 q heads, 4 kv heads, head_dim 256, 64 rotated dims,
 * sections [11,11,10,0], rope base 1e7. */
typedef struct bk_cache_config {
    int32_t n_layers;       /* full-attention layers held (16 of qwen35's 64) */
    int32_t n_seqs;         /* independent sequences (the reference has 1) */
    int32_t n_ctx;          /* rows allocated up front per (layer, sequence): BONSAI_CTX */
    int32_t n_head;
    int32_t n_kv;
    int32_t hd;
    int32_t n_rot;
    int32_t sections[4];
    float freq_base;
    int32_t rope_positions; /* positions the rope table covers; 0 = n_ctx.  Larger when a cache
                               holds a chunk of a longer sequence (context split over GPUs). */
    bk_kv_mode mode;
} bk_cache_config;

/* ---- library / context -------------------------------------------------- */

BK_API const char *bk_version(void);
BK_API const char *bk_status_string(bk_status s);

/* Replaces vk::Gpu creation as far as this path needs it (src/gdev.rs:269):
 * binds `device`, creates the stream and uploads the Givens table and the
 * Lloyd-Max codebooks (src/gdev.rs:360-368 uploads the same two tables). */
BK_API bk_status bk_ctx_create(int device, bk_ctx **out);
BK_API void bk_ctx_destroy(bk_ctx *ctx);
/* Text of the last error on `ctx` (or of the last context-less failure when ctx is NULL). */
BK_API const char *bk_last_error(const bk_ctx *ctx);
/* Blocks until the context's stream is idle (the reference blocks in
 * rec_end_submit, src/vk.rs:2340-2364). */
BK_API bk_status bk_synchronize(bk_ctx *ctx);
/* The context's cudaStream_t, for callers that enqueue their own work around the path. */
BK_API void *bk_ctx_stream(bk_ctx *ctx);
BK_API int bk_ctx_device(const bk_ctx *ctx);

/* ---- mode selection: src/kvquant.rs:515-550, src/gdev.rs:39-48 ------------ */

/* parse_mode: "" / f32, f16 / fp16 / half, planarN / isoN, trailing k = K only;
 * anything else (N outside 1..8 included) is f32.  Never fails on content. */
BK_API bk_status bk_parse_mode(const char *s, bk_kv_mode *out);
/* mode_from_env: BONSAI_KV, f32 when unset. */
BK_API bk_status bk_mode_from_env(bk_kv_mode *out);
/* n_ctx_env: BONSAI_CTX in 16..=262144, else 2048. */
BK_API int32_t bk_n_ctx_from_env(void);
BK_API void bk_default_config(bk_cache_config *cfg);

/* ---- cache: AttnCache (src/forward.rs:30-86), GDev buffers (src/gdev.rs:329-469) */

/* Allocates every row for n_ctx positions up front, as GDev::open does.
 * Quantized rows are stored as the CPU cache stores them: packed bytes
 * [pos][kv][32*bits] and norms [pos][kv] apart (src/forward.rs:40-46), not
 * interleaved with the norm word as in shaders/kv_store_q.comp:119. */
BK_API bk_status bk_cache_create(bk_ctx *ctx, const bk_cache_config *cfg, bk_cache **out);
BK_API void bk_cache_destroy(bk_cache *cache);
/* Decoder::reset (src/forward.rs:640-656): forget the tokens of one sequence (seq >= 0) or all (-1). */
BK_API bk_status bk_cache_reset(bk_cache *cache, int32_t seq);
/* AttnCache::n_pos (src/forward.rs:78-86); negative on bad arguments. */
BK_API int32_t bk_cache_n_pos(const bk_cache *cache, int32_t layer, int32_t seq);
/* Declare rows [0, n_pos) of (layer, seq) as filled without writing them (restoring a snapshot
 * through bk_cache_upload, or benchmarks that fill rows by bulk appends in another order). */
BK_API bk_status bk_cache_set_n_pos(bk_cache *cache, int32_t layer, int32_t seq, int32_t n_pos);
BK_API bk_status bk_cache_get_config(const bk_cache *cache, bk_cache_config *out);
/* Bytes of one K row / one V row per (pos, kv head) incl. the norm: 1024 f32, 512 f16, 32*bits+4. */
BK_API int32_t bk_cache_row_bytes(const bk_cache *cache, int32_t is_v);
/* Device bytes held by the cache (rows + norms), cf. the sizing report of src/gdev.rs:380-387. */
BK_API size_t bk_cache_device_bytes(const bk_cache *cache);

/* dump_kv (src/gdev.rs:1433-1445), extended to every mode: copies rows
 * [pos0, pos0+n_pos) of (layer, seq) to host.  k_rows/v_rows receive
 * n_pos*n_kv rows of f32[hd], u16[hd] or u8[32*bits]; k_norms/v_norms receive
 * n_pos*n_kv floats and are ignored for sides that hold no norms.  Any pointer
 * may be NULL to skip that part. */
BK_API bk_status bk_cache_download(bk_cache *cache, int32_t layer, int32_t seq, int32_t pos0,
                                   int32_t n_pos, void *k_rows_host, float *k_norms_host,
                                   void *v_rows_host, float *v_norms_host);
/* Inverse of bk_cache_download (snapshot restore); does not change n_pos. */
BK_API bk_status bk_cache_upload(bk_cache *cache, int32_t layer, int32_t seq, int32_t pos0,
                                 int32_t n_pos, const void *k_rows_host, const float *k_norms_host,
                                 const void *v_rows_host, const float *v_norms_host);

/* Prompt-cache snapshot of one sequence (all layers) as one self-describing
 * buffer; restores into any cache of the same KV mode, layer count and head
 * geometry (n_ctx and n_seqs may differ) and sets n_pos.  No reference
 * counterpart as a function - the reference's server has no prompt cache
 * (README.md:218-221) - but the payload is the reference's own row layout,
 * either one: layout 0 = the CPU stores of src/forward.rs:40-46 (rows, then
 * norms), layout 1 = the device rows of shaders/kv_store_q.comp:119-123
 * (packed words + norm word per row).  Header: u32 magic "BKVS", version,
 * layout, mode kind, bits, v_quant, n_layers, n_kv, hd, 3 reserved, then
 * n_pos per layer.  bk_cache_snapshot_bytes returns 0 on bad arguments. */
BK_API size_t bk_cache_snapshot_bytes(const bk_cache *cache, int32_t seq);
BK_API bk_status bk_cache_snapshot_save(bk_cache *cache, int32_t seq, int32_t layout, void *buf_host,
                                        size_t buf_bytes, size_t *written);
BK_API bk_status bk_cache_snapshot_load(bk_cache *cache, int32_t seq, const void *buf_host,
                                        size_t buf_bytes);

/* ---- append: src/forward.rs:259-285, shaders rope_imrope + kv_store* ------- */

/* One fused kernel: IMROPE on K (all four position ids = rope_pos + i, as
 * src/forward.rs:259-270 passes them), then store K and V rows by mode at row
 * index n_pos(layer, seq) + i.  k_dev/v_dev: [n_tokens][n_kv][hd] f32, K
 * already RMS-normed, not yet roped.  The reference appends with rope_pos ==
 * n_pos; a cache that holds a chunk of a longer sequence passes the global
 * position.  Stored bytes equal the reference CPU path's bit for bit. */
BK_API bk_status bk_append(bk_cache *cache, int32_t layer, int32_t seq, int32_t rope_pos,
                           int32_t n_tokens, const float *k_dev, const float *v_dev);
/* Same, host pointers (copies in through pinned staging, then runs bk_append). */
BK_API bk_status bk_append_host(bk_cache *cache, int32_t layer, int32_t seq, int32_t rope_pos,
                                int32_t n_tokens, const float *k_host, const float *v_host);
/* One token for each of n_seqs sequences in one launch (a batched decode step).
 * seq_ids/rope_pos are host arrays; seq_ids NULL = 0..n_seqs-1, rope_pos NULL = each
 * sequence's n_pos.  k_dev/v_dev: [n_seqs][n_kv][hd]. */
BK_API bk_status bk_append_batch(bk_cache *cache, int32_t layer, int32_t n_seqs,
                                 const int32_t *seq_ids, const int32_t *rope_pos,
                                 const float *k_dev, const float *v_dev);

/* ---- decode attention: src/forward.rs:247-258, 287-375; shaders attn_scores*,
 *      softmax_inplace, attn_out* ------------------------------------------------ */

/* GQA decode attention for n_seqs sequences of one layer: IMROPE on q at
 * q_pos, softmax(q.K^T/sqrt(hd)).V over rows [0, n_pos) of each sequence, kv
 * head = q head / (n_head/n_kv).  Split-K flash decoding: each K/V row is read
 * once for all q heads of its group.  q_dev/out_dev: [n_seqs][n_head][hd] f32;
 * q is RMS-normed, not yet roped; out is the pre-gate attention output
 * (src/forward.rs:374).  Host arrays: seq_ids NULL = 0..n_seqs-1; n_pos NULL =
 * all cached rows; q_pos NULL = n_pos-1 (the reference's pos).  A sequence
 * with n_pos == 0 yields zeros. */
BK_API bk_status bk_decode_attn(bk_cache *cache, int32_t layer, int32_t n_seqs,
                                const int32_t *seq_ids, const int32_t *n_pos,
                                const int32_t *q_pos, const float *q_dev, float *out_dev);
/* Same scan, but leaves the softmax unnormalised so that chunks of one long
 * sequence held by different caches/GPUs can be merged: part_dev is
 * [n_seqs][n_head][hd+2] = (acc[hd], m, l) with out = acc / l and m the
 * running maximum of the scaled scores (natural-log domain). */
BK_API bk_status bk_decode_attn_partial(bk_cache *cache, int32_t layer, int32_t n_seqs,
                                        const int32_t *seq_ids, const int32_t *n_pos,
                                        const int32_t *q_pos, const float *q_dev,
                                        float *part_dev);
/* No counterpart in the reference.  bk_decode_attn for callers that must not allocate once they
 * are running (a serving loop that gave all of HBM to the caches at start-up and forbids later
 * cudaMalloc because it synchronises the device and can fail on a fragmented heap; a thread or
 * callback in which the CUDA allocator must not be entered).  The split-K scratch is a fixed
 * array inside the library (about 4.3 MB per GPU, held until the process exits) instead of
 * allocated memory, and a call that succeeds touches no allocator of any kind (a call that
 * fails builds its error text on the host heap).  Limits: at most 64 sequences per call, else
 * BK_ERR_INVALID; the scratch holds 512 (sequence, kv head, chunk) work items, and a request
 * that would need more is cut into coarser chunks instead of being rejected, so the result
 * equals bk_decode_attn's within the parity tolerance (1e-3), not bit for bit.  Every call on
 * a device shares the array: calls that overlap on the GPU race, so serialise them.  The first
 * call on a device resolves the array's address (thread-safe, once per device); make it during
 * set-up, outside any stream capture. */
BK_API bk_status bk_decode_attn_noalloc(bk_cache *cache, int32_t layer, int32_t n_seqs,
                                        const int32_t *seq_ids, const int32_t *n_pos,
                                        const int32_t *q_pos, const float *q_dev, float *out_dev);
/* Log-sum-exp merge of n_parts partial results: parts_dev is
 * [n_parts][n_rows][hd+2], out_dev [n_rows][hd].  No reference counterpart
 * (the reference is single-device); it is the merge step of the context split. */
BK_API bk_status bk_lse_merge(bk_ctx *ctx, int32_t n_parts, int32_t n_rows, int32_t hd,
                              const float *parts_dev, float *out_dev);

/* Context split with the exchange fused into the merge, over peer memory (NVLink): no reference
 * counterpart.  Every rank creates a mailbox and hands its 64-byte IPC handle to the other
 * ranks' processes (any transport); bk_mailbox_open_peers takes all `world` handles in rank order.
 * bk_decode_attn_split then scans this rank's chunk (rows [0, n_pos) of its cache; q replicated on
 * every rank, q_pos = the global position), stores its (acc, m, l) rows into every rank's mailbox
 * with peer stores, waits - bounded; a time-out is reported by bk_synchronize - for the rows of all
 * ranks carrying `seqno`, and writes the merged [n_head][hd] output on every rank.  Every rank
 * must make the same sequence of calls with seqno = 1, 2, 3, ...  A rank whose chunk is empty
 * calls with n_pos = 0. */
typedef struct bk_mailbox bk_mailbox;
#define BK_IPC_HANDLE_BYTES 64
BK_API bk_status bk_mailbox_create(bk_ctx *ctx, int32_t world, int32_t rank, int32_t n_rows, int32_t hd,
                                   bk_mailbox **out, void *ipc_handle_out);
BK_API bk_status bk_mailbox_open_peers(bk_mailbox *mailbox, const void *handles);
BK_API void bk_mailbox_destroy(bk_mailbox *mailbox);
BK_API bk_status bk_decode_attn_split(bk_cache *cache, int32_t layer, int32_t seq, int32_t n_pos,
                                      int32_t q_pos, const float *q_dev, float *out_dev,
                                      bk_mailbox *mailbox, uint32_t seqno);
/* The whole step of a split sequence in one launch per rank: the rank that owns
 * the tail passes the new token's k/v [n_kv][hd] (they become its next row, roped
 * at q_pos), every other rank passes NULL; then as bk_decode_attn_split over
 * the rank's rows.  No reference counterpart (single-device reference). */
BK_API bk_status bk_attn_step_split(bk_cache *cache, int32_t layer, int32_t seq, int32_t q_pos,
                                    const float *q_dev, const float *k_dev, const float *v_dev,
                                    float *out_dev, bk_mailbox *mailbox, uint32_t seqno);
/* The exchange and merge on their own, for partial rows produced by other calls: part_dev is
 * [n_rows][hd + 2] = (acc, m, l) rows as bk_decode_attn_partial writes them, n_rows the row
 * count the mailbox was created with, taken in groups of n_rep consecutive rows (one CTA
 * each); every rank sends its rows to all ranks and writes the log-sum-exp merge of all
 * ranks' rows to out_dev [n_rows][hd].  With a mailbox of n_layers * n_head rows a caller
 * whose layers do not depend on one another (a benchmark; speculative or batched callers)
 * scans all layers first and pays ONE exchange per token instead of one per layer. */
BK_API bk_status bk_exchange_merge(bk_mailbox *mailbox, int32_t n_rep, const float *part_dev,
                                   float *out_dev, uint32_t seqno);

/* The attention step with the reference's own shape (src/forward.rs:247-375,
 * src/gdev.rs:584-829): rope q and k at `pos`, store k/v at row `pos` (which
 * must equal n_pos), attend over pos+1 rows.  q [n_head][hd], k/v [n_kv][hd],
 * out [n_head][hd]. */
BK_API bk_status bk_attn_step(bk_cache *cache, int32_t layer, int32_t seq, int32_t pos,
                              const float *q_dev, const float *k_dev, const float *v_dev,
                              float *out_dev);
BK_API bk_status bk_attn_step_host(bk_cache *cache, int32_t layer, int32_t seq, int32_t pos,
                                   const float *q_host, const float *k_host, const float *v_host,
                                   float *out_host);
/* The attention step for a batch of independent sequences (no counterpart in
 * the single-sequence reference; the per-sequence semantics are bk_attn_step's):
 * sequence seq_ids[i] (NULL: i) gets one new token at its next position;
 * q [n_seqs][n_head][hd], k/v [n_seqs][n_kv][hd], out [n_seqs][n_head][hd].
 * One launch when every sequence is long enough for a tensor-core kernel. */
BK_API bk_status bk_attn_step_batch(bk_cache *cache, int32_t layer, int32_t n_seqs,
                                    const int32_t *seq_ids, const float *q_dev, const float *k_dev,
                                    const float *v_dev, float *out_dev);
/* Batched (prefill) form: causal attention of n_tokens consecutive prompt
 * tokens of one sequence whose K/V rows are already in the cache; token i
 * (rope position pos0 + i) attends rows 0 .. pos0 + i.  q and out are
 * [n_tokens][n_head][hd].  Same result as n_tokens successive attention
 * steps, which is how the reference handles prompts on quantized caches
 * (src/gdev.rs:1366-1372 refuses the batched pass there; src/forward.rs:247-375
 * per token).  bk_prefill_step appends the block first (pos0 must be n_pos). */
BK_API bk_status bk_prefill_attn(bk_cache *cache, int32_t layer, int32_t seq, int32_t pos0,
                                 int32_t n_tokens, const float *q_dev, float *out_dev);
BK_API bk_status bk_prefill_step(bk_cache *cache, int32_t layer, int32_t seq, int32_t pos0,
                                 int32_t n_tokens, const float *q_dev, const float *k_dev,
                                 const float *v_dev, float *out_dev);
/* The layer form of the step: everything full_attention_layer does between the
 * q/k/v projections and the output projection (src/forward.rs:237-382;
 * src/gdev.rs:584-829 with norm_rows / split_qgate / elem mode 4 around it).
 *   qfull  [n_head][2*hd]  projection output, per head [q | gate] (:237-241)
 *   kraw, vraw [n_kv][hd]  projection outputs
 *   q_norm_w, k_norm_w [hd] per-head RMSNorm weights (kernels.rs:97-122), eps
 *   out    [n_head][hd]    attention * sigmoid(gate), the input of attn_output
 * On caches that take the tensor-core decode path this is one launch.  The
 * stored K/V rows equal the reference's bit for bit (the k norm keeps the
 * reference's summation order). */
BK_API bk_status bk_attn_layer_step(bk_cache *cache, int32_t layer, int32_t seq, int32_t pos,
                                    const float *qfull_dev, const float *kraw_dev,
                                    const float *vraw_dev, const float *q_norm_w_dev,
                                    const float *k_norm_w_dev, float eps, float *out_dev);
BK_API bk_status bk_attn_layer_step_host(bk_cache *cache, int32_t layer, int32_t seq, int32_t pos,
                                         const float *qfull_host, const float *kraw_host,
                                         const float *vraw_host, const float *q_norm_w_host,
                                         const float *k_norm_w_host, float eps, float *out_host);
/* rms_norm_rows (src/kernels.rs:97-122): n_rows rows of row_len (<= 1024)
 * sharing one weight; bit-exact (sequential sum of squares). */
BK_API bk_status bk_rms_norm_rows(bk_ctx *ctx, int32_t n_rows, int32_t row_len, const float *x_host,
                                  const float *w_host, float eps, float *out_host);
/* PQ2_0 ternary rows (src/kernels.rs:204-211): ceil(ne0 / 128) blocks of 34
 * bytes (f16 scale + 128 two-bit codes, weight = (code - 1) * scale). */
BK_API size_t bk_pq2_row_bytes(int64_t ne0);
/* pq2_matvec_range / pq2_matmul_n (src/kernels.rs:265-330, 333-420; the device
 * form is Gpu::matvec_pq2, shaders/pq2_matvec_fused.comp):
 * y[t * n_rows + r] = sum_j x[t * ne0 + j] * W[base_row + r][j] for n_tok
 * activations.  payload_dev is the tensor's whole contiguous data in device
 * memory (rows back to back, bk_pq2_row_bytes apart; 16-byte alignment of the
 * first row of the range lets the TMA engine stream it, any even address
 * works); like the reference the call fails (BK_ERR_RANGE) when the rows asked
 * for do not lie inside payload_bytes.  Two tokens share one pass over the
 * weights.  The block sums run on the integer tensor cores with x in 25-bit
 * fixed point and are exact; the result differs from the reference's scalar
 * path by the rounding order across blocks, like the reference's own AVX2
 * path (src/kernels.rs:652-660). */
BK_API bk_status bk_pq2_matvec(bk_ctx *ctx, const void *payload_dev, size_t payload_bytes, int64_t ne0,
                               int64_t base_row, int64_t n_rows, const float *x_dev, int32_t n_tok,
                               float *y_dev);
/* Up to four row ranges of tensors with the same ne0 against the same x in ONE
 * launch (attn_q, attn_k and attn_v of a layer: src/forward.rs:219-236 makes
 * three matvec calls on one input); range s writes y_dev [n_tok][n_rows].  No
 * reference counterpart as a call; results equal the separate calls bit for bit. */
typedef struct bk_pq2_seg {
    const void *payload_dev;
    size_t payload_bytes;
    int64_t base_row, n_rows;
    float *y_dev;
} bk_pq2_seg;
BK_API bk_status bk_pq2_matvec_multi(bk_ctx *ctx, int32_t n_seg, const bk_pq2_seg *segs, int64_t ne0,
                                     const float *x_dev, int32_t n_tok);
/* The same with host x and y (weights stay resident in device memory). */
BK_API bk_status bk_pq2_matvec_host(bk_ctx *ctx, const void *payload_dev, size_t payload_bytes,
                                    int64_t ne0, int64_t base_row, int64_t n_rows, const float *x_host,
                                    int32_t n_tok, float *y_host);
/* Gpu::attn_step (src/vk.rs:1671-1752): one-shot f32 attention over host
 * k/v caches [n_pos][kvheads][hd], no rope; validates sizes like the
 * reference (hd must be 256 here). */
BK_API bk_status bk_attn_oneshot_host(bk_ctx *ctx, const float *q_host, const float *k_host,
                                      const float *v_host, int32_t n_pos, int32_t nheads,
                                      int32_t kvheads, int32_t hd, float *out_host);

/* ---- kvquant.rs entry points (host in/out, computed on the GPU) ----------- */

/* PlanarQuant::packed_len (src/kvquant.rs:348-350); 0 on bad arguments. */
BK_API size_t bk_kvq_packed_len(int32_t hd, int32_t bits);
/* codebook(d, bits) (src/kvquant.rs:103-114): 2^bits ascending centroids. */
BK_API bk_status bk_kvq_codebook(int32_t hd, int32_t bits, float *out_host);
/* givens_table(d) (src/kvquant.rs:131-145): ceil(hd/2) (cos, sin) pairs. */
BK_API bk_status bk_kvq_givens(int32_t hd, float *out_host);
/* No counterpart in the reference: the table behind the bulk append's nearest-centroid search for head
 * dimension 256 and widths 1..4, for checking that search against the reference's scan
 * (src/kvquant.rs:357-370) without a GPU.  512 cells of width 2^-10 over [-0.25, 0.25): out_host[2k] = how
 * many decision thresholds lie in cells below k, out_host[2k + 1] = the bits of the one threshold inside
 * cell k (+inf if none).  nearest(v) = out[2k] + (v >= threshold) with k = clamp(floor((v + 0.25) * 1024)),
 * all in f32.  Host only. */
BK_API bk_status bk_kvq_threshold_cells(int32_t bits, uint32_t *out_host);
/* PlanarQuant::quantize (src/kvquant.rs:397-412) for n_vec vectors of hd floats. */
BK_API bk_status bk_kvq_quantize(bk_ctx *ctx, int32_t hd, int32_t bits, int32_t n_vec,
                                 const float *x_host, uint8_t *packed_host, float *norms_host);
/* PlanarQuant::dequantize (src/kvquant.rs:415-428). */
BK_API bk_status bk_kvq_dequantize(bk_ctx *ctx, int32_t hd, int32_t bits, int32_t n_vec,
                                   const uint8_t *packed_host, const float *norms_host,
                                   float *out_host);
/* PlanarQuant::rotate / rotate_inv (src/kvquant.rs:373-394). */
BK_API bk_status bk_kvq_rotate(bk_ctx *ctx, int32_t hd, int32_t n_vec, int32_t inverse,
                               const float *x_host, float *out_host);
/* PlanarQuant::dot_rotated (src/kvquant.rs:455-477): out[i] = dot(q_rot[i], row i) * norm[i]. */
BK_API bk_status bk_kvq_dot_rotated(bk_ctx *ctx, int32_t hd, int32_t bits, int32_t n_vec,
                                    const float *q_rot_host, const uint8_t *packed_host,
                                    const float *norms_host, float *out_host);
/* rope_imrope (src/rope.rs:9-70) on n_heads head vectors of hd floats, in place. */
BK_API bk_status bk_rope_imrope(bk_ctx *ctx, int32_t n_heads, int32_t hd, float *heads_host,
                                int64_t p_t, int64_t p_h, int64_t p_w, int64_t p_e,
                                int32_t n_dims, const int32_t sections[4], float freq_base);
/* f32_to_half / half_to_f32 (src/gguf.rs:881-944), element-wise. */
BK_API bk_status bk_f32_to_half(bk_ctx *ctx, size_t n, const float *in_host, uint16_t *out_host);
BK_API bk_status bk_half_to_f32(bk_ctx *ctx, size_t n, const uint16_t *in_host, float *out_host);

/* ---- device memory and timing helpers for hosts without a CUDA binding ---- */

BK_API bk_status bk_dev_alloc(bk_ctx *ctx, size_t bytes, void **out_dev);
BK_API bk_status bk_dev_free(bk_ctx *ctx, void *dev);
BK_API bk_status bk_host_alloc_pinned(bk_ctx *ctx, size_t bytes, void **out_host);
BK_API bk_status bk_host_free_pinned(bk_ctx *ctx, void *host);
/* Asynchronous on the context's stream; src/dst host memory should be pinned. */
BK_API bk_status bk_memcpy_h2d(bk_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes);
BK_API bk_status bk_memcpy_d2h(bk_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes);
BK_API bk_status bk_memset_dev(bk_ctx *ctx, void *dst_dev, int value, size_t bytes);
/* CUDA events on the context's stream (GDEV_TIME=1 wall timers in src/gdev.rs:913, 939-948). */
BK_API bk_status bk_event_create(bk_ctx *ctx, bk_event **out);
BK_API void bk_event_destroy(bk_event *ev);
BK_API bk_status bk_event_record(bk_ctx *ctx, bk_event *ev);
BK_API bk_status bk_event_elapsed_ms(bk_ctx *ctx, bk_event *start, bk_event *stop, float *ms);
/* Kernels this library has launched on the context since creation. */
BK_API uint64_t bk_ctx_launch_count(const bk_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif /* BONSAI_KV_H */
