// Internal declarations shared by the translation units of libbonsai_kv.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <memory>
#include <string>
#include <vector>

#include "bonsai_kv.h"

namespace bk {

constexpr int kHd = 256;               // head_dim every kernel is specialised for
constexpr int kMaxBits = 8;
constexpr int kBookStride = 256;       // floats reserved per codebook in device memory
constexpr int kMaxSeqsPerLaunch = 64;  // sequences one decode launch can carry in its parameters
constexpr int kMaxItems = 4096;        // split-K work items one decode launch may create
constexpr int kMaxRep = 8;             // q heads per kv head the scratch is sized for
constexpr int kPartStride = kHd + 2;   // floats per partial result handed to callers: acc[hd], m, l
constexpr int kScratchStride = kHd + 4; // floats per partial in the split-K scratch (16-byte aligned rows)
constexpr int kMmaMinPos = 2048;       // 4-, 3- and 2-bit caches: launches with a shorter sequence carry the table's rounding remainders
constexpr int kRowMinPos = 128;        // sequences shorter than this take the generic f32 decode kernel (speed only)
constexpr int kMaxWorld = 8;            // ranks a context-split mailbox can connect
// The arrival counters of the split-K scratch, one per (sequence in the launch, kv head) pair i (i < 512),
// in three sets of kCtrSet: set 0 for the generic kernel, whose last arriver puts its counter back to zero;
// sets 1 and 2 for the tensor-core kernels, which alternate between them from launch to launch: a launch
// counts in one set and clears what the launch before the previous one left in the other, so that no CTA
// has to stay behind to reset anything.
constexpr int kCtrSet = 512, kCtrTotal = 3 * kCtrSet;
constexpr int kDescSlots = 8;          // launches of bk_append_batch that may be in flight
constexpr int kDescCap = 4096;         // tokens one bk_append_batch call may carry

// Host set-up math (bk_host_tables.cpp).  The reference computes the same three tables on
// the CPU and uploads them: src/gdev.rs:360-368 (Givens + codebook), src/rope.rs:23-57.
void host_codebook(int hd, int bits, float *out);
void host_givens(int hd, float *out);
// cos/sin of the IMROPE angle of pair j at position p: out[(p - pos0) * (n_rot/2) + j] = (cos, sin).
void host_rope_rows(int64_t pos0, int64_t n_pos, int n_rot, float freq_base, float2 *out);
// Which of the four position ids (t, h, w, e -> 0..3) pair j takes: src/rope.rs:37-49.
int host_rope_band(int j, const int32_t sections[4]);

struct RopeTable {
    int n_rot = 0;
    float freq_base = 0.f;
    int n_pos = 0;
    float2 *d = nullptr;  // [n_pos][n_rot/2]
    int device = 0;
    ~RopeTable();
};

enum RowKind : int { ROW_F32 = 0, ROW_F16 = 1, ROW_PLANAR = 2 };

}  // namespace bk

struct bk_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    std::string err;
    uint64_t launches = 0;
    float *d_givens = nullptr;     // 128 (cos, sin) pairs
    float *d_codebooks = nullptr;  // 8 books, book of width b at (b-1)*kBookStride
    uint2 *d_cell_tabs = nullptr;  // widths 1..4: 512 (index, threshold) cells each, table of width b at (b-1)*512 (bk_device.cuh)
    float h_givens[bk::kHd];
    float h_codebooks[bk::kMaxBits * bk::kBookStride];
    float lut_alpha[bk::kMaxBits + 1] = {};  // per width: scale applied to centroids before f16 rounding
    bool prefill_umma = true;              // batched attention on tcgen05; BONSAI_KV_PREFILL=mma picks the mma.sync kernel
    bool force_generic = false;            // BONSAI_KV_GENERIC=1: never take the tensor-core path
    bool qsplit = true;                    // q as f16 hi + lo in the tensor-core path (BONSAI_KV_QSPLIT=0: hi only)
    int mma_min_rows = 0;                  // BONSAI_KV_MMA_MIN: rows from which the row kernel (f16, f32, K-only) is taken; 0 = built-in
    int dyn_tiles = 0; bool dist_combine = true;  // BONSAI_KV_DYN=0 / BONSAI_KV_DIST=0 switch them off
    // staging for the *_host entry points (grown on demand)
    void *h_stage = nullptr;
    size_t h_stage_bytes = 0;
    void *d_stage = nullptr;
    size_t d_stage_bytes = 0;
    float *d_layer = nullptr;              // normed q and k rows of the layer step (generic decode path)
    size_t d_layer_floats = 0;
    float *d_prefill = nullptr;            // (O, m, l) triples of the prefill attention's context chunks
    size_t d_prefill_floats = 0;
    // split-K scratch of the decode kernel: partial results and arrival counters
    float *d_partials = nullptr;
    unsigned *d_counters = nullptr;
    int ctr_set = 0;               // which of the two tensor-core counter sets the next launch counts in
    int ctr_dirty[2] = {0, 0};     // entries of each set that a launch has left non-zero
    // Set by a kernel whose bounded wait ran out (the code says which wait).  The word lives in pinned host
    // memory that the device writes directly, so every host-side wait for the stream can look at it for free.
    int *d_err = nullptr;          // device view
    volatile int *h_err = nullptr; // host view of the same word
    int xch_polls = 1 << 20;       // polls of one arrival word of the context-split exchange before giving up (BONSAI_KV_XCH_POLLS)
    int n_sms = 148;
    std::vector<std::shared_ptr<bk::RopeTable>> ropes;
    // token descriptors of bk_append_batch: a ring of pinned/device slots, one event per slot
    // so that a slot is rewritten only after the launch that read it has finished
    int4 *h_desc = nullptr, *d_desc = nullptr;
    cudaEvent_t desc_ev[bk::kDescSlots] = {};
    unsigned desc_next = 0;
};

struct bk_cache {
    bk_ctx *ctx = nullptr;
    bk_cache_config cfg{};
    int k_kind = 0, v_kind = 0;         // bk::RowKind
    size_t k_row_bytes = 0, v_row_bytes = 0;  // bytes of one (pos, kv head) row, norms excluded
    uint8_t *d_k = nullptr, *d_v = nullptr;   // [layer][seq][n_ctx][n_kv][row_bytes]
    float *d_kn = nullptr, *d_vn = nullptr;   // [layer][seq][n_ctx][n_kv], planar sides only
    std::vector<int32_t> n_pos;               // [layer][seq]
    std::shared_ptr<bk::RopeTable> rope;
    size_t device_bytes = 0;
    alignas(64) unsigned char tmap_k[128], tmap_v[128];  // CUtensorMap objects (4/3-bit planar and f16 K+V caches): boxes of 16 positions
    bool has_tmaps = false;

    size_t slab(int layer, int seq) const { return (size_t)layer * cfg.n_seqs + seq; }
    uint8_t *k_rows(int layer, int seq) const {
        return d_k + slab(layer, seq) * cfg.n_ctx * cfg.n_kv * k_row_bytes;
    }
    uint8_t *v_rows(int layer, int seq) const {
        return d_v + slab(layer, seq) * cfg.n_ctx * cfg.n_kv * v_row_bytes;
    }
    float *k_norms(int layer, int seq) const {
        return d_kn ? d_kn + slab(layer, seq) * cfg.n_ctx * cfg.n_kv : nullptr;
    }
    float *v_norms(int layer, int seq) const {
        return d_vn ? d_vn + slab(layer, seq) * cfg.n_ctx * cfg.n_kv : nullptr;
    }
};

#ifdef __CUDACC__
namespace bk {
// Raise the context's error word from a kernel (plain store: the word may live in host memory).
__device__ __forceinline__ void raise_error(int *flag, int code) {
    if (flag) {
        *reinterpret_cast<volatile int *>(flag) = code;
        __threadfence_system();
    }
}
}  // namespace bk
#endif

struct bk_event {
    cudaEvent_t ev = nullptr;
    int device = 0;
};

namespace bk {

bk_status fail(bk_ctx *ctx, bk_status st, const std::string &msg);
bk_status cuda_fail(bk_ctx *ctx, cudaError_t e, const char *what);
#define BK_CUDA(ctx, call)                                              \
    do {                                                                \
        cudaError_t e__ = (call);                                       \
        if (e__ != cudaSuccess) return bk::cuda_fail((ctx), e__, #call); \
    } while (0)

bk_status ensure_stage(bk_ctx *ctx, size_t bytes);
// Wait for the context's stream, then look at the error word the kernels raise when a bounded wait runs
// out: BK_ERR_CUDA (and the word and the split-K counters cleared) if one did.
bk_status sync_and_check(bk_ctx *ctx);

// ---- kernel launchers (bk_append.cu, bk_decode.cu, bk_kvq.cu) --------------

struct AppendArgs {
    const float *k, *v;        // [n_tokens][n_kv][hd]
    uint8_t *k_rows, *v_rows;  // slab base of (layer, seq) when desc == nullptr, else of layer
    float *k_norms, *v_norms;
    const float2 *rope;        // [rope_n_pos][n_rot/2]
    const float *givens;
    const float *book;         // codebook of this width (null unless planar)
    const uint2 *cell_tab;     // widths 1..4: the 512 cells of nearest_centroid_thr() (null otherwise)
    const int4 *desc;          // per token (seq, row, rope_pos, 0); nullptr = contiguous single sequence
    size_t seq_stride_rows;    // rows (pos*n_kv units) between sequences of one layer
    int n_tokens, n_kv, n_rot, bits;
    int row0, pos0;            // first cache row and rope position when desc == nullptr
    int k_kind, v_kind;
    size_t k_row_bytes, v_row_bytes;
};
bk_status launch_append(bk_ctx *ctx, const AppendArgs &a);

struct DecodeMeta {
    int n_seqs;
    int chunk_len;   // positions per split-K work item
    int n_items;
    int slot[kMaxSeqsPerLaunch];     // row of this sequence in the caller's q / out arrays
    int seq_id[kMaxSeqsPerLaunch];
    int n_pos[kMaxSeqsPerLaunch];
    int q_pos[kMaxSeqsPerLaunch];
    int item_start[kMaxSeqsPerLaunch + 1];
};
struct DecodeArgs {
    const uint8_t *k_rows, *v_rows;  // layer base: [seq][n_ctx][n_kv][row_bytes]
    const float *k_norms, *v_norms;  // layer base
    size_t seq_stride_rows;          // n_ctx * n_kv
    const float *q;                  // [n_seqs][n_head][hd]
    float *out;                      // [n_seqs][n_head][hd] or [n_seqs][n_head][hd+2] when partial
    int partial;
    const float2 *rope;
    int n_rot;
    const float *givens, *book;
    int bits, n_head, n_kv, k_kind, v_kind;
    size_t k_row_bytes, v_row_bytes;
    float *partials;
    unsigned *counters;
    int no_rope;  // 1: q is used as given (one-shot f32 attention)
    // tensor-core path only: host copies of the cache's tensor maps, and where (layer, sequence)
    // sits in them: position index = layer_pos0 + seq * n_ctx + pos
    const void *h_tmap_k, *h_tmap_v;
    int layer_pos0, n_ctx;
    // tensor-core path only: when set, the launch also stores the newest token (the fused form of
    // append + attend): k/v of that token, [n_kv][hd]; its row is n_pos - 1, its rope position q_pos
    const float *new_k, *new_v;
    uint8_t *k_rows_w, *v_rows_w;   // writable aliases of k_rows / v_rows
    float *k_norms_w, *v_norms_w;
    // The layer form of the step (src/forward.rs:237-245, 379-382 around the attention core):
    //   q_stride    floats between the q rows of consecutive heads (hd, or 2*hd when q is read in
    //               place from the interleaved [q | gate] projection output); tensor-core path only
    //   q_norm_w    when set, every q row gets the per-head RMSNorm with this weight [hd] first
    //               (tensor-core path only; the generic path norms q in a kernel of its own)
    //   k_norm_w    when set, the fused append norms the new k rows the same way before the rope
    //   gate        when set (and not partial), out = attention * sigmoid(gate): row of head h at
    //               gate + (slot * n_head + h) * gate_stride
    int q_stride, gate_stride;
    const float *q_norm_w, *k_norm_w, *gate;
    float eps;
    // Context split over several GPUs (bk_p2p.cu): when xch_peer is set, the CTA that finishes a
    // kv head does not write its rows to `out` but sends them (acc, m in ln units, l) to slot
    // [xch_rank] of every rank's mailbox, publishes them with the call's sequence number, waits
    // (bounded) for the same rows of every rank and writes their log-sum-exp merge to `out`.
    uint8_t *const *xch_peer;
    int xch_world, xch_rank;
    unsigned xch_seqno;
    int *xch_err;
    int xch_spin;  // polls of one arrival word before the exchange gives up
    // Set by launch_decode_group for the tensor-core kernels:
    //   dyn   bit 0: the warps of a CTA draw their tiles from a counter in shared memory instead of taking
    //         fixed shares (off by default: with it the last bits of a result depend on timing)
    //   dist  every CTA of the launch is resident at once (items <= SMs): the split-K combine is
    //         done in slices by all CTAs of a kv head instead of by the last one to arrive
    //   counters_other / other_n  the counter set the next launch will count in, and how many of its
    //         entries an earlier launch has left non-zero: CTA 0 clears them
    int dyn, dist;
    unsigned *counters_other;
    int other_n;
};
bk_status launch_decode(bk_ctx *ctx, const DecodeArgs &a, const DecodeMeta &m);

// Host-side planning shared by the decode entry points (bk_api.cu).
struct DecodeEntry {
    int slot, seq, np, qp;  // row in the caller's q/out arrays, sequence id, positions to scan, q position
};
void fill_decode_args(const bk_cache *c, int layer, int partial, DecodeArgs *out);
bk_status check_decode_entry(const bk_cache *c, int layer, int slot, const int32_t *seq_ids, const int32_t *n_pos,
                             const int32_t *q_pos, const char *who, DecodeEntry *e);
bk_status launch_decode_group(bk_ctx *ctx, const DecodeArgs &a, const DecodeEntry *list, int nb, bool use_mma,
                              int max_items);
bool decode_entry_uses_mma(const bk_ctx *ctx, const DecodeArgs &a, int n_pos);
bk_status bind_device(bk_ctx *ctx);
// One sequence's decode attention whose finishing CTAs exchange and merge their rows through the
// ranks' mailboxes (bk_api.cu; used by bk_decode_attn_split).
bk_status decode_with_exchange(bk_cache *c, int layer, int seq, int n_pos, int q_pos, const float *q_dev, float *out_dev,
                               uint8_t *const *d_peer, int world, int rank, unsigned seqno,
                               const float *new_k = nullptr, const float *new_v = nullptr);
// Tensor-core paths: 4-bit planar K and V (bk_decode_mma.cu) and f16 K and V (bk_decode_f16.cu).
// Chunks must be multiples of 16 positions.
bool decode_p4_mma_supported(const DecodeArgs &a);
bool decode_f16_mma_supported(const DecodeArgs &a);
inline bool decode_mma_supported(const DecodeArgs &a) { return decode_p4_mma_supported(a) || decode_f16_mma_supported(a); }
bk_status make_tile_tensor_maps(bk_ctx *ctx, const void *k_rows, const void *v_rows, size_t k_row_bytes, size_t v_row_bytes, int n_kv,
                                size_t total_pos, int box_rows, void *out_k, void *out_v);
bk_status launch_decode_p4_mma(bk_ctx *ctx, const DecodeArgs &a, const DecodeMeta &m, float alpha, bool qsplit, bool precise);
bk_status launch_decode_f16_mma(bk_ctx *ctx, const DecodeArgs &a, const DecodeMeta &m, float lut_alpha, bool qsplit);
// RMSNorm over rows (bk_layer.cu): up to two row groups per launch, each with its own source
// stride, weight and contiguous destination.
struct NormSeg {
    const float *src;
    size_t stride;   // floats between consecutive source rows
    const float *w;  // [row_len]
    float *dst;      // [n_rows][row_len]
    int n_rows;
};
bk_status launch_rms_norm_rows(bk_ctx *ctx, const NormSeg &s0, const NormSeg &s1, int row_len, float eps);

// PQ2_0 ternary rows (bk_pq2.cu): bytes per row, and y[t][r] = x[t] . row r for up to 2 tokens and 4 row ranges a launch.
size_t pq2_row_bytes(int64_t ne0);
bk_status launch_pq2_matvec(bk_ctx *ctx, int n_seg, const uint8_t *const *rows, const int *n_rows, float *const *y, int ne0,
                            const float *x, int n_tok);
// Batched causal attention of a block of prompt tokens over a 4- or 3-bit planar cache (bk_prefill.cu).
bool prefill_mma_supported(const DecodeArgs &a);
bk_status launch_prefill_mma(bk_ctx *ctx, const DecodeArgs &a, int seq, int pos0, int n_tokens, float alpha);
// The same on tcgen05 tensor cores with the accumulators in tensor memory (bk_prefill_umma.cu).
bool prefill_umma_supported(const DecodeArgs &a);  // planar4 / planar3 / f16 caches
bk_status launch_prefill_umma(bk_ctx *ctx, const DecodeArgs &a, int seq, int pos0, int n_tokens, float alpha);
bk_status launch_lse_merge(bk_ctx *ctx, int n_parts, int n_rows, int hd, const float *parts, float *out);

bk_status launch_quantize(bk_ctx *ctx, int bits, int n_vec, const float *x, uint8_t *packed, float *norms);
bk_status launch_dequantize(bk_ctx *ctx, int bits, int n_vec, const uint8_t *packed, const float *norms,
                            float *out);
bk_status launch_rotate(bk_ctx *ctx, int n_vec, int inverse, const float *x, float *out);
bk_status launch_dot_rotated(bk_ctx *ctx, int bits, int n_vec, const float *q_rot, const uint8_t *packed,
                             const float *norms, float *out);
// heads: [n_heads][hd] in place; rows4: [4][n_dims/2] (cos, sin) rows of the ids t, h, w, e;
// band: [n_dims/2] which of the four rows pair j uses.
bk_status launch_rope(bk_ctx *ctx, int n_heads, int hd, float *heads, const float2 *rows4, int n_dims,
                      const int *band);
bk_status launch_f32_to_half(bk_ctx *ctx, size_t n, const float *in, uint16_t *out);
bk_status launch_half_to_f32(bk_ctx *ctx, size_t n, const uint16_t *in, float *out);

}  // namespace bk
