// Prompt-cache snapshots: the cached tokens of one sequence, every layer, as one self-describing
// byte buffer that can be restored into any cache of the same mode and head geometry.
//
// The payload comes in either of the reference's two row layouts:
//   layout 0  the CPU stores of src/forward.rs:40-46: per layer K then V; f32 rows, or f16 rows
//             (k16/v16), or packed rows [pos][kv][32*bits] followed by the norms [pos][kv]
//             (kq, kn, then vq, vn - or v as f32 rows when only K is quantized);
//   layout 1  the device rows of shaders/kv_store_q.comp:119-123 for quantized sides: per
//             (pos, kv) the 8*bits packed words and then the norm's bit pattern as one more word;
//             f32 and f16 sides are as in layout 0.
// Header (little-endian u32 words): magic "BKVS", version 1, layout, mode kind, bits, v_quant,
// n_layers, n_kv, hd, reserved[3]; then n_layers words with the number of cached positions of
// each layer; then the layers' payloads.  Everything is host code over bk_cache_download /
// bk_cache_upload; the file or socket that carries the buffer is the caller's.
#include <cstring>
#include <string>
#include <vector>

#include "bk_internal.h"

namespace {

constexpr uint32_t kMagic = 0x53564b42u;  // "BKVS"
constexpr uint32_t kVersion = 1;
constexpr int kHeaderWords = 12;

struct Side {
    int kind;          // ROW_F32 / ROW_F16 / ROW_PLANAR
    size_t row_bytes;  // as stored in the cache (packed bytes for planar)
};

size_t side_bytes(const Side &s, size_t rows) {
    return rows * s.row_bytes + (s.kind == bk::ROW_PLANAR ? rows * sizeof(float) : 0);  // same total in both layouts
}

}  // namespace

extern "C" {

size_t bk_cache_snapshot_bytes(const bk_cache *c, int32_t seq) {
    if (!c || seq < 0 || seq >= c->cfg.n_seqs) return 0;
    const Side ks{c->k_kind, c->k_row_bytes}, vs{c->v_kind, c->v_row_bytes};
    size_t total = (size_t)(kHeaderWords + c->cfg.n_layers) * 4;
    for (int l = 0; l < c->cfg.n_layers; l++) {
        const size_t rows = (size_t)c->n_pos[c->slab(l, seq)] * c->cfg.n_kv;
        total += side_bytes(ks, rows) + side_bytes(vs, rows);
    }
    return total;
}

bk_status bk_cache_snapshot_save(bk_cache *c, int32_t seq, int32_t layout, void *buf, size_t buf_bytes, size_t *written) {
    using namespace bk;
    if (!c) return fail(nullptr, BK_ERR_INVALID, "bk_cache_snapshot_save: cache is null");
    bk_ctx *ctx = c->ctx;
    if (seq < 0 || seq >= c->cfg.n_seqs || (layout != 0 && layout != 1) || !buf)
        return fail(ctx, BK_ERR_INVALID, "bk_cache_snapshot_save: bad argument");
    const size_t need = bk_cache_snapshot_bytes(c, seq);
    if (buf_bytes < need)
        return fail(ctx, BK_ERR_RANGE, "bk_cache_snapshot_save: buffer of " + std::to_string(buf_bytes) + " bytes, " +
                                           std::to_string(need) + " needed");
    uint8_t *out = static_cast<uint8_t *>(buf);
    uint32_t hdr[kHeaderWords] = {kMagic, kVersion, (uint32_t)layout, (uint32_t)c->cfg.mode.kind,
                                  (uint32_t)(c->cfg.mode.kind == BK_MODE_PLANAR ? c->cfg.mode.bits : 0),
                                  (uint32_t)(c->cfg.mode.kind == BK_MODE_PLANAR ? c->cfg.mode.v_quant : 0),
                                  (uint32_t)c->cfg.n_layers, (uint32_t)c->cfg.n_kv, (uint32_t)c->cfg.hd, 0, 0, 0};
    memcpy(out, hdr, sizeof(hdr));
    size_t off = sizeof(hdr);
    for (int l = 0; l < c->cfg.n_layers; l++) {
        const uint32_t np = (uint32_t)c->n_pos[c->slab(l, seq)];
        memcpy(out + off, &np, 4);
        off += 4;
    }
    const Side sides[2] = {{c->k_kind, c->k_row_bytes}, {c->v_kind, c->v_row_bytes}};
    std::vector<uint8_t> rows_tmp;
    std::vector<float> norms_tmp;
    for (int l = 0; l < c->cfg.n_layers; l++) {
        const int np = c->n_pos[c->slab(l, seq)];
        const size_t rows = (size_t)np * c->cfg.n_kv;
        if (rows == 0) continue;
        for (int side = 0; side < 2; side++) {
            const Side &sd = sides[side];
            const bool planar = sd.kind == ROW_PLANAR;
            uint8_t *dst = out + off;
            void *rows_dst = dst;
            float *norms_dst = planar ? reinterpret_cast<float *>(dst + rows * sd.row_bytes) : nullptr;
            if (planar && layout == 1) {  // gather into temporaries, interleave below
                rows_tmp.resize(rows * sd.row_bytes);
                norms_tmp.resize(rows);
                rows_dst = rows_tmp.data();
                norms_dst = norms_tmp.data();
            }
            const bk_status st = side == 0 ? bk_cache_download(c, l, seq, 0, np, rows_dst, norms_dst, nullptr, nullptr)
                                           : bk_cache_download(c, l, seq, 0, np, nullptr, nullptr, rows_dst, norms_dst);
            if (st != BK_OK) return st;
            if (planar && layout == 1) {
                const size_t rb = sd.row_bytes;
                for (size_t r = 0; r < rows; r++) {
                    memcpy(dst + r * (rb + 4), rows_tmp.data() + r * rb, rb);
                    memcpy(dst + r * (rb + 4) + rb, &norms_tmp[r], 4);
                }
            }
            off += side_bytes(sd, rows);
        }
    }
    if (written) *written = off;
    return BK_OK;
}

bk_status bk_cache_snapshot_load(bk_cache *c, int32_t seq, const void *buf, size_t buf_bytes) {
    using namespace bk;
    if (!c) return fail(nullptr, BK_ERR_INVALID, "bk_cache_snapshot_load: cache is null");
    bk_ctx *ctx = c->ctx;
    if (seq < 0 || seq >= c->cfg.n_seqs || !buf) return fail(ctx, BK_ERR_INVALID, "bk_cache_snapshot_load: bad argument");
    const uint8_t *in = static_cast<const uint8_t *>(buf);
    uint32_t hdr[kHeaderWords];
    if (buf_bytes < sizeof(hdr)) return fail(ctx, BK_ERR_INVALID, "bk_cache_snapshot_load: buffer shorter than the header");
    memcpy(hdr, in, sizeof(hdr));
    if (hdr[0] != kMagic || hdr[1] != kVersion) return fail(ctx, BK_ERR_INVALID, "bk_cache_snapshot_load: not a snapshot (magic/version)");
    const uint32_t layout = hdr[2];
    if (layout > 1) return fail(ctx, BK_ERR_INVALID, "bk_cache_snapshot_load: unknown layout");
    const bool planar_mode = c->cfg.mode.kind == BK_MODE_PLANAR;
    if (hdr[3] != (uint32_t)c->cfg.mode.kind || hdr[4] != (uint32_t)(planar_mode ? c->cfg.mode.bits : 0) ||
        hdr[5] != (uint32_t)(planar_mode ? c->cfg.mode.v_quant : 0))
        return fail(ctx, BK_ERR_INVALID, "bk_cache_snapshot_load: the snapshot was taken in another KV mode");
    if (hdr[6] != (uint32_t)c->cfg.n_layers || hdr[7] != (uint32_t)c->cfg.n_kv || hdr[8] != (uint32_t)c->cfg.hd)
        return fail(ctx, BK_ERR_INVALID, "bk_cache_snapshot_load: layer count or head geometry differs");
    size_t off = sizeof(hdr);
    if (buf_bytes < off + (size_t)c->cfg.n_layers * 4) return fail(ctx, BK_ERR_INVALID, "bk_cache_snapshot_load: truncated");
    std::vector<uint32_t> np(c->cfg.n_layers);
    memcpy(np.data(), in + off, np.size() * 4);
    off += np.size() * 4;
    const Side sides[2] = {{c->k_kind, c->k_row_bytes}, {c->v_kind, c->v_row_bytes}};
    size_t need = off;
    for (int l = 0; l < c->cfg.n_layers; l++) {
        if (np[l] > (uint32_t)c->cfg.n_ctx)
            return fail(ctx, BK_ERR_RANGE, "bk_cache_snapshot_load: " + std::to_string(np[l]) + " positions exceed context " +
                                               std::to_string(c->cfg.n_ctx) + " (raise BONSAI_CTX)");
        const size_t rows = (size_t)np[l] * c->cfg.n_kv;
        need += side_bytes(sides[0], rows) + side_bytes(sides[1], rows);
    }
    if (buf_bytes < need) return fail(ctx, BK_ERR_INVALID, "bk_cache_snapshot_load: truncated");
    std::vector<uint8_t> rows_tmp;
    std::vector<float> norms_tmp;
    for (int l = 0; l < c->cfg.n_layers; l++) {
        const size_t rows = (size_t)np[l] * c->cfg.n_kv;
        if (rows > 0) {
            for (int side = 0; side < 2; side++) {
                const Side &sd = sides[side];
                const bool planar = sd.kind == ROW_PLANAR;
                const uint8_t *src = in + off;
                const void *rows_src = src;
                const float *norms_src = planar ? reinterpret_cast<const float *>(src + rows * sd.row_bytes) : nullptr;
                if (planar && layout == 1) {
                    const size_t rb = sd.row_bytes;
                    rows_tmp.resize(rows * rb);
                    norms_tmp.resize(rows);
                    for (size_t r = 0; r < rows; r++) {
                        memcpy(rows_tmp.data() + r * rb, src + r * (rb + 4), rb);
                        memcpy(&norms_tmp[r], src + r * (rb + 4) + rb, 4);
                    }
                    rows_src = rows_tmp.data();
                    norms_src = norms_tmp.data();
                } else if (planar) {  // the norms may sit at an address that is not 4-byte aligned for float access
                    norms_tmp.resize(rows);
                    memcpy(norms_tmp.data(), src + rows * sd.row_bytes, rows * 4);
                    norms_src = norms_tmp.data();
                }
                const bk_status st = side == 0
                                         ? bk_cache_upload(c, l, seq, 0, (int32_t)np[l], rows_src, norms_src, nullptr, nullptr)
                                         : bk_cache_upload(c, l, seq, 0, (int32_t)np[l], nullptr, nullptr, rows_src, norms_src);
                if (st != BK_OK) return st;
                off += side_bytes(sd, rows);
            }
        }
        const bk_status st = bk_cache_set_n_pos(c, l, seq, (int32_t)np[l]);
        if (st != BK_OK) return st;
    }
    return BK_OK;
}

}  // extern "C"
