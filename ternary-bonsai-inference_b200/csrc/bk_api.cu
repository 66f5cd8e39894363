// The C ABI of libbonsai_kv.so: contexts, caches, argument checks and launches.
// Declarations and the reference interface each entry point replaces are in
// include/bonsai_kv.h.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <new>
#include <string>

#include <cuda_fp16.h>

#include "bk_internal.h"

namespace bk {

// Scale alpha in [1, 2) that minimises the worst relative error of f16(alpha * c) / alpha over a
// codebook: the centroids are only 2^bits distinct values, so a good alpha makes all of them
// round almost exactly and the tensor-core path loses nothing to the f16 table.
// Host side of nearest_centroid_thr() (bk_device.cuh): the 512 (count, threshold) cells of one ascending
// codebook of n <= 16 centroids.  Everything is computed with the kernels' own single-precision operations
// (this file is built without floating-point contraction).  Returns false if a cell would hold two thresholds.
static bool build_threshold_cells(const float *book, int n, uint2 *tab) {
    auto key = [](float f) -> int64_t {  // floats in ascending order as integers
        int32_t b;
        memcpy(&b, &f, 4);
        return b >= 0 ? (int64_t)b : -(int64_t)(b & 0x7fffffff);
    };
    auto unkey = [](int64_t k) -> float {
        const int32_t b = k >= 0 ? (int32_t)k : (int32_t)((uint32_t)(-k) | 0x80000000u);
        float f;
        memcpy(&f, &b, 4);
        return f;
    };
    auto cell_of = [](float v) -> int {
        volatile float t = v + 0.25f;
        volatile float u = t * 1024.0f;
        const int c = (int)floorf(u);
        return c < 0 ? 0 : (c > 511 ? 511 : c);
    };
    float thr[16];
    int thr_cell[16];
    for (int i = 0; i + 1 < n; i++) {
        const float c0 = book[i], c1 = book[i + 1];
        auto beats = [&](float v) {  // does the scan move from centroid i to i + 1 at v?
            volatile float d0 = v - c0, d1 = v - c1;
            return fabsf(d1) < fabsf(d0);
        };
        int64_t lo = key(c0), hi = key(c1);  // beats(c0) is false, beats(c1) is true
        if (beats(c0) || !beats(c1)) return false;
        while (hi - lo > 1) {
            const int64_t mid = lo + (hi - lo) / 2;
            if (beats(unkey(mid))) hi = mid;
            else lo = mid;
        }
        thr[i] = unkey(hi);
        thr_cell[i] = cell_of(thr[i]);
        if (i > 0 && thr_cell[i] <= thr_cell[i - 1]) return false;  // two thresholds in one cell (or out of order)
    }
    const float inf = INFINITY;
    for (int k = 0; k < 512; k++) {
        uint32_t below = 0;
        float mine = inf;
        for (int i = 0; i + 1 < n; i++) {
            if (thr_cell[i] < k) below++;
            else if (thr_cell[i] == k) mine = thr[i];
        }
        uint32_t bits;
        memcpy(&bits, &mine, 4);
        tab[k] = make_uint2(below, bits);
    }
    return true;
}

static float best_lut_alpha(const float *book, int n) {
    // What reaches the output is the ABSOLUTE error of a centroid (times a row norm), and with a softmax
    // peaked on a few rows nothing averages it out: minimise the largest absolute error, the largest
    // relative one breaking ties.  (4 bit: 5.7e-6 on centroids up to 0.17; 3 bit: 7e-7.)
    float best_a = 1.0f, best_abs = 1e30f, best_rel = 1e30f;
    for (int i = 0; i < 65536; i++) {  // (one binade covers every alignment of the f16 grid)
        const float al = 1.0f + (float)i / 65536.0f;
        float worst_abs = 0.f, worst_rel = 0.f;
        for (int k = 0; k < n; k++) {
            const float c = book[k];
            if (c == 0.f) continue;
            const float r = __half2float(__float2half_rn(c * al)) / al;
            worst_abs = std::max(worst_abs, fabsf(r - c));
            worst_rel = std::max(worst_rel, fabsf(r - c) / fabsf(c));
        }
        if (worst_abs < best_abs || (worst_abs == best_abs && worst_rel < best_rel)) {
            best_abs = worst_abs;
            best_rel = worst_rel;
            best_a = al;
        }
    }
    return best_a;
}

static thread_local std::string g_err;  // failures that have no context to hang on

bk_status fail(bk_ctx *ctx, bk_status st, const std::string &msg) {
    if (ctx) ctx->err = msg;
    else g_err = msg;
    return st;
}

bk_status cuda_fail(bk_ctx *ctx, cudaError_t e, const char *what) {
    const bk_status st = (e == cudaErrorMemoryAllocation) ? BK_ERR_OOM : BK_ERR_CUDA;
    return fail(ctx, st, std::string(what) + ": " + cudaGetErrorString(e));
}

RopeTable::~RopeTable() {
    if (d) {
        cudaSetDevice(device);
        cudaFree(d);
    }
}

bk_status ensure_stage(bk_ctx *ctx, size_t bytes) {
    if (bytes <= ctx->h_stage_bytes && bytes <= ctx->d_stage_bytes) return BK_OK;
    BK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    size_t want = std::max<size_t>(bytes, 1 << 20);
    want = (want + 255) & ~(size_t)255;
    if (ctx->h_stage) cudaFreeHost(ctx->h_stage);
    if (ctx->d_stage) cudaFree(ctx->d_stage);
    ctx->h_stage = ctx->d_stage = nullptr;
    ctx->h_stage_bytes = ctx->d_stage_bytes = 0;
    BK_CUDA(ctx, cudaMallocHost(&ctx->h_stage, want));
    ctx->h_stage_bytes = want;
    BK_CUDA(ctx, cudaMalloc(&ctx->d_stage, want));
    ctx->d_stage_bytes = want;
    return BK_OK;
}

bk_status bind_device(bk_ctx *ctx) {
    BK_CUDA(ctx, cudaSetDevice(ctx->device));
    return BK_OK;
}
static bk_status bind(bk_ctx *ctx) { return bind_device(ctx); }

// A rope table for (n_rot, freq_base) that covers n_pos positions, shared between caches.
static bk_status get_rope(bk_ctx *ctx, int n_rot, float freq_base, int n_pos, std::shared_ptr<RopeTable> *out) {
    for (auto &t : ctx->ropes)
        if (t->n_rot == n_rot && t->freq_base == freq_base && t->n_pos >= n_pos) {
            *out = t;
            return BK_OK;
        }
    auto t = std::make_shared<RopeTable>();
    t->n_rot = n_rot;
    t->freq_base = freq_base;
    t->n_pos = n_pos;
    t->device = ctx->device;
    const size_t n = (size_t)n_pos * (n_rot / 2);
    if (n == 0) {
        *out = t;
        return BK_OK;
    }
    float2 *h = (float2 *)malloc(n * sizeof(float2));
    if (!h) return fail(ctx, BK_ERR_OOM, "rope table: host allocation failed");
    host_rope_rows(0, n_pos, n_rot, freq_base, h);
    cudaError_t e = cudaMalloc(&t->d, n * sizeof(float2));
    if (e == cudaSuccess) e = cudaMemcpy(t->d, h, n * sizeof(float2), cudaMemcpyHostToDevice);
    free(h);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "rope table upload");
    ctx->ropes.push_back(t);
    *out = t;
    return BK_OK;
}

static size_t row_bytes_of(int kind, int bits, int hd) {
    switch (kind) {
        case ROW_F32: return (size_t)hd * 4;
        case ROW_F16: return (size_t)hd * 2;
        default: return (size_t)hd * bits / 8;
    }
}

static bool valid_layer_seq(const bk_cache *c, int layer, int seq) {
    return c && layer >= 0 && layer < c->cfg.n_layers && seq >= 0 && seq < c->cfg.n_seqs;
}

// Rust's str::parse::<u32>: optional '+', then ASCII digits only.
static bool parse_u32(const char *s, size_t len, uint32_t *out) {
    size_t i = 0;
    if (len == 0) return false;
    if (s[0] == '+') i = 1;
    if (i >= len) return false;
    uint64_t v = 0;
    for (; i < len; i++) {
        if (s[i] < '0' || s[i] > '9') return false;
        v = v * 10 + (uint64_t)(s[i] - '0');
        if (v > 0xffffffffULL) return false;
    }
    *out = (uint32_t)v;
    return true;
}

}  // namespace bk

using namespace bk;

extern "C" {

const char *bk_version(void) { return "bonsai-kv-b200 0.1 (sm_100a)"; }

const char *bk_status_string(bk_status s) {
    switch (s) {
        case BK_OK: return "ok";
        case BK_ERR_INVALID: return "invalid argument";
        case BK_ERR_CUDA: return "CUDA error";
        case BK_ERR_OOM: return "out of memory";
        case BK_ERR_RANGE: return "position beyond the allocated context";
        case BK_ERR_UNSUPPORTED: return "unsupported geometry";
    }
    return "unknown status";
}

bk_status bk_ctx_create(int device, bk_ctx **out) {
    if (!out) return fail(nullptr, BK_ERR_INVALID, "bk_ctx_create: out is null");
    *out = nullptr;
    int n_dev = 0;
    cudaError_t e = cudaGetDeviceCount(&n_dev);
    if (e != cudaSuccess) return cuda_fail(nullptr, e, "cudaGetDeviceCount");
    if (device < 0 || device >= n_dev)
        return fail(nullptr, BK_ERR_INVALID, "bk_ctx_create: no CUDA device " + std::to_string(device));
    bk_ctx *ctx = new (std::nothrow) bk_ctx();
    if (!ctx) return fail(nullptr, BK_ERR_OOM, "bk_ctx_create: host allocation failed");
    ctx->device = device;
    auto bail = [&](cudaError_t err, const char *what) {
        bk_status st = cuda_fail(nullptr, err, what);
        bk_ctx_destroy(ctx);
        return st;
    };
    if ((e = cudaSetDevice(device)) != cudaSuccess) return bail(e, "cudaSetDevice");
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return bail(e, "cudaGetDeviceProperties");
    ctx->n_sms = prop.multiProcessorCount;
    if ((e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)) != cudaSuccess)
        return bail(e, "cudaStreamCreate");
    host_givens(kHd, ctx->h_givens);
    memset(ctx->h_codebooks, 0, sizeof(ctx->h_codebooks));
    for (int b = 1; b <= kMaxBits; b++) {
        host_codebook(kHd, b, ctx->h_codebooks + (b - 1) * kBookStride);
        ctx->lut_alpha[b] = best_lut_alpha(ctx->h_codebooks + (b - 1) * kBookStride, 1 << b);
        // the binary-search nearest-centroid of the kernels relies on well separated centroids
        const float *cb = ctx->h_codebooks + (b - 1) * kBookStride;
        for (int i = 0; i + 1 < (1 << b); i++)
            if (!(cb[i + 1] - cb[i] > 1e-5f)) {
                fail(nullptr, BK_ERR_UNSUPPORTED, "codebook centroids are not separated by more than 1e-5");
                bk_ctx_destroy(ctx);
                return BK_ERR_UNSUPPORTED;
            }
    }
    {
        const char *e1 = getenv("BONSAI_KV_GENERIC"), *e2 = getenv("BONSAI_KV_QSPLIT");
        ctx->force_generic = e1 && e1[0] == '1';
        const char *e3 = getenv("BONSAI_KV_PREFILL");
        ctx->prefill_umma = !(e3 && std::string(e3) == "mma");  // tcgen05 kernel unless BONSAI_KV_PREFILL=mma
        ctx->qsplit = !(e2 && e2[0] == '0');  // on unless BONSAI_KV_QSPLIT=0
        const char *e5 = getenv("BONSAI_KV_DYN"), *e6 = getenv("BONSAI_KV_DIST");
        ctx->dyn_tiles = e5 ? atoi(e5) : 0;
        ctx->dist_combine = !(e6 && e6[0] == '0');
    }
    if ((e = cudaMalloc(&ctx->d_givens, sizeof(ctx->h_givens))) != cudaSuccess) return bail(e, "cudaMalloc givens");
    {   // the threshold cells of the widths 1..4 (the append kernel's nearest-centroid search)
        std::vector<uint2> tabs(4 * 512);
        for (int b = 1; b <= 4; b++)
            if (!build_threshold_cells(ctx->h_codebooks + (b - 1) * kBookStride, 1 << b, tabs.data() + (b - 1) * 512)) {
                fail(nullptr, BK_ERR_UNSUPPORTED, "codebook thresholds do not fit the cell table");
                bk_ctx_destroy(ctx);
                return BK_ERR_UNSUPPORTED;
            }
        if ((e = cudaMalloc(&ctx->d_cell_tabs, tabs.size() * sizeof(uint2))) != cudaSuccess) return bail(e, "cudaMalloc cell tables");
        if ((e = cudaMemcpy(ctx->d_cell_tabs, tabs.data(), tabs.size() * sizeof(uint2), cudaMemcpyHostToDevice)) != cudaSuccess)
            return bail(e, "cudaMemcpy cell tables");
    }
    if ((e = cudaMalloc(&ctx->d_codebooks, sizeof(ctx->h_codebooks))) != cudaSuccess)
        return bail(e, "cudaMalloc codebooks");
    if ((e = cudaMemcpy(ctx->d_givens, ctx->h_givens, sizeof(ctx->h_givens), cudaMemcpyHostToDevice)) != cudaSuccess)
        return bail(e, "upload givens");
    if ((e = cudaMemcpy(ctx->d_codebooks, ctx->h_codebooks, sizeof(ctx->h_codebooks), cudaMemcpyHostToDevice)) !=
        cudaSuccess)
        return bail(e, "upload codebooks");
    const size_t part_bytes = (size_t)kMaxItems * kMaxRep * kScratchStride * sizeof(float);
    if ((e = cudaMalloc(&ctx->d_partials, part_bytes)) != cudaSuccess) return bail(e, "cudaMalloc partials");
    const size_t cnt_bytes = (size_t)kCtrTotal * sizeof(unsigned);
    if ((e = cudaMalloc(&ctx->d_counters, cnt_bytes)) != cudaSuccess) return bail(e, "cudaMalloc counters");
    if ((e = cudaMemset(ctx->d_counters, 0, cnt_bytes)) != cudaSuccess) return bail(e, "clear counters");
    {
        void *herr = nullptr, *derr = nullptr;
        if ((e = cudaHostAlloc(&herr, sizeof(int), cudaHostAllocMapped)) != cudaSuccess) return bail(e, "cudaHostAlloc error word");
        ctx->h_err = static_cast<volatile int *>(herr);
        *ctx->h_err = 0;
        if ((e = cudaHostGetDevicePointer(&derr, herr, 0)) != cudaSuccess) return bail(e, "cudaHostGetDevicePointer error word");
        ctx->d_err = static_cast<int *>(derr);
        const char *e7 = getenv("BONSAI_KV_XCH_POLLS");
        if (e7 && atoi(e7) > 0) ctx->xch_polls = atoi(e7);
        const char *e8 = getenv("BONSAI_KV_MMA_MIN");
        if (e8 && atoi(e8) > 0) ctx->mma_min_rows = atoi(e8);
    }
    *out = ctx;
    return BK_OK;
}

void bk_ctx_destroy(bk_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    ctx->ropes.clear();
    if (ctx->d_givens) cudaFree(ctx->d_givens);
    if (ctx->d_codebooks) cudaFree(ctx->d_codebooks);
    if (ctx->d_cell_tabs) cudaFree(ctx->d_cell_tabs);
    if (ctx->d_partials) cudaFree(ctx->d_partials);
    if (ctx->d_counters) cudaFree(ctx->d_counters);
    if (ctx->h_err) cudaFreeHost(const_cast<int *>(ctx->h_err));
    if (ctx->h_stage) cudaFreeHost(ctx->h_stage);
    if (ctx->d_stage) cudaFree(ctx->d_stage);
    if (ctx->d_layer) cudaFree(ctx->d_layer);
    if (ctx->d_prefill) cudaFree(ctx->d_prefill);
    if (ctx->h_desc) cudaFreeHost(ctx->h_desc);
    if (ctx->d_desc) cudaFree(ctx->d_desc);
    for (int i = 0; i < kDescSlots; i++)
        if (ctx->desc_ev[i]) cudaEventDestroy(ctx->desc_ev[i]);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char *bk_last_error(const bk_ctx *ctx) { return ctx ? ctx->err.c_str() : g_err.c_str(); }

}  // extern "C"

namespace bk {
bk_status sync_and_check(bk_ctx *ctx) {
    BK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const int flag = ctx->h_err ? *ctx->h_err : 0;
    if (flag) {
        *ctx->h_err = 0;
        // a kernel that gave up may have left arrival counters behind: start the next launch from zero
        cudaMemsetAsync(ctx->d_counters, 0, sizeof(unsigned) * kCtrTotal, ctx->stream);
        ctx->ctr_dirty[0] = ctx->ctr_dirty[1] = 0;
        static const char *const what[] = {"", "a tile copy did not arrive", "no room for the tile ring", "the context-split exchange (a peer never sent its rows) or a split-K copy did not arrive",
                                           "a tensor-memory operation of the prefill kernel did not complete", "a weight tile of the PQ2_0 matvec did not arrive",
                                           "the CTAs of a kv head did not all arrive for the split-K combine"};
        return fail(ctx, BK_ERR_CUDA, std::string("a kernel gave up a bounded wait (code ") + std::to_string(flag) + ": " +
                                          (flag > 0 && flag < 7 ? what[flag] : "unknown") + "); results of the calls since the last check are invalid");
    }
    return BK_OK;
}
}  // namespace bk

extern "C" {

bk_status bk_synchronize(bk_ctx *ctx) {
    if (!ctx) return fail(nullptr, BK_ERR_INVALID, "bk_synchronize: ctx is null");
    return sync_and_check(ctx);
}

void *bk_ctx_stream(bk_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }
int bk_ctx_device(const bk_ctx *ctx) { return ctx ? ctx->device : -1; }
uint64_t bk_ctx_launch_count(const bk_ctx *ctx) { return ctx ? ctx->launches : 0; }

/* ---- modes ----------------------------------------------------------------- */

bk_status bk_parse_mode(const char *s, bk_kv_mode *out) {
    if (!s || !out) return fail(nullptr, BK_ERR_INVALID, "bk_parse_mode: null argument");
    out->kind = BK_MODE_F32;
    out->bits = 0;
    out->v_quant = 0;
    size_t len = strlen(s);
    if (len == 0 || !strcmp(s, "f32")) return BK_OK;
    if (!strcmp(s, "f16") || !strcmp(s, "fp16") || !strcmp(s, "half")) {
        out->kind = BK_MODE_F16;
        return BK_OK;
    }
    bool k_only = false;
    if (s[len - 1] == 'k') {
        k_only = true;
        len--;
    }
    const char *digits = nullptr;
    size_t n_digits = 0;
    if (len >= 6 && !strncmp(s, "planar", 6)) {
        digits = s + 6;
        n_digits = len - 6;
    } else if (len >= 3 && !strncmp(s, "iso", 3)) {
        digits = s + 3;
        n_digits = len - 3;
    }
    uint32_t b = 0;
    if (!digits || !parse_u32(digits, n_digits, &b) || b < 1 || b > 8) return BK_OK;
    out->kind = BK_MODE_PLANAR;
    out->bits = (int32_t)b;
    out->v_quant = k_only ? 0 : 1;
    return BK_OK;
}

bk_status bk_mode_from_env(bk_kv_mode *out) {
    const char *v = getenv("BONSAI_KV");
    return bk_parse_mode(v ? v : "", out);
}

int32_t bk_n_ctx_from_env(void) {
    const char *v = getenv("BONSAI_CTX");
    uint32_t n = 0;
    if (v && parse_u32(v, strlen(v), &n) && n >= 16 && n <= 262144) return (int32_t)n;
    return 2048;
}

void bk_default_config(bk_cache_config *cfg) {
    if (!cfg) return;
    memset(cfg, 0, sizeof(*cfg));
    cfg->n_layers = 16;
    cfg->n_seqs = 1;
    cfg->n_ctx = 2048;
    cfg->n_head = 24;
    cfg->n_kv = 4;
    cfg->hd = 256;
    cfg->n_rot = 64;
    cfg->sections[0] = 11;
    cfg->sections[1] = 11;
    cfg->sections[2] = 10;
    cfg->sections[3] = 0;
    cfg->freq_base = 1e7f;
    cfg->rope_positions = 0;
    cfg->mode.kind = BK_MODE_F32;
}

/* ---- cache ----------------------------------------------------------------- */

bk_status bk_cache_create(bk_ctx *ctx, const bk_cache_config *cfg, bk_cache **out) {
    if (!ctx || !cfg || !out) return fail(ctx, BK_ERR_INVALID, "bk_cache_create: null argument");
    *out = nullptr;
    if (cfg->hd != kHd)
        return fail(ctx, BK_ERR_UNSUPPORTED, "bk_cache_create: head_dim must be 256, got " + std::to_string(cfg->hd));
    if (cfg->n_layers < 1 || cfg->n_seqs < 1 || cfg->n_ctx < 1 || cfg->n_kv < 1 || cfg->n_head < 1)
        return fail(ctx, BK_ERR_INVALID, "bk_cache_create: sizes must be positive");
    if (cfg->n_kv > 8) return fail(ctx, BK_ERR_UNSUPPORTED, "bk_cache_create: at most 8 kv heads");
    if (cfg->n_head % cfg->n_kv != 0)
        return fail(ctx, BK_ERR_INVALID, "bk_cache_create: n_head must be a multiple of n_kv");
    const int n_rep = cfg->n_head / cfg->n_kv;
    if (!(n_rep == 1 || n_rep == 2 || n_rep == 4 || n_rep == 6 || n_rep == 8))
        return fail(ctx, BK_ERR_UNSUPPORTED, "bk_cache_create: n_head/n_kv must be 1, 2, 4, 6 or 8");
    if (cfg->n_rot < 0 || cfg->n_rot > cfg->hd || (cfg->n_rot & 1))
        return fail(ctx, BK_ERR_INVALID, "bk_cache_create: n_rot must be even and <= head_dim");
    const int rope_n = cfg->rope_positions > 0 ? cfg->rope_positions : cfg->n_ctx;
    if (rope_n < cfg->n_ctx && cfg->rope_positions > 0)
        return fail(ctx, BK_ERR_INVALID, "bk_cache_create: rope_positions smaller than n_ctx");
    int k_kind, v_kind, bits = 0;
    switch (cfg->mode.kind) {
        case BK_MODE_F32: k_kind = v_kind = ROW_F32; break;
        case BK_MODE_F16: k_kind = v_kind = ROW_F16; break;
        case BK_MODE_PLANAR:
            bits = cfg->mode.bits;
            if (bits < 1 || bits > 8) return fail(ctx, BK_ERR_INVALID, "bk_cache_create: bits must be 1..8");
            k_kind = ROW_PLANAR;
            v_kind = cfg->mode.v_quant ? ROW_PLANAR : ROW_F32;
            break;
        default: return fail(ctx, BK_ERR_INVALID, "bk_cache_create: unknown mode");
    }
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    bk_cache *c = new (std::nothrow) bk_cache();
    if (!c) return fail(ctx, BK_ERR_OOM, "bk_cache_create: host allocation failed");
    c->ctx = ctx;
    c->cfg = *cfg;
    c->cfg.rope_positions = rope_n;
    c->k_kind = k_kind;
    c->v_kind = v_kind;
    c->k_row_bytes = row_bytes_of(k_kind, bits, kHd);
    c->v_row_bytes = row_bytes_of(v_kind, bits, kHd);
    // packed rows must stay 16-byte aligned for 128-bit access (cf. the word-alignment check
    // of src/gdev.rs:353-357); 32*bits bytes always is for hd = 256
    const size_t rows = (size_t)cfg->n_layers * cfg->n_seqs * cfg->n_ctx * cfg->n_kv;
    auto alloc = [&](void **p, size_t bytes) -> bk_status {
        cudaError_t e = cudaMalloc(p, bytes);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return cuda_fail(ctx, e, "cudaMalloc cache");
        }
        c->device_bytes += bytes;
        return BK_OK;
    };
    if ((st = alloc((void **)&c->d_k, rows * c->k_row_bytes)) != BK_OK ||
        (st = alloc((void **)&c->d_v, rows * c->v_row_bytes)) != BK_OK ||
        // norms carry one tile (32 positions) of slack: the tensor-core decode copies whole tiles
        (k_kind == ROW_PLANAR && (st = alloc((void **)&c->d_kn, (rows + 32 * cfg->n_kv) * 4)) != BK_OK) ||
        (v_kind == ROW_PLANAR && (st = alloc((void **)&c->d_vn, (rows + 32 * cfg->n_kv) * 4)) != BK_OK) ||
        (st = get_rope(ctx, cfg->n_rot, cfg->freq_base, rope_n, &c->rope)) != BK_OK) {
        bk_cache_destroy(c);
        return st;
    }
    c->n_pos.assign((size_t)cfg->n_layers * cfg->n_seqs, 0);
    // tiles of 16 positions: f16, f32, and 4- or 3-bit K beside f32 V; tiles of 32: K and V both 4, 3 or 2 bit
    const bool row_tiles = (k_kind == ROW_F16 && v_kind == ROW_F16) || (k_kind == ROW_F32 && v_kind == ROW_F32) ||
                           (k_kind == ROW_PLANAR && (bits == 4 || bits == 3) && v_kind == ROW_F32);
    if ((k_kind == ROW_PLANAR && v_kind == ROW_PLANAR && (bits == 4 || bits == 3 || bits == 2)) || row_tiles) {
        st = make_tile_tensor_maps(ctx, c->d_k, c->d_v, c->k_row_bytes, c->v_row_bytes, cfg->n_kv,
                                   (size_t)cfg->n_layers * cfg->n_seqs * cfg->n_ctx, row_tiles ? 16 : 32, c->tmap_k, c->tmap_v);
        if (st != BK_OK) {
            bk_cache_destroy(c);
            return st;
        }
        c->has_tmaps = true;
    }
    *out = c;
    return BK_OK;
}

void bk_cache_destroy(bk_cache *c) {
    if (!c) return;
    cudaSetDevice(c->ctx->device);
    cudaStreamSynchronize(c->ctx->stream);
    if (c->d_k) cudaFree(c->d_k);
    if (c->d_v) cudaFree(c->d_v);
    if (c->d_kn) cudaFree(c->d_kn);
    if (c->d_vn) cudaFree(c->d_vn);
    delete c;
}

bk_status bk_cache_reset(bk_cache *c, int32_t seq) {
    if (!c) return fail(nullptr, BK_ERR_INVALID, "bk_cache_reset: cache is null");
    if (seq >= c->cfg.n_seqs) return fail(c->ctx, BK_ERR_INVALID, "bk_cache_reset: no such sequence");
    for (int l = 0; l < c->cfg.n_layers; l++)
        for (int s = 0; s < c->cfg.n_seqs; s++)
            if (seq < 0 || s == seq) c->n_pos[c->slab(l, s)] = 0;
    return BK_OK;
}

int32_t bk_cache_n_pos(const bk_cache *c, int32_t layer, int32_t seq) {
    if (!valid_layer_seq(c, layer, seq)) return -1;
    return c->n_pos[c->slab(layer, seq)];
}

bk_status bk_cache_set_n_pos(bk_cache *c, int32_t layer, int32_t seq, int32_t n_pos) {
    if (!valid_layer_seq(c, layer, seq)) return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, "bk_cache_set_n_pos: bad layer/seq");
    if (n_pos < 0 || n_pos > c->cfg.n_ctx) return fail(c->ctx, BK_ERR_RANGE, "bk_cache_set_n_pos: beyond n_ctx");
    c->n_pos[c->slab(layer, seq)] = n_pos;
    return BK_OK;
}

bk_status bk_cache_get_config(const bk_cache *c, bk_cache_config *out) {
    if (!c || !out) return fail(nullptr, BK_ERR_INVALID, "bk_cache_get_config: null argument");
    *out = c->cfg;
    return BK_OK;
}

int32_t bk_cache_row_bytes(const bk_cache *c, int32_t is_v) {
    if (!c) return -1;
    const int kind = is_v ? c->v_kind : c->k_kind;
    return (int32_t)((is_v ? c->v_row_bytes : c->k_row_bytes) + (kind == ROW_PLANAR ? 4 : 0));
}

size_t bk_cache_device_bytes(const bk_cache *c) { return c ? c->device_bytes : 0; }

static bk_status cache_copy(bk_cache *c, int layer, int seq, int pos0, int n_pos, void *k_rows, float *k_norms,
                            void *v_rows, float *v_norms, bool to_host, const char *who) {
    if (!valid_layer_seq(c, layer, seq)) return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, std::string(who) + ": bad layer/seq");
    bk_ctx *ctx = c->ctx;
    if (pos0 < 0 || n_pos < 0 || (int64_t)pos0 + n_pos > c->cfg.n_ctx)
        return fail(ctx, BK_ERR_RANGE, std::string(who) + ": rows beyond n_ctx");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    if (n_pos == 0) return BK_OK;
    const size_t r0 = (size_t)pos0 * c->cfg.n_kv, nr = (size_t)n_pos * c->cfg.n_kv;
    const cudaMemcpyKind kind = to_host ? cudaMemcpyDeviceToHost : cudaMemcpyHostToDevice;
    auto cp = [&](void *host, void *dev, size_t bytes) -> cudaError_t {
        return to_host ? cudaMemcpyAsync(host, dev, bytes, kind, ctx->stream)
                       : cudaMemcpyAsync(dev, host, bytes, kind, ctx->stream);
    };
    if (k_rows) BK_CUDA(ctx, cp(k_rows, c->k_rows(layer, seq) + r0 * c->k_row_bytes, nr * c->k_row_bytes));
    if (v_rows) BK_CUDA(ctx, cp(v_rows, c->v_rows(layer, seq) + r0 * c->v_row_bytes, nr * c->v_row_bytes));
    if (k_norms && c->d_kn) BK_CUDA(ctx, cp(k_norms, c->k_norms(layer, seq) + r0, nr * 4));
    if (v_norms && c->d_vn) BK_CUDA(ctx, cp(v_norms, c->v_norms(layer, seq) + r0, nr * 4));
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    return BK_OK;
}

bk_status bk_cache_download(bk_cache *c, int32_t layer, int32_t seq, int32_t pos0, int32_t n_pos, void *k_rows,
                            float *k_norms, void *v_rows, float *v_norms) {
    return cache_copy(c, layer, seq, pos0, n_pos, k_rows, k_norms, v_rows, v_norms, true, "bk_cache_download");
}

bk_status bk_cache_upload(bk_cache *c, int32_t layer, int32_t seq, int32_t pos0, int32_t n_pos, const void *k_rows,
                          const float *k_norms, const void *v_rows, const float *v_norms) {
    return cache_copy(c, layer, seq, pos0, n_pos, (void *)k_rows, (float *)k_norms, (void *)v_rows, (float *)v_norms,
                      false, "bk_cache_upload");
}

/* ---- append ---------------------------------------------------------------- */

static AppendArgs base_append_args(const bk_cache *c, const float *k, const float *v) {
    AppendArgs a{};
    a.k = k;
    a.v = v;
    a.rope = c->rope->d;
    a.givens = c->ctx->d_givens;
    a.book = c->cfg.mode.kind == BK_MODE_PLANAR ? c->ctx->d_codebooks + (c->cfg.mode.bits - 1) * kBookStride : nullptr;
    a.cell_tab = (c->cfg.mode.kind == BK_MODE_PLANAR && c->cfg.mode.bits <= 4) ? c->ctx->d_cell_tabs + (c->cfg.mode.bits - 1) * 512 : nullptr;
    a.seq_stride_rows = (size_t)c->cfg.n_ctx * c->cfg.n_kv;
    a.n_kv = c->cfg.n_kv;
    a.n_rot = c->cfg.n_rot;
    a.bits = c->cfg.mode.kind == BK_MODE_PLANAR ? c->cfg.mode.bits : 0;
    a.k_kind = c->k_kind;
    a.v_kind = c->v_kind;
    a.k_row_bytes = c->k_row_bytes;
    a.v_row_bytes = c->v_row_bytes;
    return a;
}

bk_status bk_append(bk_cache *c, int32_t layer, int32_t seq, int32_t rope_pos, int32_t n_tokens, const float *k_dev,
                    const float *v_dev) {
    if (!valid_layer_seq(c, layer, seq)) return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, "bk_append: bad layer/seq");
    bk_ctx *ctx = c->ctx;
    if (n_tokens < 0 || rope_pos < 0) return fail(ctx, BK_ERR_INVALID, "bk_append: negative count or position");
    if (n_tokens == 0) return BK_OK;
    if (!k_dev || !v_dev) return fail(ctx, BK_ERR_INVALID, "bk_append: null k/v");
    int32_t &np = c->n_pos[c->slab(layer, seq)];
    if ((int64_t)np + n_tokens > c->cfg.n_ctx)
        return fail(ctx, BK_ERR_RANGE,
                    "bk_append: position " + std::to_string(np + n_tokens - 1) + " exceeds context " +
                        std::to_string(c->cfg.n_ctx) + " (raise BONSAI_CTX)");
    if ((int64_t)rope_pos + n_tokens > c->rope->n_pos)
        return fail(ctx, BK_ERR_RANGE, "bk_append: rope position beyond the rope table (rope_positions)");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    AppendArgs a = base_append_args(c, k_dev, v_dev);
    a.k_rows = c->k_rows(layer, seq);
    a.v_rows = c->v_rows(layer, seq);
    a.k_norms = c->k_norms(layer, seq);
    a.v_norms = c->v_norms(layer, seq);
    a.desc = nullptr;
    a.n_tokens = n_tokens;
    a.row0 = np;
    a.pos0 = rope_pos;
    st = launch_append(ctx, a);
    if (st == BK_OK) np += n_tokens;
    return st;
}

bk_status bk_append_host(bk_cache *c, int32_t layer, int32_t seq, int32_t rope_pos, int32_t n_tokens,
                         const float *k_host, const float *v_host) {
    if (!valid_layer_seq(c, layer, seq)) return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, "bk_append_host: bad layer/seq");
    bk_ctx *ctx = c->ctx;
    if (n_tokens < 0) return fail(ctx, BK_ERR_INVALID, "bk_append_host: negative count");
    if (n_tokens == 0) return BK_OK;
    if (!k_host || !v_host) return fail(ctx, BK_ERR_INVALID, "bk_append_host: null k/v");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    const size_t per = (size_t)n_tokens * c->cfg.n_kv * kHd * sizeof(float);
    if ((st = ensure_stage(ctx, 2 * per)) != BK_OK) return st;
    memcpy(ctx->h_stage, k_host, per);
    memcpy((char *)ctx->h_stage + per, v_host, per);
    BK_CUDA(ctx, cudaMemcpyAsync(ctx->d_stage, ctx->h_stage, 2 * per, cudaMemcpyHostToDevice, ctx->stream));
    st = bk_append(c, layer, seq, rope_pos, n_tokens, (const float *)ctx->d_stage,
                   (const float *)((char *)ctx->d_stage + per));
    if (st != BK_OK) return st;
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    return BK_OK;
}

bk_status bk_append_batch(bk_cache *c, int32_t layer, int32_t n_seqs, const int32_t *seq_ids, const int32_t *rope_pos,
                          const float *k_dev, const float *v_dev) {
    if (!c || layer < 0 || layer >= c->cfg.n_layers) return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, "bk_append_batch: bad layer");
    bk_ctx *ctx = c->ctx;
    if (n_seqs < 0) return fail(ctx, BK_ERR_INVALID, "bk_append_batch: negative count");
    if (n_seqs == 0) return BK_OK;
    if (!k_dev || !v_dev) return fail(ctx, BK_ERR_INVALID, "bk_append_batch: null k/v");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    if (n_seqs > kDescCap) return fail(ctx, BK_ERR_INVALID, "bk_append_batch: more than 4096 sequences in one call");
    if (!ctx->h_desc) {
        BK_CUDA(ctx, cudaMallocHost(&ctx->h_desc, sizeof(int4) * kDescCap * kDescSlots));
        BK_CUDA(ctx, cudaMalloc(&ctx->d_desc, sizeof(int4) * kDescCap * kDescSlots));
        for (int i = 0; i < kDescSlots; i++) BK_CUDA(ctx, cudaEventCreateWithFlags(&ctx->desc_ev[i], cudaEventDisableTiming));
    }
    const unsigned slot = ctx->desc_next % kDescSlots;
    if (ctx->desc_next >= (unsigned)kDescSlots) BK_CUDA(ctx, cudaEventSynchronize(ctx->desc_ev[slot]));
    int4 *h = ctx->h_desc + (size_t)slot * kDescCap;
    int4 *d = ctx->d_desc + (size_t)slot * kDescCap;
    const size_t slot_bytes = (size_t)n_seqs * sizeof(int4);
    for (int i = 0; i < n_seqs; i++) {
        const int s = seq_ids ? seq_ids[i] : i;
        if (s < 0 || s >= c->cfg.n_seqs) return fail(ctx, BK_ERR_INVALID, "bk_append_batch: bad sequence id");
        for (int j = 0; seq_ids && j < i; j++)
            if (seq_ids[j] == s) return fail(ctx, BK_ERR_INVALID, "bk_append_batch: duplicate sequence id");
        const int np = c->n_pos[c->slab(layer, s)];
        const int rp = rope_pos ? rope_pos[i] : np;
        if (np + 1 > c->cfg.n_ctx)
            return fail(ctx, BK_ERR_RANGE, "bk_append_batch: sequence " + std::to_string(s) + " is full (raise BONSAI_CTX)");
        if (rp < 0 || rp >= c->rope->n_pos) return fail(ctx, BK_ERR_RANGE, "bk_append_batch: rope position out of range");
        h[i] = make_int4(s, np, rp, 0);
    }
    BK_CUDA(ctx, cudaMemcpyAsync(d, h, slot_bytes, cudaMemcpyHostToDevice, ctx->stream));
    AppendArgs a = base_append_args(c, k_dev, v_dev);
    a.k_rows = c->k_rows(layer, 0);
    a.v_rows = c->v_rows(layer, 0);
    a.k_norms = c->k_norms(layer, 0);
    a.v_norms = c->v_norms(layer, 0);
    a.desc = d;
    a.n_tokens = n_seqs;
    st = launch_append(ctx, a);
    if (st != BK_OK) return st;
    BK_CUDA(ctx, cudaEventRecord(ctx->desc_ev[slot], ctx->stream));
    ctx->desc_next++;
    for (int i = 0; i < n_seqs; i++) c->n_pos[c->slab(layer, seq_ids ? seq_ids[i] : i)]++;
    return BK_OK;
}

/* ---- decode ---------------------------------------------------------------- */

}  // extern "C"

namespace bk {

void fill_decode_args(const bk_cache *c, int layer, int partial, DecodeArgs *out) {
    bk_ctx *ctx = c->ctx;
    DecodeArgs a{};
    a.k_rows = c->k_rows(layer, 0);
    a.v_rows = c->v_rows(layer, 0);
    a.k_norms = c->k_norms(layer, 0);
    a.v_norms = c->v_norms(layer, 0);
    a.seq_stride_rows = (size_t)c->cfg.n_ctx * c->cfg.n_kv;
    a.partial = partial;
    a.rope = c->rope->d;
    a.n_rot = c->cfg.n_rot;
    a.givens = ctx->d_givens;
    a.bits = c->cfg.mode.kind == BK_MODE_PLANAR ? c->cfg.mode.bits : 0;
    a.book = a.bits ? ctx->d_codebooks + (a.bits - 1) * kBookStride : nullptr;
    a.n_head = c->cfg.n_head;
    a.n_kv = c->cfg.n_kv;
    a.k_kind = c->k_kind;
    a.v_kind = c->v_kind;
    a.k_row_bytes = c->k_row_bytes;
    a.v_row_bytes = c->v_row_bytes;
    a.partials = ctx->d_partials;
    a.counters = ctx->d_counters;
    a.no_rope = 0;
    a.h_tmap_k = c->has_tmaps ? c->tmap_k : nullptr;
    a.h_tmap_v = c->has_tmaps ? c->tmap_v : nullptr;
    a.layer_pos0 = layer * c->cfg.n_seqs * c->cfg.n_ctx;
    a.n_ctx = c->cfg.n_ctx;
    a.new_k = a.new_v = nullptr;
    a.q_stride = a.gate_stride = kHd;
    a.q_norm_w = a.k_norm_w = a.gate = nullptr;
    a.eps = 0.f;
    a.xch_peer = nullptr;
    a.xch_world = a.xch_rank = 0;
    a.xch_seqno = 0;
    a.xch_err = ctx->d_err;
    a.xch_spin = ctx->xch_polls;
    a.dyn = a.dist = 0;
    a.counters_other = nullptr;
    a.other_n = 0;
    a.k_rows_w = c->k_rows(layer, 0);
    a.v_rows_w = c->v_rows(layer, 0);
    a.k_norms_w = c->k_norms(layer, 0);
    a.v_norms_w = c->v_norms(layer, 0);
    *out = a;
}

bk_status check_decode_entry(const bk_cache *c, int layer, int slot, const int32_t *seq_ids, const int32_t *n_pos,
                             const int32_t *q_pos, const char *who, DecodeEntry *e) {
    bk_ctx *ctx = c->ctx;
    const int s = seq_ids ? seq_ids[slot] : slot;
    if (s < 0 || s >= c->cfg.n_seqs) return fail(ctx, BK_ERR_INVALID, std::string(who) + ": bad sequence id");
    const int np = n_pos ? n_pos[slot] : c->n_pos[c->slab(layer, s)];
    if (np < 0 || np > c->cfg.n_ctx) return fail(ctx, BK_ERR_RANGE, std::string(who) + ": n_pos beyond n_ctx");
    const int qp = q_pos ? q_pos[slot] : std::max(np - 1, 0);
    if (qp < 0 || qp >= c->rope->n_pos)
        return fail(ctx, BK_ERR_RANGE, std::string(who) + ": q position beyond the rope table");
    *e = DecodeEntry{slot, s, np, qp};
    return BK_OK;
}

// One launch for up to kMaxSeqsPerLaunch sequences of one class.  Chunk length: generic kernel
// about 4 CTAs per SM over the whole launch, at least 64 positions each; tensor-core kernel one
// CTA per SM in one wave (chunks in units of 128 positions), or whole sequences when there are
// at least as many (sequence, kv head) pairs as SMs; never more than max_items work items (the
// capacity of the split-K scratch behind a.partials).
bk_status launch_decode_group(bk_ctx *ctx, const DecodeArgs &a, const DecodeEntry *list, int nb, bool use_mma,
                              int max_items) {
    const int n_kv = a.n_kv;
    if ((int64_t)nb * n_kv > max_items)
        return fail(ctx, BK_ERR_INVALID, "decode: more (sequence, kv head) pairs than the split-K scratch holds");
    DecodeMeta m{};
    m.n_seqs = nb;
    // Longest first: the hardware hands CTAs out in index order, so a launch of more items than SMs then
    // ends with its short items (slot[] keeps every sequence's place in the caller's arrays).
    int order[kMaxSeqsPerLaunch];
    for (int i = 0; i < nb; i++) order[i] = i;
    std::stable_sort(order, order + nb, [&](int x, int y) { return list[x].np > list[y].np; });
    int64_t total = 0;
    int max_np = 0, min_np = INT32_MAX;
    for (int i = 0; i < nb; i++) {
        const DecodeEntry &e = list[order[i]];
        m.slot[i] = e.slot;
        m.seq_id[i] = e.seq;
        m.n_pos[i] = e.np;
        m.q_pos[i] = e.qp;
        total += e.np;
        max_np = std::max(max_np, e.np);
        min_np = std::min(min_np, e.np);
    }
    const int64_t gran = use_mma ? 128 : 64;
    auto items_for = [&](int64_t len) {
        int64_t items = 0;
        for (int i = 0; i < nb; i++) items += (int64_t)n_kv * ((m.n_pos[i] + len - 1) / len);
        return items;
    };
    int64_t L;
    if (use_mma && (int64_t)nb * n_kv >= ctx->n_sms) {
        // At least one (sequence, kv head) pair per SM: no split at all.  Every CTA scans a whole sequence
        // and writes its output itself: no partials, no combine, and the SMs pick up the next pair as they
        // finish (longest first).
        L = ((int64_t)max_np + gran - 1) / gran * gran;
    } else if (use_mma) {
        // Fewer pairs than SMs: one wave.  The balanced chunk length, grown until the items fit the SMs, so
        // that all CTAs are resident together (which the slice form of the split-K combine needs) and no
        // second, nearly empty wave doubles the launch.
        const int64_t target_items = std::max<int64_t>(1, (int64_t)ctx->n_sms / n_kv);
        L = (total + target_items - 1) / target_items;
        L = std::max<int64_t>(gran, (L + gran - 1) / gran * gran);
        while (items_for(L) > ctx->n_sms && L < max_np) L += gran;
    } else {
        const int64_t target_items = std::max<int64_t>(1, (int64_t)ctx->n_sms * 4 / n_kv);  // about four CTAs per SM
        L = (total + target_items - 1) / target_items;
        L = std::max<int64_t>(gran, (L + gran - 1) / gran * gran);
    }
    while (items_for(L) > max_items) L *= 2;
    m.chunk_len = (int)L;
    int items = 0;
    for (int i = 0; i < nb; i++) {
        m.item_start[i] = items;
        items += n_kv * (int)((m.n_pos[i] + L - 1) / L);
    }
    m.item_start[nb] = items;
    m.n_items = items;
    if (!use_mma) return launch_decode(ctx, a, m);
    DecodeArgs a2 = a;
    a2.dyn = ctx->dyn_tiles;
    if (a.counters == ctx->d_counters) {  // (a caller with its own scratch clears it itself before every call)
        const int set = ctx->ctr_set;
        a2.counters = ctx->d_counters + (size_t)kCtrSet * (1 + set);
        a2.counters_other = ctx->d_counters + (size_t)kCtrSet * (2 - set);
        a2.other_n = ctx->ctr_dirty[1 - set];
        ctx->ctr_dirty[set] = std::max(ctx->ctr_dirty[set], nb * n_kv);
        ctx->ctr_dirty[1 - set] = 0;
        ctx->ctr_set = 1 - set;
    }
    // every CTA holds a whole SM, so a launch of at most n_sms items is resident all at once
    a2.dist = (ctx->dist_combine && items <= ctx->n_sms) ? 1 : 0;
    return decode_f16_mma_supported(a) ? launch_decode_f16_mma(ctx, a2, m, a.k_kind == ROW_PLANAR ? ctx->lut_alpha[a.bits] : 1.0f, ctx->qsplit)
                               : launch_decode_p4_mma(ctx, a2, m, ctx->lut_alpha[a.bits], ctx->qsplit, min_np < kMmaMinPos);
}

bool decode_entry_uses_mma(const bk_ctx *ctx, const DecodeArgs &a, int n_pos) {
    // Sequences of kRowMinPos rows and more take the tensor-core kernels (append fused in, one launch: faster than
    // the generic kernel plus the append kernel even at 256 rows).  The row kernel (f16, f32, K-only) carries about
    // 22 bits at any length; the 4-, 3- and 2-bit kernel's f16 table (relative error ~1e-4 per centroid) is only
    // averaged out over long contexts, so a launch with a sequence below kMmaMinPos rows runs its precise form
    // (launch_decode_group), which carries the table's rounding remainders.
    if (ctx->force_generic || !decode_mma_supported(a)) return false;
    return n_pos >= (ctx->mma_min_rows > 0 ? ctx->mma_min_rows : kRowMinPos);
}

}  // namespace bk

static bk_status decode_impl(bk_cache *c, int32_t layer, int32_t n_seqs, const int32_t *seq_ids, const int32_t *n_pos,
                             const int32_t *q_pos, const float *q_dev, float *out_dev, int partial, const char *who,
                             const float *gate_dev = nullptr, int gate_stride = kHd) {
    if (!c || layer < 0 || layer >= c->cfg.n_layers)
        return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, std::string(who) + ": bad layer");
    bk_ctx *ctx = c->ctx;
    if (n_seqs < 0) return fail(ctx, BK_ERR_INVALID, std::string(who) + ": negative count");
    if (n_seqs == 0) return BK_OK;
    if (!q_dev || !out_dev) return fail(ctx, BK_ERR_INVALID, std::string(who) + ": null q/out");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    const size_t out_stride = (size_t)c->cfg.n_head * (partial ? kPartStride : kHd);
    DecodeArgs a;
    fill_decode_args(c, layer, partial, &a);
    a.q = q_dev;
    a.out = out_dev;
    a.gate = partial ? nullptr : gate_dev;
    a.gate_stride = gate_stride;

    // Validate everything first, then sort the sequences into the two kernel classes.
    std::vector<DecodeEntry> cls[2];
    for (int i = 0; i < n_seqs; i++) {
        DecodeEntry e;
        if ((st = check_decode_entry(c, layer, i, seq_ids, n_pos, q_pos, who, &e)) != BK_OK) return st;
        if (e.np == 0) {  // nothing to attend to: zeros (and l = 0 for partials)
            BK_CUDA(ctx, cudaMemsetAsync(out_dev + (size_t)i * out_stride, 0, out_stride * sizeof(float), ctx->stream));
            continue;
        }
        cls[decode_entry_uses_mma(ctx, a, e.np) ? 1 : 0].push_back(e);
    }
    for (int k = 0; k < 2; k++)
        for (size_t base = 0; base < cls[k].size(); base += kMaxSeqsPerLaunch) {
            const int nb = (int)std::min<size_t>(kMaxSeqsPerLaunch, cls[k].size() - base);
            if ((st = launch_decode_group(ctx, a, cls[k].data() + base, nb, k == 1, kMaxItems)) != BK_OK) return st;
        }
    return BK_OK;
}

namespace bk {
bk_status decode_with_exchange(bk_cache *c, int layer, int seq, int n_pos, int q_pos, const float *q_dev, float *out_dev,
                               uint8_t *const *d_peer, int world, int rank, unsigned seqno, const float *new_k,
                               const float *new_v) {
    bk_ctx *ctx = c->ctx;
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    DecodeArgs a;
    fill_decode_args(c, layer, 0, &a);
    if (new_k) {  // this rank owns the tail: the new token becomes row n_pos - 1 (already counted in n_pos)
        if (decode_entry_uses_mma(ctx, a, n_pos)) {
            a.new_k = new_k;
            a.new_v = new_v;
        } else {  // caches without the fused append: store first (n_pos is one ahead of the cache's count)
            if ((st = bk_append(c, layer, seq, q_pos, 1, new_k, new_v)) != BK_OK) return st;
        }
    }
    a.q = q_dev;
    a.out = out_dev;
    a.xch_peer = d_peer;
    a.xch_world = world;
    a.xch_rank = rank;
    a.xch_seqno = seqno;
    DecodeEntry e;
    if ((st = check_decode_entry(c, layer, 0, &seq, &n_pos, &q_pos, "bk_decode_attn_split", &e)) != BK_OK) return st;
    if (e.np <= 0) return fail(ctx, BK_ERR_INVALID, "bk_decode_attn_split: empty chunk on the fused path");
    return launch_decode_group(ctx, a, &e, 1, decode_entry_uses_mma(ctx, a, e.np), kMaxItems);
}
}  // namespace bk

extern "C" {

bk_status bk_decode_attn(bk_cache *c, int32_t layer, int32_t n_seqs, const int32_t *seq_ids, const int32_t *n_pos,
                         const int32_t *q_pos, const float *q_dev, float *out_dev) {
    return decode_impl(c, layer, n_seqs, seq_ids, n_pos, q_pos, q_dev, out_dev, 0, "bk_decode_attn");
}

bk_status bk_decode_attn_partial(bk_cache *c, int32_t layer, int32_t n_seqs, const int32_t *seq_ids,
                                 const int32_t *n_pos, const int32_t *q_pos, const float *q_dev, float *part_dev) {
    return decode_impl(c, layer, n_seqs, seq_ids, n_pos, q_pos, q_dev, part_dev, 1, "bk_decode_attn_partial");
}

bk_status bk_lse_merge(bk_ctx *ctx, int32_t n_parts, int32_t n_rows, int32_t hd, const float *parts_dev,
                       float *out_dev) {
    if (!ctx) return fail(nullptr, BK_ERR_INVALID, "bk_lse_merge: ctx is null");
    if (n_parts < 1 || n_rows < 0 || hd < 1 || !parts_dev || !out_dev)
        return fail(ctx, BK_ERR_INVALID, "bk_lse_merge: bad argument");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    return launch_lse_merge(ctx, n_parts, n_rows, hd, parts_dev, out_dev);
}

bk_status bk_attn_step(bk_cache *c, int32_t layer, int32_t seq, int32_t pos, const float *q_dev, const float *k_dev,
                       const float *v_dev, float *out_dev) {
    if (!valid_layer_seq(c, layer, seq)) return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, "bk_attn_step: bad layer/seq");
    bk_ctx *ctx = c->ctx;
    if (pos >= c->cfg.n_ctx)
        return fail(ctx, BK_ERR_RANGE,
                    "bk_attn_step: position " + std::to_string(pos) + " exceeds context " +
                        std::to_string(c->cfg.n_ctx) + " (raise BONSAI_CTX)");
    if (pos != c->n_pos[c->slab(layer, seq)])  // debug_assert_eq!(cache.n_pos(il), pos + 1), src/forward.rs:285
        return fail(ctx, BK_ERR_INVALID,
                    "bk_attn_step: pos " + std::to_string(pos) + " is not the next row (" +
                        std::to_string(c->n_pos[c->slab(layer, seq)]) + ")");
    const int32_t np = pos + 1, qp = pos;
    // Long 4-bit caches: one launch does both halves of the step (the CTA that scans the last
    // chunk of each kv head first ropes, quantizes and stores that head's new rows).
    {
        DecodeArgs a;
        fill_decode_args(c, layer, 0, &a);
        if (decode_entry_uses_mma(ctx, a, np)) {
            if (!q_dev || !k_dev || !v_dev || !out_dev) return fail(ctx, BK_ERR_INVALID, "bk_attn_step: null argument");
            if (pos >= c->rope->n_pos) return fail(ctx, BK_ERR_RANGE, "bk_attn_step: position beyond the rope table");
            bk_status st = bind(ctx);
            if (st != BK_OK) return st;
            a.q = q_dev;
            a.out = out_dev;
            a.new_k = k_dev;
            a.new_v = v_dev;
            const DecodeEntry e{0, seq, np, qp};
            st = launch_decode_group(ctx, a, &e, 1, true, kMaxItems);
            if (st == BK_OK) c->n_pos[c->slab(layer, seq)] = np;
            return st;
        }
    }
    bk_status st = bk_append(c, layer, seq, pos, 1, k_dev, v_dev);
    if (st != BK_OK) return st;
    return decode_impl(c, layer, 1, &seq, &np, &qp, q_dev, out_dev, 0, "bk_attn_step");
}

bk_status bk_attn_step_host(bk_cache *c, int32_t layer, int32_t seq, int32_t pos, const float *q_host,
                            const float *k_host, const float *v_host, float *out_host) {
    if (!valid_layer_seq(c, layer, seq)) return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, "bk_attn_step_host: bad layer/seq");
    bk_ctx *ctx = c->ctx;
    if (!q_host || !k_host || !v_host || !out_host) return fail(ctx, BK_ERR_INVALID, "bk_attn_step_host: null argument");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    const size_t qb = (size_t)c->cfg.n_head * kHd * sizeof(float), kb = (size_t)c->cfg.n_kv * kHd * sizeof(float);
    if ((st = ensure_stage(ctx, 2 * qb + 2 * kb)) != BK_OK) return st;
    char *h = (char *)ctx->h_stage, *d = (char *)ctx->d_stage;
    memcpy(h, q_host, qb);
    memcpy(h + qb, k_host, kb);
    memcpy(h + qb + kb, v_host, kb);
    BK_CUDA(ctx, cudaMemcpyAsync(d, h, qb + 2 * kb, cudaMemcpyHostToDevice, ctx->stream));
    // The output goes straight into the pinned staging buffer (device-addressable under unified
    // addressing): the CTAs that finish the kv heads write their 6 KB over the bus themselves, which
    // saves the copy-back call of a step that is all latency.
    float *h_out = (float *)(h + qb + 2 * kb);
    st = bk_attn_step(c, layer, seq, pos, (const float *)d, (const float *)(d + qb), (const float *)(d + qb + kb), h_out);
    if (st != BK_OK) return st;
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    memcpy(out_host, h_out, qb);
    return BK_OK;
}

bk_status bk_attn_step_batch(bk_cache *c, int32_t layer, int32_t n_seqs, const int32_t *seq_ids, const float *q_dev,
                             const float *k_dev, const float *v_dev, float *out_dev) {
    if (!c || layer < 0 || layer >= c->cfg.n_layers) return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, "bk_attn_step_batch: bad layer");
    bk_ctx *ctx = c->ctx;
    if (n_seqs < 0) return fail(ctx, BK_ERR_INVALID, "bk_attn_step_batch: negative count");
    if (n_seqs == 0) return BK_OK;
    if (!q_dev || !k_dev || !v_dev || !out_dev) return fail(ctx, BK_ERR_INVALID, "bk_attn_step_batch: null argument");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    DecodeArgs a;
    fill_decode_args(c, layer, 0, &a);
    // One launch when every sequence takes a tensor-core kernel (which stores the new rows itself);
    // otherwise the batched append and the batched decode, two launches.
    bool all_fused = n_seqs <= kMaxSeqsPerLaunch;
    std::vector<DecodeEntry> list((size_t)n_seqs);
    for (int i = 0; i < n_seqs && all_fused; i++) {
        const int s = seq_ids ? seq_ids[i] : i;
        if (s < 0 || s >= c->cfg.n_seqs) return fail(ctx, BK_ERR_INVALID, "bk_attn_step_batch: bad sequence id");
        for (int j = 0; seq_ids && j < i; j++)
            if (seq_ids[j] == s) return fail(ctx, BK_ERR_INVALID, "bk_attn_step_batch: duplicate sequence id");
        const int np = c->n_pos[c->slab(layer, s)];
        if (np + 1 > c->cfg.n_ctx)
            return fail(ctx, BK_ERR_RANGE, "bk_attn_step_batch: sequence " + std::to_string(s) + " is full (raise BONSAI_CTX)");
        if (np >= c->rope->n_pos) return fail(ctx, BK_ERR_RANGE, "bk_attn_step_batch: position beyond the rope table");
        all_fused = decode_entry_uses_mma(ctx, a, np + 1);
        list[i] = DecodeEntry{i, s, np + 1, np};
    }
    if (all_fused) {
        a.q = q_dev;
        a.out = out_dev;
        a.new_k = k_dev;
        a.new_v = v_dev;
        st = launch_decode_group(ctx, a, list.data(), n_seqs, true, kMaxItems);
        if (st != BK_OK) return st;
        for (int i = 0; i < n_seqs; i++) c->n_pos[c->slab(layer, list[i].seq)]++;
        return BK_OK;
    }
    if ((st = bk_append_batch(c, layer, n_seqs, seq_ids, nullptr, k_dev, v_dev)) != BK_OK) return st;
    return decode_impl(c, layer, n_seqs, seq_ids, nullptr, nullptr, q_dev, out_dev, 0, "bk_attn_step_batch");
}

bk_status bk_prefill_attn(bk_cache *c, int32_t layer, int32_t seq, int32_t pos0, int32_t n_tokens, const float *q_dev,
                          float *out_dev) {
    if (!valid_layer_seq(c, layer, seq)) return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, "bk_prefill_attn: bad layer/seq");
    bk_ctx *ctx = c->ctx;
    if (pos0 < 0 || n_tokens < 0) return fail(ctx, BK_ERR_INVALID, "bk_prefill_attn: negative position or count");
    if (n_tokens == 0) return BK_OK;
    if (!q_dev || !out_dev) return fail(ctx, BK_ERR_INVALID, "bk_prefill_attn: null q/out");
    const int32_t have = c->n_pos[c->slab(layer, seq)];
    if ((int64_t)pos0 + n_tokens > have)
        return fail(ctx, BK_ERR_RANGE,
                    "bk_prefill_attn: tokens " + std::to_string(pos0) + ".." + std::to_string(pos0 + n_tokens - 1) +
                        " are not in the cache yet (" + std::to_string(have) + " rows): append them first");
    if ((int64_t)pos0 + n_tokens > c->rope->n_pos)
        return fail(ctx, BK_ERR_RANGE, "bk_prefill_attn: position beyond the rope table");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    DecodeArgs a;
    fill_decode_args(c, layer, 0, &a);
    a.q = q_dev;
    a.out = out_dev;
    if (!ctx->force_generic && n_tokens >= 4) {
        const float alpha = a.bits ? ctx->lut_alpha[a.bits] : 1.0f;
        if (ctx->prefill_umma && prefill_umma_supported(a)) return launch_prefill_umma(ctx, a, seq, pos0, n_tokens, alpha);
        if (prefill_mma_supported(a)) return launch_prefill_mma(ctx, a, seq, pos0, n_tokens, alpha);
    }
    // Other caches and very short blocks: the decode kernels with one entry per token (each token
    // re-reads the rows it sees).
    std::vector<int32_t> ids(kMaxSeqsPerLaunch, seq), np(kMaxSeqsPerLaunch), qp(kMaxSeqsPerLaunch);
    for (int t0 = 0; t0 < n_tokens; t0 += kMaxSeqsPerLaunch) {
        const int nb = std::min<int>(kMaxSeqsPerLaunch, n_tokens - t0);
        for (int i = 0; i < nb; i++) {
            np[i] = pos0 + t0 + i + 1;
            qp[i] = pos0 + t0 + i;
        }
        st = decode_impl(c, layer, nb, ids.data(), np.data(), qp.data(), q_dev + (size_t)t0 * c->cfg.n_head * kHd,
                         out_dev + (size_t)t0 * c->cfg.n_head * kHd, 0, "bk_prefill_attn");
        if (st != BK_OK) return st;
    }
    return BK_OK;
}

bk_status bk_prefill_step(bk_cache *c, int32_t layer, int32_t seq, int32_t pos0, int32_t n_tokens, const float *q_dev,
                          const float *k_dev, const float *v_dev, float *out_dev) {
    if (!valid_layer_seq(c, layer, seq)) return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, "bk_prefill_step: bad layer/seq");
    if (pos0 != c->n_pos[c->slab(layer, seq)])
        return fail(c->ctx, BK_ERR_INVALID,
                    "bk_prefill_step: pos " + std::to_string(pos0) + " is not the next row (" +
                        std::to_string(c->n_pos[c->slab(layer, seq)]) + ")");
    bk_status st = bk_append(c, layer, seq, pos0, n_tokens, k_dev, v_dev);
    if (st != BK_OK) return st;
    return bk_prefill_attn(c, layer, seq, pos0, n_tokens, q_dev, out_dev);
}

bk_status bk_attn_layer_step(bk_cache *c, int32_t layer, int32_t seq, int32_t pos, const float *qfull_dev,
                             const float *kraw_dev, const float *vraw_dev, const float *q_norm_w_dev,
                             const float *k_norm_w_dev, float eps, float *out_dev) {
    if (!valid_layer_seq(c, layer, seq)) return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, "bk_attn_layer_step: bad layer/seq");
    bk_ctx *ctx = c->ctx;
    if (!qfull_dev || !kraw_dev || !vraw_dev || !q_norm_w_dev || !k_norm_w_dev || !out_dev)
        return fail(ctx, BK_ERR_INVALID, "bk_attn_layer_step: null argument");
    if (pos >= c->cfg.n_ctx)
        return fail(ctx, BK_ERR_RANGE,
                    "bk_attn_layer_step: position " + std::to_string(pos) + " exceeds context " +
                        std::to_string(c->cfg.n_ctx) + " (raise BONSAI_CTX)");
    if (pos != c->n_pos[c->slab(layer, seq)])
        return fail(ctx, BK_ERR_INVALID,
                    "bk_attn_layer_step: pos " + std::to_string(pos) + " is not the next row (" +
                        std::to_string(c->n_pos[c->slab(layer, seq)]) + ")");
    if (pos >= c->rope->n_pos) return fail(ctx, BK_ERR_RANGE, "bk_attn_layer_step: position beyond the rope table");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    const int32_t np = pos + 1, qp = pos;
    const int n_head = c->cfg.n_head, n_kv = c->cfg.n_kv;
    DecodeArgs a;
    fill_decode_args(c, layer, 0, &a);
    if (decode_entry_uses_mma(ctx, a, np)) {
        // One launch: q is read in place from the interleaved projection output and normed in the
        // kernel's q set-up, the new k row is normed in the fused append, the gate is applied where
        // the output is written.
        a.q = qfull_dev;
        a.q_stride = 2 * kHd;
        a.q_norm_w = q_norm_w_dev;
        a.k_norm_w = k_norm_w_dev;
        a.eps = eps;
        a.gate = qfull_dev + kHd;
        a.gate_stride = 2 * kHd;
        a.out = out_dev;
        a.new_k = kraw_dev;
        a.new_v = vraw_dev;
        const DecodeEntry e{0, seq, np, qp};
        st = launch_decode_group(ctx, a, &e, 1, true, kMaxItems);
        if (st == BK_OK) c->n_pos[c->slab(layer, seq)] = np;
        return st;
    }
    // Other caches: norm q and k in one small launch, then append and decode as usual; the gate is
    // applied by the decode kernel's output stage.
    const size_t need = (size_t)(n_head + n_kv) * kHd;
    if (ctx->d_layer_floats < need) {
        BK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->d_layer) cudaFree(ctx->d_layer);
        ctx->d_layer = nullptr;
        ctx->d_layer_floats = 0;
        BK_CUDA(ctx, cudaMalloc((void **)&ctx->d_layer, need * sizeof(float)));
        ctx->d_layer_floats = need;
    }
    float *qn = ctx->d_layer, *kn = ctx->d_layer + (size_t)n_head * kHd;
    const NormSeg sq{qfull_dev, (size_t)2 * kHd, q_norm_w_dev, qn, n_head};
    const NormSeg sk{kraw_dev, (size_t)kHd, k_norm_w_dev, kn, n_kv};
    if ((st = launch_rms_norm_rows(ctx, sq, sk, kHd, eps)) != BK_OK) return st;
    if ((st = bk_append(c, layer, seq, pos, 1, kn, vraw_dev)) != BK_OK) return st;
    return decode_impl(c, layer, 1, &seq, &np, &qp, qn, out_dev, 0, "bk_attn_layer_step", qfull_dev + kHd, 2 * kHd);
}

bk_status bk_attn_layer_step_host(bk_cache *c, int32_t layer, int32_t seq, int32_t pos, const float *qfull_host,
                                  const float *kraw_host, const float *vraw_host, const float *q_norm_w_host,
                                  const float *k_norm_w_host, float eps, float *out_host) {
    if (!valid_layer_seq(c, layer, seq))
        return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, "bk_attn_layer_step_host: bad layer/seq");
    bk_ctx *ctx = c->ctx;
    if (!qfull_host || !kraw_host || !vraw_host || !q_norm_w_host || !k_norm_w_host || !out_host)
        return fail(ctx, BK_ERR_INVALID, "bk_attn_layer_step_host: null argument");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    const size_t qfb = (size_t)c->cfg.n_head * 2 * kHd * sizeof(float), kb = (size_t)c->cfg.n_kv * kHd * sizeof(float);
    const size_t wb = kHd * sizeof(float), ob = (size_t)c->cfg.n_head * kHd * sizeof(float);
    const size_t in_bytes = qfb + 2 * kb + 2 * wb;
    if ((st = ensure_stage(ctx, in_bytes + ob)) != BK_OK) return st;
    char *h = (char *)ctx->h_stage, *d = (char *)ctx->d_stage;
    memcpy(h, qfull_host, qfb);
    memcpy(h + qfb, kraw_host, kb);
    memcpy(h + qfb + kb, vraw_host, kb);
    memcpy(h + qfb + 2 * kb, q_norm_w_host, wb);
    memcpy(h + qfb + 2 * kb + wb, k_norm_w_host, wb);
    BK_CUDA(ctx, cudaMemcpyAsync(d, h, in_bytes, cudaMemcpyHostToDevice, ctx->stream));
    float *h_out = (float *)(h + in_bytes);  // written by the kernel directly (see bk_attn_step_host)
    st = bk_attn_layer_step(c, layer, seq, pos, (const float *)d, (const float *)(d + qfb), (const float *)(d + qfb + kb),
                            (const float *)(d + qfb + 2 * kb), (const float *)(d + qfb + 2 * kb + wb), eps, h_out);
    if (st != BK_OK) return st;
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    memcpy(out_host, h_out, ob);
    return BK_OK;
}

bk_status bk_rms_norm_rows(bk_ctx *ctx, int32_t n_rows, int32_t row_len, const float *x_host, const float *w_host,
                           float eps, float *out_host) {
    if (!ctx) return fail(nullptr, BK_ERR_INVALID, "bk_rms_norm_rows: ctx is null");
    if (n_rows < 0 || row_len < 1 || !x_host || !w_host || !out_host)
        return fail(ctx, BK_ERR_INVALID, "bk_rms_norm_rows: bad argument");
    if (row_len > 1024) return fail(ctx, BK_ERR_UNSUPPORTED, "bk_rms_norm_rows: row_len above 1024");
    if (n_rows == 0) return BK_OK;
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    const size_t xb = (size_t)n_rows * row_len * sizeof(float), wb = (size_t)row_len * sizeof(float);
    if ((st = ensure_stage(ctx, 2 * xb + wb)) != BK_OK) return st;
    char *h = (char *)ctx->h_stage, *d = (char *)ctx->d_stage;
    memcpy(h, x_host, xb);
    memcpy(h + xb, w_host, wb);
    BK_CUDA(ctx, cudaMemcpyAsync(d, h, xb + wb, cudaMemcpyHostToDevice, ctx->stream));
    const NormSeg s0{(const float *)d, (size_t)row_len, (const float *)(d + xb), (float *)(d + xb + wb), n_rows};
    const NormSeg s1{nullptr, 0, nullptr, nullptr, 0};
    if ((st = launch_rms_norm_rows(ctx, s0, s1, row_len, eps)) != BK_OK) return st;
    BK_CUDA(ctx, cudaMemcpyAsync(h + xb + wb, d + xb + wb, xb, cudaMemcpyDeviceToHost, ctx->stream));
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    memcpy(out_host, h + xb + wb, xb);
    return BK_OK;
}

/* ---- PQ2_0 ternary matvec -------------------------------------------------- */

size_t bk_pq2_row_bytes(int64_t ne0) { return ne0 > 0 ? pq2_row_bytes(ne0) : 0; }

static bk_status pq2_check(bk_ctx *ctx, const char *who, const void *payload, size_t payload_bytes, int64_t ne0, int64_t base_row,
                           int64_t n_rows, int32_t n_tok, const void *x, const void *y) {
    if (!ctx) return fail(nullptr, BK_ERR_INVALID, std::string(who) + ": ctx is null");
    if (ne0 < 1 || ne0 > (1 << 24) || base_row < 0 || n_rows < 0 || n_tok < 0)
        return fail(ctx, BK_ERR_INVALID, std::string(who) + ": bad sizes");
    if (n_rows > 0 && n_tok > 0 && (!payload || !x || !y)) return fail(ctx, BK_ERR_INVALID, std::string(who) + ": null argument");
    if ((uintptr_t)payload % 2 != 0) return fail(ctx, BK_ERR_INVALID, std::string(who) + ": payload must be 2-byte aligned");
    const size_t rb = pq2_row_bytes(ne0);
    // the reference's range check (src/kernels.rs:288-299): the rows asked for must lie inside the payload
    const unsigned __int128 need = (unsigned __int128)(base_row + n_rows) * rb;
    if (need > payload_bytes)
        return fail(ctx, BK_ERR_RANGE, std::string(who) + ": rows " + std::to_string(base_row) + ".." + std::to_string(base_row + n_rows) +
                                           " need " + std::to_string((unsigned long long)need) + " bytes, payload is " +
                                           std::to_string(payload_bytes));
    if (n_rows > (int64_t)INT32_MAX - 16) return fail(ctx, BK_ERR_UNSUPPORTED, std::string(who) + ": too many rows for one call");
    return BK_OK;
}

// y of range s: [n_tok][n_rows_s]; two tokens share one pass over the weights
static bk_status pq2_run_multi(bk_ctx *ctx, int n_seg, const bk_pq2_seg *segs, int64_t ne0, const float *x_dev, int32_t n_tok) {
    const size_t rb = pq2_row_bytes(ne0);
    for (int t0 = 0; t0 < n_tok; t0 += 2) {
        const uint8_t *rows[4];
        float *y[4];
        int n_rows[4];
        for (int i = 0; i < n_seg; i++) {
            rows[i] = (const uint8_t *)segs[i].payload_dev + (size_t)segs[i].base_row * rb;
            n_rows[i] = (int)segs[i].n_rows;
            y[i] = segs[i].y_dev + (size_t)t0 * segs[i].n_rows;
        }
        bk_status st = launch_pq2_matvec(ctx, n_seg, rows, n_rows, y, (int)ne0, x_dev + (size_t)t0 * ne0, std::min(2, n_tok - t0));
        if (st != BK_OK) return st;
    }
    return BK_OK;
}

static bk_status pq2_run(bk_ctx *ctx, const uint8_t *payload, int64_t ne0, int64_t base_row, int64_t n_rows, const float *x_dev,
                         int32_t n_tok, float *y_dev) {
    const bk_pq2_seg seg{payload, 0, base_row, n_rows, y_dev};
    return pq2_run_multi(ctx, 1, &seg, ne0, x_dev, n_tok);
}

bk_status bk_pq2_matvec_multi(bk_ctx *ctx, int32_t n_seg, const bk_pq2_seg *segs, int64_t ne0, const float *x_dev, int32_t n_tok) {
    if (!ctx) return fail(nullptr, BK_ERR_INVALID, "bk_pq2_matvec_multi: ctx is null");
    if (n_seg < 0 || n_seg > 4 || (n_seg > 0 && !segs)) return fail(ctx, BK_ERR_INVALID, "bk_pq2_matvec_multi: 0..4 row ranges");
    for (int i = 0; i < n_seg; i++) {
        bk_status st = pq2_check(ctx, "bk_pq2_matvec_multi", segs[i].payload_dev, segs[i].payload_bytes, ne0, segs[i].base_row,
                                 segs[i].n_rows, n_tok, x_dev, segs[i].y_dev);
        if (st != BK_OK) return st;
    }
    if (n_seg == 0 || n_tok == 0) return BK_OK;
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    return pq2_run_multi(ctx, n_seg, segs, ne0, x_dev, n_tok);
}

bk_status bk_pq2_matvec(bk_ctx *ctx, const void *payload_dev, size_t payload_bytes, int64_t ne0, int64_t base_row, int64_t n_rows,
                        const float *x_dev, int32_t n_tok, float *y_dev) {
    bk_status st = pq2_check(ctx, "bk_pq2_matvec", payload_dev, payload_bytes, ne0, base_row, n_rows, n_tok, x_dev, y_dev);
    if (st != BK_OK) return st;
    if (n_rows == 0 || n_tok == 0) return BK_OK;
    if ((st = bind(ctx)) != BK_OK) return st;
    return pq2_run(ctx, (const uint8_t *)payload_dev, ne0, base_row, n_rows, x_dev, n_tok, y_dev);
}

bk_status bk_pq2_matvec_host(bk_ctx *ctx, const void *payload_dev, size_t payload_bytes, int64_t ne0, int64_t base_row,
                             int64_t n_rows, const float *x_host, int32_t n_tok, float *y_host) {
    bk_status st = pq2_check(ctx, "bk_pq2_matvec_host", payload_dev, payload_bytes, ne0, base_row, n_rows, n_tok, x_host, y_host);
    if (st != BK_OK) return st;
    if (n_rows == 0 || n_tok == 0) return BK_OK;
    if ((st = bind(ctx)) != BK_OK) return st;
    const size_t xb = (size_t)n_tok * ne0 * sizeof(float), yb = (size_t)n_tok * n_rows * sizeof(float);
    const size_t xpad = (xb + 255) / 256 * 256;
    if ((st = ensure_stage(ctx, xpad + yb)) != BK_OK) return st;
    char *h = (char *)ctx->h_stage, *d = (char *)ctx->d_stage;
    memcpy(h, x_host, xb);
    BK_CUDA(ctx, cudaMemcpyAsync(d, h, xb, cudaMemcpyHostToDevice, ctx->stream));
    // y is written straight into the pinned staging buffer by the kernel
    if ((st = pq2_run(ctx, (const uint8_t *)payload_dev, ne0, base_row, n_rows, (const float *)d, n_tok, (float *)(h + xpad))) != BK_OK)
        return st;
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    memcpy(y_host, h + xpad, yb);
    return BK_OK;
}

bk_status bk_attn_oneshot_host(bk_ctx *ctx, const float *q_host, const float *k_host, const float *v_host,
                               int32_t n_pos, int32_t nheads, int32_t kvheads, int32_t hd, float *out_host) {
    if (!ctx) return fail(nullptr, BK_ERR_INVALID, "bk_attn_oneshot_host: ctx is null");
    if (!q_host || !k_host || !v_host || !out_host || n_pos < 1 || nheads < 1 || kvheads < 1 || nheads % kvheads != 0)
        return fail(ctx, BK_ERR_INVALID, "attn_step: bad q/k/v sizes");
    if (hd != kHd) return fail(ctx, BK_ERR_UNSUPPORTED, "attn_step: head_dim must be 256");
    if (kvheads > 8) return fail(ctx, BK_ERR_UNSUPPORTED, "attn_step: at most 8 kv heads");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    const size_t qb = (size_t)nheads * hd * 4, kvb = (size_t)n_pos * kvheads * hd * 4;
    if ((st = ensure_stage(ctx, 2 * qb + 2 * kvb)) != BK_OK) return st;
    char *h = (char *)ctx->h_stage, *d = (char *)ctx->d_stage;
    memcpy(h, q_host, qb);
    memcpy(h + qb, k_host, kvb);
    memcpy(h + qb + kvb, v_host, kvb);
    BK_CUDA(ctx, cudaMemcpyAsync(d, h, qb + 2 * kvb, cudaMemcpyHostToDevice, ctx->stream));
    DecodeArgs a{};
    a.k_rows = (const uint8_t *)(d + qb);
    a.v_rows = (const uint8_t *)(d + qb + kvb);
    a.seq_stride_rows = 0;
    a.q = (const float *)d;
    a.out = (float *)(d + qb + 2 * kvb);
    a.n_head = nheads;
    a.n_kv = kvheads;
    a.k_kind = a.v_kind = ROW_F32;
    a.k_row_bytes = a.v_row_bytes = (size_t)hd * 4;
    a.partials = ctx->d_partials;
    a.counters = ctx->d_counters;
    a.no_rope = 1;
    DecodeMeta m{};
    m.n_seqs = 1;
    m.n_pos[0] = n_pos;
    int64_t L = std::max<int64_t>(64, ((int64_t)n_pos * kvheads / (ctx->n_sms * 4) + 63) / 64 * 64);
    while ((int64_t)kvheads * ((n_pos + L - 1) / L) > kMaxItems) L *= 2;
    m.chunk_len = (int)L;
    m.n_items = kvheads * (int)((n_pos + L - 1) / L);
    m.item_start[1] = m.n_items;
    if ((st = launch_decode(ctx, a, m)) != BK_OK) return st;
    BK_CUDA(ctx, cudaMemcpyAsync(h + qb + 2 * kvb, a.out, qb, cudaMemcpyDeviceToHost, ctx->stream));
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    memcpy(out_host, h + qb + 2 * kvb, qb);
    return BK_OK;
}

/* ---- kvquant entry points -------------------------------------------------- */

size_t bk_kvq_packed_len(int32_t hd, int32_t bits) {
    if (hd < 1 || bits < 1 || bits > 8) return 0;
    const size_t padded = ((size_t)hd + 1) / 2 * 2;
    return (padded * bits + 7) / 8;
}

bk_status bk_kvq_codebook(int32_t hd, int32_t bits, float *out) {
    if (!out || hd < 1 || bits < 1 || bits > 8) return fail(nullptr, BK_ERR_INVALID, "bk_kvq_codebook: bad argument");
    host_codebook(hd, bits, out);
    return BK_OK;
}

bk_status bk_kvq_threshold_cells(int32_t bits, uint32_t *out) {
    if (!out || bits < 1 || bits > 4) return fail(nullptr, BK_ERR_INVALID, "bk_kvq_threshold_cells: bits must be 1..4");
    float book[256];
    host_codebook(kHd, bits, book);
    static_assert(sizeof(uint2) == 2 * sizeof(uint32_t), "cell layout");
    if (!build_threshold_cells(book, 1 << bits, reinterpret_cast<uint2 *>(out)))
        return fail(nullptr, BK_ERR_UNSUPPORTED, "codebook thresholds do not fit the cell table");
    return BK_OK;
}

bk_status bk_kvq_givens(int32_t hd, float *out) {
    if (!out || hd < 1) return fail(nullptr, BK_ERR_INVALID, "bk_kvq_givens: bad argument");
    host_givens(hd, out);
    return BK_OK;
}

// Shared shape of the host-in/host-out parity calls: stage inputs, run, stage outputs back.
struct HostIo {
    bk_ctx *ctx;
    char *h, *d;
    size_t used = 0;
    size_t take(size_t bytes) {
        const size_t off = used;
        used += (bytes + 255) & ~(size_t)255;
        return off;
    }
};

static bk_status kvq_check(bk_ctx *ctx, int hd, int bits, int n_vec, bool need_bits, const char *who) {
    if (!ctx) return fail(nullptr, BK_ERR_INVALID, std::string(who) + ": ctx is null");
    if (hd != kHd) return fail(ctx, BK_ERR_UNSUPPORTED, std::string(who) + ": head_dim must be 256");
    if (need_bits && (bits < 1 || bits > 8)) return fail(ctx, BK_ERR_INVALID, std::string(who) + ": bits must be 1..8");
    if (n_vec < 0) return fail(ctx, BK_ERR_INVALID, std::string(who) + ": negative count");
    return bind(ctx);
}

bk_status bk_kvq_quantize(bk_ctx *ctx, int32_t hd, int32_t bits, int32_t n_vec, const float *x, uint8_t *packed,
                          float *norms) {
    bk_status st = kvq_check(ctx, hd, bits, n_vec, true, "bk_kvq_quantize");
    if (st != BK_OK || n_vec == 0) return st;
    if (!x || !packed || !norms) return fail(ctx, BK_ERR_INVALID, "bk_kvq_quantize: null argument");
    const size_t xb = (size_t)n_vec * hd * 4, pb = (size_t)n_vec * 32 * bits, nb = (size_t)n_vec * 4;
    HostIo io{ctx};
    const size_t ox = io.take(xb), op = io.take(pb), on = io.take(nb);
    if ((st = ensure_stage(ctx, io.used)) != BK_OK) return st;
    char *h = (char *)ctx->h_stage, *d = (char *)ctx->d_stage;
    memcpy(h + ox, x, xb);
    BK_CUDA(ctx, cudaMemcpyAsync(d + ox, h + ox, xb, cudaMemcpyHostToDevice, ctx->stream));
    if ((st = launch_quantize(ctx, bits, n_vec, (const float *)(d + ox), (uint8_t *)(d + op), (float *)(d + on))) != BK_OK)
        return st;
    BK_CUDA(ctx, cudaMemcpyAsync(h + op, d + op, pb, cudaMemcpyDeviceToHost, ctx->stream));
    BK_CUDA(ctx, cudaMemcpyAsync(h + on, d + on, nb, cudaMemcpyDeviceToHost, ctx->stream));
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    memcpy(packed, h + op, pb);
    memcpy(norms, h + on, nb);
    return BK_OK;
}

bk_status bk_kvq_dequantize(bk_ctx *ctx, int32_t hd, int32_t bits, int32_t n_vec, const uint8_t *packed,
                            const float *norms, float *out) {
    bk_status st = kvq_check(ctx, hd, bits, n_vec, true, "bk_kvq_dequantize");
    if (st != BK_OK || n_vec == 0) return st;
    if (!packed || !norms || !out) return fail(ctx, BK_ERR_INVALID, "bk_kvq_dequantize: null argument");
    const size_t xb = (size_t)n_vec * hd * 4, pb = (size_t)n_vec * 32 * bits, nb = (size_t)n_vec * 4;
    HostIo io{ctx};
    const size_t op = io.take(pb), on = io.take(nb), ox = io.take(xb);
    if ((st = ensure_stage(ctx, io.used)) != BK_OK) return st;
    char *h = (char *)ctx->h_stage, *d = (char *)ctx->d_stage;
    memcpy(h + op, packed, pb);
    memcpy(h + on, norms, nb);
    BK_CUDA(ctx, cudaMemcpyAsync(d + op, h + op, ox - op, cudaMemcpyHostToDevice, ctx->stream));
    if ((st = launch_dequantize(ctx, bits, n_vec, (const uint8_t *)(d + op), (const float *)(d + on), (float *)(d + ox))) != BK_OK)
        return st;
    BK_CUDA(ctx, cudaMemcpyAsync(h + ox, d + ox, xb, cudaMemcpyDeviceToHost, ctx->stream));
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    memcpy(out, h + ox, xb);
    return BK_OK;
}

bk_status bk_kvq_rotate(bk_ctx *ctx, int32_t hd, int32_t n_vec, int32_t inverse, const float *x, float *out) {
    bk_status st = kvq_check(ctx, hd, 0, n_vec, false, "bk_kvq_rotate");
    if (st != BK_OK || n_vec == 0) return st;
    if (!x || !out) return fail(ctx, BK_ERR_INVALID, "bk_kvq_rotate: null argument");
    const size_t xb = (size_t)n_vec * hd * 4;
    HostIo io{ctx};
    const size_t ox = io.take(xb), oo = io.take(xb);
    if ((st = ensure_stage(ctx, io.used)) != BK_OK) return st;
    char *h = (char *)ctx->h_stage, *d = (char *)ctx->d_stage;
    memcpy(h + ox, x, xb);
    BK_CUDA(ctx, cudaMemcpyAsync(d + ox, h + ox, xb, cudaMemcpyHostToDevice, ctx->stream));
    if ((st = launch_rotate(ctx, n_vec, inverse, (const float *)(d + ox), (float *)(d + oo))) != BK_OK) return st;
    BK_CUDA(ctx, cudaMemcpyAsync(h + oo, d + oo, xb, cudaMemcpyDeviceToHost, ctx->stream));
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    memcpy(out, h + oo, xb);
    return BK_OK;
}

bk_status bk_kvq_dot_rotated(bk_ctx *ctx, int32_t hd, int32_t bits, int32_t n_vec, const float *q_rot,
                             const uint8_t *packed, const float *norms, float *out) {
    bk_status st = kvq_check(ctx, hd, bits, n_vec, true, "bk_kvq_dot_rotated");
    if (st != BK_OK || n_vec == 0) return st;
    if (!q_rot || !packed || !norms || !out) return fail(ctx, BK_ERR_INVALID, "bk_kvq_dot_rotated: null argument");
    const size_t xb = (size_t)n_vec * hd * 4, pb = (size_t)n_vec * 32 * bits, nb = (size_t)n_vec * 4;
    HostIo io{ctx};
    const size_t oq = io.take(xb), op = io.take(pb), on = io.take(nb), oo = io.take(nb);
    if ((st = ensure_stage(ctx, io.used)) != BK_OK) return st;
    char *h = (char *)ctx->h_stage, *d = (char *)ctx->d_stage;
    memcpy(h + oq, q_rot, xb);
    memcpy(h + op, packed, pb);
    memcpy(h + on, norms, nb);
    BK_CUDA(ctx, cudaMemcpyAsync(d + oq, h + oq, oo - oq, cudaMemcpyHostToDevice, ctx->stream));
    if ((st = launch_dot_rotated(ctx, bits, n_vec, (const float *)(d + oq), (const uint8_t *)(d + op),
                                 (const float *)(d + on), (float *)(d + oo))) != BK_OK)
        return st;
    BK_CUDA(ctx, cudaMemcpyAsync(h + oo, d + oo, nb, cudaMemcpyDeviceToHost, ctx->stream));
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    memcpy(out, h + oo, nb);
    return BK_OK;
}

bk_status bk_rope_imrope(bk_ctx *ctx, int32_t n_heads, int32_t hd, float *heads, int64_t p_t, int64_t p_h,
                         int64_t p_w, int64_t p_e, int32_t n_dims, const int32_t sections[4], float freq_base) {
    if (!ctx) return fail(nullptr, BK_ERR_INVALID, "bk_rope_imrope: ctx is null");
    if (!heads || !sections || n_heads < 0 || hd < 1 || n_dims < 0 || n_dims > hd || (n_dims & 1) || n_dims > 512)
        return fail(ctx, BK_ERR_INVALID, "bk_rope_imrope: bad argument");
    if (n_heads == 0 || n_dims == 0) return BK_OK;
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    const int half = n_dims / 2;
    const size_t hb = (size_t)n_heads * hd * 4, rb = (size_t)4 * half * sizeof(float2), bb = (size_t)half * 4;
    HostIo io{ctx};
    const size_t oh = io.take(hb), orow = io.take(rb), ob = io.take(bb);
    if ((st = ensure_stage(ctx, io.used)) != BK_OK) return st;
    char *h = (char *)ctx->h_stage, *d = (char *)ctx->d_stage;
    memcpy(h + oh, heads, hb);
    const int64_t ids[4] = {p_t, p_h, p_w, p_e};
    for (int b = 0; b < 4; b++) host_rope_rows(ids[b], 1, n_dims, freq_base, (float2 *)(h + orow) + (size_t)b * half);
    for (int j = 0; j < half; j++) ((int *)(h + ob))[j] = host_rope_band(j, sections);
    BK_CUDA(ctx, cudaMemcpyAsync(d, h, io.used, cudaMemcpyHostToDevice, ctx->stream));
    if ((st = launch_rope(ctx, n_heads, hd, (float *)(d + oh), (const float2 *)(d + orow), n_dims, (const int *)(d + ob))) != BK_OK)
        return st;
    BK_CUDA(ctx, cudaMemcpyAsync(h + oh, d + oh, hb, cudaMemcpyDeviceToHost, ctx->stream));
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    memcpy(heads, h + oh, hb);
    return BK_OK;
}

bk_status bk_f32_to_half(bk_ctx *ctx, size_t n, const float *in, uint16_t *out) {
    if (!ctx) return fail(nullptr, BK_ERR_INVALID, "bk_f32_to_half: ctx is null");
    if (n == 0) return BK_OK;
    if (!in || !out) return fail(ctx, BK_ERR_INVALID, "bk_f32_to_half: null argument");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    HostIo io{ctx};
    const size_t oi = io.take(n * 4), oo = io.take(n * 2);
    if ((st = ensure_stage(ctx, io.used)) != BK_OK) return st;
    char *h = (char *)ctx->h_stage, *d = (char *)ctx->d_stage;
    memcpy(h + oi, in, n * 4);
    BK_CUDA(ctx, cudaMemcpyAsync(d + oi, h + oi, n * 4, cudaMemcpyHostToDevice, ctx->stream));
    if ((st = launch_f32_to_half(ctx, n, (const float *)(d + oi), (uint16_t *)(d + oo))) != BK_OK) return st;
    BK_CUDA(ctx, cudaMemcpyAsync(h + oo, d + oo, n * 2, cudaMemcpyDeviceToHost, ctx->stream));
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    memcpy(out, h + oo, n * 2);
    return BK_OK;
}

bk_status bk_half_to_f32(bk_ctx *ctx, size_t n, const uint16_t *in, float *out) {
    if (!ctx) return fail(nullptr, BK_ERR_INVALID, "bk_half_to_f32: ctx is null");
    if (n == 0) return BK_OK;
    if (!in || !out) return fail(ctx, BK_ERR_INVALID, "bk_half_to_f32: null argument");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    HostIo io{ctx};
    const size_t oi = io.take(n * 2), oo = io.take(n * 4);
    if ((st = ensure_stage(ctx, io.used)) != BK_OK) return st;
    char *h = (char *)ctx->h_stage, *d = (char *)ctx->d_stage;
    memcpy(h + oi, in, n * 2);
    BK_CUDA(ctx, cudaMemcpyAsync(d + oi, h + oi, n * 2, cudaMemcpyHostToDevice, ctx->stream));
    if ((st = launch_half_to_f32(ctx, n, (const uint16_t *)(d + oi), (float *)(d + oo))) != BK_OK) return st;
    BK_CUDA(ctx, cudaMemcpyAsync(h + oo, d + oo, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    memcpy(out, h + oo, n * 4);
    return BK_OK;
}

/* ---- memory and timing helpers ----------------------------------------------- */

bk_status bk_dev_alloc(bk_ctx *ctx, size_t bytes, void **out) {
    if (!ctx || !out) return fail(ctx, BK_ERR_INVALID, "bk_dev_alloc: null argument");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    *out = nullptr;
    cudaError_t e = cudaMalloc(out, bytes ? bytes : 1);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return cuda_fail(ctx, e, "cudaMalloc");
    }
    return BK_OK;
}

bk_status bk_dev_free(bk_ctx *ctx, void *dev) {
    if (!ctx) return fail(nullptr, BK_ERR_INVALID, "bk_dev_free: ctx is null");
    if (!dev) return BK_OK;
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    BK_CUDA(ctx, cudaFree(dev));
    return BK_OK;
}

bk_status bk_host_alloc_pinned(bk_ctx *ctx, size_t bytes, void **out) {
    if (!ctx || !out) return fail(ctx, BK_ERR_INVALID, "bk_host_alloc_pinned: null argument");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    *out = nullptr;
    BK_CUDA(ctx, cudaMallocHost(out, bytes ? bytes : 1));
    return BK_OK;
}

bk_status bk_host_free_pinned(bk_ctx *ctx, void *host) {
    if (!ctx) return fail(nullptr, BK_ERR_INVALID, "bk_host_free_pinned: ctx is null");
    if (!host) return BK_OK;
    {
        const bk_status st_sync = sync_and_check(ctx);
        if (st_sync != BK_OK) return st_sync;
    }
    BK_CUDA(ctx, cudaFreeHost(host));
    return BK_OK;
}

bk_status bk_memcpy_h2d(bk_ctx *ctx, void *dst, const void *src, size_t bytes) {
    if (!ctx || (bytes && (!dst || !src))) return fail(ctx, BK_ERR_INVALID, "bk_memcpy_h2d: null argument");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    BK_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return BK_OK;
}

bk_status bk_memcpy_d2h(bk_ctx *ctx, void *dst, const void *src, size_t bytes) {
    if (!ctx || (bytes && (!dst || !src))) return fail(ctx, BK_ERR_INVALID, "bk_memcpy_d2h: null argument");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    BK_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return BK_OK;
}

bk_status bk_memset_dev(bk_ctx *ctx, void *dst, int value, size_t bytes) {
    if (!ctx || (bytes && !dst)) return fail(ctx, BK_ERR_INVALID, "bk_memset_dev: null argument");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    BK_CUDA(ctx, cudaMemsetAsync(dst, value, bytes, ctx->stream));
    return BK_OK;
}

bk_status bk_event_create(bk_ctx *ctx, bk_event **out) {
    if (!ctx || !out) return fail(ctx, BK_ERR_INVALID, "bk_event_create: null argument");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    bk_event *ev = new (std::nothrow) bk_event();
    if (!ev) return fail(ctx, BK_ERR_OOM, "bk_event_create: host allocation failed");
    ev->device = ctx->device;
    cudaError_t e = cudaEventCreate(&ev->ev);
    if (e != cudaSuccess) {
        delete ev;
        return cuda_fail(ctx, e, "cudaEventCreate");
    }
    *out = ev;
    return BK_OK;
}

void bk_event_destroy(bk_event *ev) {
    if (!ev) return;
    cudaSetDevice(ev->device);
    if (ev->ev) cudaEventDestroy(ev->ev);
    delete ev;
}

bk_status bk_event_record(bk_ctx *ctx, bk_event *ev) {
    if (!ctx || !ev) return fail(ctx, BK_ERR_INVALID, "bk_event_record: null argument");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    BK_CUDA(ctx, cudaEventRecord(ev->ev, ctx->stream));
    return BK_OK;
}

bk_status bk_event_elapsed_ms(bk_ctx *ctx, bk_event *start, bk_event *stop, float *ms) {
    if (!ctx || !start || !stop || !ms) return fail(ctx, BK_ERR_INVALID, "bk_event_elapsed_ms: null argument");
    bk_status st = bind(ctx);
    if (st != BK_OK) return st;
    BK_CUDA(ctx, cudaEventSynchronize(stop->ev));
    BK_CUDA(ctx, cudaEventElapsedTime(ms, start->ev, stop->ev));
    // a time between two events is worthless if a kernel between them gave up a wait: report it here too
    if (ctx->h_err && *ctx->h_err) return sync_and_check(ctx);
    return BK_OK;
}

}  // extern "C"
