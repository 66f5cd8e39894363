// bk_decode_attn_noalloc: decode attention whose split-K scratch is a fixed array inside the
// library instead of memory obtained from the CUDA allocator.
//
// Who needs it: hosts that drive the decode step from a place where allocating is off limits.
// Two real cases for this library are (1) a serving loop that has handed its whole HBM budget to
// the KV caches at start-up and treats any later cudaMalloc as a bug, because cudaMalloc
// synchronises the device (stalling every other stream for the duration) and may fail when the
// heap is fragmented, and (2) code that runs the step on a thread or in a callback where the
// CUDA allocator must not be entered at all.  Such a caller creates its context and caches once,
// early, and afterwards wants a decode call that is guaranteed to touch no allocator: not
// cudaMalloc/cudaFree, not the host heap, not a tensor library.
//
// What it costs: every GPU that loads this library reserves kStaticItems partial results
// (about 4.3 MB) plus 1024 counters for as long as the process lives, whether or not the entry
// point is ever called.  One call handles at most 64 sequences (more are rejected, not split); the
// work of a call is cut into at most kStaticItems (sequence, kv head, chunk) items, with coarser
// chunks than bk_decode_attn would use if need be, so the two agree within the parity tolerance
// rather than bit for bit.
//
// All calls on a device share the one array.  It keeps whatever the previous call left in it;
// the only part that must start from zero, the arrival counters, is cleared at the start of
// every call.  Two calls whose kernels overlap on the GPU (different contexts or streams, or
// mixed with nothing else - the normal entry points use their own per-context scratch) race on
// the array and give wrong results: serialise them.
//
// The first call on each device looks up the array's device address (cudaGetSymbolAddress), once,
// under std::call_once.  Make that first call during set-up, outside any stream capture.  A call
// that succeeds enters no allocator; a failing call builds its message as a std::string.
#include <mutex>

#include "bk_internal.h"

namespace bk {

namespace {

constexpr int kStaticItems = 512;     // work items one call may create
constexpr int kStaticCounters = kCtrTotal; // three counters per (sequence-in-call, kv head) pair, up to 512 pairs
constexpr int kStaticSeqs = kMaxSeqsPerLaunch;

// The scratch itself.  In host code these names are only handles for the runtime: the device
// address comes from cudaGetSymbolAddress below, never from taking '&' on the host.
static __device__ __align__(256) float g_static_partials[(size_t)kStaticItems * kMaxRep * kScratchStride];
static __device__ __align__(256) unsigned g_static_counters[kStaticCounters];

struct DeviceScratch {
    std::once_flag once;
    float *partials = nullptr;
    unsigned *counters = nullptr;
    cudaError_t err = cudaSuccess;
};
DeviceScratch g_scratch[64];

// Once per device, with that device current (the caller has bound it).
bk_status static_scratch(bk_ctx *ctx, DeviceScratch **out) {
    if (ctx->device < 0 || ctx->device >= 64) return fail(ctx, BK_ERR_UNSUPPORTED, "bk_decode_attn_noalloc: device index above 63");
    DeviceScratch &s = g_scratch[ctx->device];
    std::call_once(s.once, [&s]() {
        s.err = cudaGetSymbolAddress((void **)&s.partials, g_static_partials);
        if (s.err == cudaSuccess) s.err = cudaGetSymbolAddress((void **)&s.counters, g_static_counters);
    });
    if (s.err != cudaSuccess) return cuda_fail(ctx, s.err, "cudaGetSymbolAddress(static split-K scratch)");
    *out = &s;
    return BK_OK;
}

}  // namespace

}  // namespace bk

using namespace bk;

extern "C" bk_status bk_decode_attn_noalloc(bk_cache *c, int32_t layer, int32_t n_seqs, const int32_t *seq_ids,
                                            const int32_t *n_pos, const int32_t *q_pos, const float *q_dev,
                                            float *out_dev) {
    const char *who = "bk_decode_attn_noalloc";
    if (!c || layer < 0 || layer >= c->cfg.n_layers) return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, "bk_decode_attn_noalloc: bad layer");
    bk_ctx *ctx = c->ctx;
    if (n_seqs < 0) return fail(ctx, BK_ERR_INVALID, "bk_decode_attn_noalloc: negative count");
    if (n_seqs == 0) return BK_OK;
    if (n_seqs > kStaticSeqs)
        return fail(ctx, BK_ERR_INVALID, "bk_decode_attn_noalloc: at most 64 sequences per call (the fixed scratch holds no more)");
    static_assert(kStaticSeqs * 8 <= kStaticItems, "64 sequences x 8 kv heads always fit the fixed scratch");
    if (!q_dev || !out_dev) return fail(ctx, BK_ERR_INVALID, "bk_decode_attn_noalloc: null q/out");
    bk_status st = bind_device(ctx);
    if (st != BK_OK) return st;
    DeviceScratch *scr = nullptr;
    if ((st = static_scratch(ctx, &scr)) != BK_OK) return st;

    DecodeArgs a;
    fill_decode_args(c, layer, 0, &a);
    a.q = q_dev;
    a.out = out_dev;
    a.partials = scr->partials;  // device addresses obtained through cudaGetSymbolAddress
    a.counters = scr->counters;

    DecodeEntry cls[2][kStaticSeqs];  // on the stack: the call itself allocates nothing
    int n_cls[2] = {0, 0};
    const size_t out_stride = (size_t)c->cfg.n_head * kHd;
    for (int i = 0; i < n_seqs; i++) {
        DecodeEntry e;
        if ((st = check_decode_entry(c, layer, i, seq_ids, n_pos, q_pos, who, &e)) != BK_OK) return st;
        if (e.np == 0) {
            BK_CUDA(ctx, cudaMemsetAsync(out_dev + (size_t)i * out_stride, 0, out_stride * sizeof(float), ctx->stream));
            continue;
        }
        const int k = decode_entry_uses_mma(ctx, a, e.np) ? 1 : 0;
        cls[k][n_cls[k]++] = e;
    }
    // the counters must read zero when the kernel starts, whatever an earlier call left behind
    BK_CUDA(ctx, cudaMemsetAsync(scr->counters, 0, sizeof(unsigned) * kStaticCounters, ctx->stream));
    for (int k = 0; k < 2; k++)
        if (n_cls[k] > 0 && (st = launch_decode_group(ctx, a, cls[k], n_cls[k], k == 1, kStaticItems)) != BK_OK) return st;
    return BK_OK;
}
