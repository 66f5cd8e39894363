// Context split over the GPUs of one node: exchange of the per-chunk partial results through
// peer memory, fused with their log-sum-exp merge.  No counterpart in the reference (it is
// single-device); it is the exchange step of "one long sequence, context chunks per GPU".
//
// Every rank owns a mailbox (one cudaMalloc, shared with the other ranks' processes through CUDA
// IPC; ranks of one process find each other's mailbox in a process-local registry): two parities x
// world slots of n_rows x (hd + 2) eight-byte words, each a value and the sequence number of the call
// that wrote it.  The exchange runs slice by slice (exchange_slice() in bk_decode_common.cuh): whoever
// holds dims [d0, d0 + dn) of a kv head's rows, merged over the rank's own chunks, stores them as such
// words into slot [rank] of every rank's mailbox with plain 8-byte peer stores (which arrive whole, so a
// word whose second half is the call's sequence number is valid: no flags, no fences), reads the same
// words of all ranks from its own mailbox until they carry that number (bounded), and merges them.
// In the one-launch form the holders are the CTAs of the decode launch itself, each with its slice of
// the split-K combine; exchange_merge_kernel below is the stand-alone form (one CTA per kv head, all
// dims) for a rank whose decode ran as a separate launch or whose chunk is empty, and for
// bk_exchange_merge.  The transfer is 50 KB per rank and layer, so what matters is latency: no host
// synchronisation, no collective-library call, one trip over the link.
//
// The only cross-GPU dependency is between kernels on DIFFERENT GPUs; every wait gives up after
// a bounded number of polls and raises the context's error word instead of hanging.  Slots alternate
// with the parity of the sequence number, so a rank that runs ahead by one call never overwrites words
// still being merged.  No TMA and no multicast is used on peer memory.
#include <cuda/atomic>
#include <math_constants.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "bk_decode_common.cuh"
#include "bk_internal.h"

struct bk_mailbox {
    bk_ctx *ctx = nullptr;
    int world = 0, rank = 0, n_rows = 0, hd = 0;
    size_t bytes = 0;
    uint8_t *local = nullptr;           // this rank's mailbox
    uint8_t *peer[bk::kMaxWorld] = {};  // every rank's mailbox as seen from here ([rank] == local)
    bool opened[bk::kMaxWorld] = {};
    float *part = nullptr;              // staging for the local partial rows
    uint8_t **d_peer = nullptr;         // device copy of peer[]
    unsigned char handle[BK_IPC_HANDLE_BYTES] = {};  // what bk_mailbox_create handed out for `local`
};

namespace bk {

namespace {

// Mailboxes of this process: ranks that live in one process (threads, or a test that plays several
// ranks) cannot open each other's IPC handles - CUDA refuses a handle in the process that made it - so
// bk_mailbox_open_peers looks a handle up here first and uses the allocation directly.
std::mutex g_boxes_mu;
std::vector<bk_mailbox *> g_boxes;

__host__ __device__ inline size_t slot_floats(int n_rows, int hd) { return (size_t)n_rows * (hd + 2); }
// two parities x world slots of eight-byte (value, sequence number) words
__host__ __device__ inline size_t mailbox_bytes(int world, int n_rows, int hd) {
    return 2 * (size_t)world * slot_floats(n_rows, hd) * sizeof(uint2);
}

// The exchange on its own, for a rank whose rows were produced by another launch (or that has no rows: l = 0):
// one CTA per kv head sends that head's rows of `part` ([n_rows][hd + 2]: acc, m in natural-log units, l) and
// merges what arrives, in the protocol of exchange_slice().
__global__ void __launch_bounds__(256) exchange_merge_kernel(DecodeArgs a, int n_rep, const float *part) {
    __shared__ float s_M[kMaxRep], s_L[kMaxRep];
    __shared__ int s_ok;
    extern __shared__ float s_vals[];  // [n_rep][hd]
    const int kv = blockIdx.x, tid = threadIdx.x, stride = kHd + 2;
    for (int i = tid; i < n_rep * kHd; i += blockDim.x) {
        const int rr = i / kHd, d = i - rr * kHd;
        s_vals[i] = part[(size_t)(kv * n_rep + rr) * stride + d];
    }
    if (tid < n_rep) {
        s_M[tid] = part[(size_t)(kv * n_rep + tid) * stride + kHd] * 1.4426950408889634f;  // exchange_slice sends m * ln 2
        s_L[tid] = part[(size_t)(kv * n_rep + tid) * stride + kHd + 1];
    }
    __syncthreads();
    exchange_slice(a, n_rep, 0, kv, 0, kHd, s_vals, s_M, s_L, &s_ok);
}

}  // namespace

}  // namespace bk

using namespace bk;

extern "C" {

bk_status bk_mailbox_create(bk_ctx *ctx, int32_t world, int32_t rank, int32_t n_rows, int32_t hd, bk_mailbox **out,
                            void *ipc_handle_out) {
    if (!ctx || !out || !ipc_handle_out) return fail(ctx, BK_ERR_INVALID, "bk_mailbox_create: null argument");
    *out = nullptr;
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || n_rows < 1 || hd < 1)
        return fail(ctx, BK_ERR_INVALID, "bk_mailbox_create: bad world/rank/sizes (world <= 8)");
    static_assert(sizeof(cudaIpcMemHandle_t) == BK_IPC_HANDLE_BYTES, "IPC handle size");
    bk_status st = bind_device(ctx);
    if (st != BK_OK) return st;
    bk_mailbox *m = new (std::nothrow) bk_mailbox();
    if (!m) return fail(ctx, BK_ERR_OOM, "bk_mailbox_create: host allocation failed");
    m->ctx = ctx;
    m->world = world;
    m->rank = rank;
    m->n_rows = n_rows;
    m->hd = hd;
    m->bytes = mailbox_bytes(world, n_rows, hd);
    cudaError_t e = cudaMalloc(&m->local, m->bytes);
    if (e == cudaSuccess) e = cudaMemset(m->local, 0, m->bytes);  // arrival words start at 0: sequence numbers start at 1
    if (e == cudaSuccess) e = cudaMalloc(&m->part, slot_floats(n_rows, hd) * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&m->d_peer, sizeof(uint8_t *) * kMaxWorld);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t *>(ipc_handle_out), m->local);
    if (e != cudaSuccess) {
        bk_mailbox_destroy(m);
        return cuda_fail(ctx, e, "bk_mailbox_create");
    }
    m->peer[rank] = m->local;
    e = cudaMemcpy(m->d_peer, m->peer, sizeof(uint8_t *) * kMaxWorld, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        bk_mailbox_destroy(m);
        return cuda_fail(ctx, e, "bk_mailbox_create");
    }
    memcpy(m->handle, ipc_handle_out, BK_IPC_HANDLE_BYTES);
    {
        std::lock_guard<std::mutex> lock(g_boxes_mu);
        g_boxes.push_back(m);
    }
    *out = m;
    return BK_OK;
}

bk_status bk_mailbox_open_peers(bk_mailbox *m, const void *handles) {
    if (!m || !handles) return fail(m ? m->ctx : nullptr, BK_ERR_INVALID, "bk_mailbox_open_peers: null argument");
    bk_ctx *ctx = m->ctx;
    bk_status st = bind_device(ctx);
    if (st != BK_OK) return st;
    const cudaIpcMemHandle_t *h = static_cast<const cudaIpcMemHandle_t *>(handles);
    // Direct peer access to every other visible GPU, so that the mapped mailboxes are reached over
    // NVLink whatever else the process has (or has not) initialised; "already enabled" and GPUs
    // without a peer path are not errors here (the open below reports a real failure).
    {
        int n_dev = 0;
        if (cudaGetDeviceCount(&n_dev) == cudaSuccess)
            for (int d = 0; d < n_dev; d++) {
                int can = 0;
                if (d == ctx->device || cudaDeviceCanAccessPeer(&can, ctx->device, d) != cudaSuccess || !can) continue;
                cudaDeviceEnablePeerAccess(d, 0);
            }
        cudaGetLastError();
    }
    for (int r = 0; r < m->world; r++) {
        if (r == m->rank || m->opened[r] || m->peer[r]) continue;
        {   // a rank of this very process: use its allocation as it is
            std::lock_guard<std::mutex> lock(g_boxes_mu);
            for (bk_mailbox *o : g_boxes)
                if (o != m && memcmp(o->handle, &h[r], BK_IPC_HANDLE_BYTES) == 0) m->peer[r] = o->local;
        }
        if (m->peer[r]) continue;
        void *p = nullptr;
        BK_CUDA(ctx, cudaIpcOpenMemHandle(&p, h[r], cudaIpcMemLazyEnablePeerAccess));
        m->peer[r] = static_cast<uint8_t *>(p);
        m->opened[r] = true;
    }
    BK_CUDA(ctx, cudaMemcpy(m->d_peer, m->peer, sizeof(uint8_t *) * kMaxWorld, cudaMemcpyHostToDevice));
    return BK_OK;
}

void bk_mailbox_destroy(bk_mailbox *m) {
    if (!m) return;
    {
        std::lock_guard<std::mutex> lock(g_boxes_mu);
        for (size_t i = 0; i < g_boxes.size(); i++)
            if (g_boxes[i] == m) {
                g_boxes.erase(g_boxes.begin() + (long)i);
                break;
            }
    }
    cudaSetDevice(m->ctx->device);
    cudaStreamSynchronize(m->ctx->stream);
    for (int r = 0; r < m->world; r++)
        if (m->opened[r] && m->peer[r]) cudaIpcCloseMemHandle(m->peer[r]);
    if (m->local) cudaFree(m->local);
    if (m->part) cudaFree(m->part);
    if (m->d_peer) cudaFree(m->d_peer);
    delete m;
}

bk_status bk_decode_attn_split(bk_cache *c, int32_t layer, int32_t seq, int32_t n_pos, int32_t q_pos, const float *q_dev,
                               float *out_dev, bk_mailbox *m, uint32_t seqno) {
    if (!c || !m) return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, "bk_decode_attn_split: null argument");
    bk_ctx *ctx = c->ctx;
    if (m->ctx != ctx) return fail(ctx, BK_ERR_INVALID, "bk_decode_attn_split: mailbox belongs to another context");
    if (m->n_rows != c->cfg.n_head || m->hd != c->cfg.hd)
        return fail(ctx, BK_ERR_INVALID, "bk_decode_attn_split: mailbox geometry does not match the cache");
    if (seqno == 0) return fail(ctx, BK_ERR_INVALID, "bk_decode_attn_split: sequence numbers start at 1");
    for (int r = 0; r < m->world; r++)
        if (!m->peer[r]) return fail(ctx, BK_ERR_INVALID, "bk_decode_attn_split: peers are not opened");
    // A rank with rows to scan does everything in the decode launch: the CTA that finishes a kv head
    // sends, waits and merges that head's rows itself.  An empty chunk has no such CTA and goes the
    // two-step way (zero rows, then the exchange kernel); both speak the same mailbox protocol.
    if (n_pos > 0 && !getenv("BONSAI_KV_SPLIT_UNFUSED"))
        return decode_with_exchange(c, layer, seq, n_pos, q_pos, q_dev, out_dev, m->d_peer, m->world, m->rank, seqno);
    bk_status st = bk_decode_attn_partial(c, layer, 1, &seq, &n_pos, &q_pos, q_dev, m->part);
    if (st != BK_OK) return st;
    DecodeArgs xa;
    fill_decode_args(c, layer, 0, &xa);
    xa.out = out_dev;
    xa.xch_peer = m->d_peer;
    xa.xch_world = m->world;
    xa.xch_rank = m->rank;
    xa.xch_seqno = seqno;
    const int n_rep = c->cfg.n_head / c->cfg.n_kv;
    exchange_merge_kernel<<<c->cfg.n_kv, 256, (size_t)n_rep * kHd * sizeof(float), ctx->stream>>>(xa, n_rep, m->part);
    ctx->launches++;
    BK_CUDA(ctx, cudaGetLastError());
    return BK_OK;
}

bk_status bk_exchange_merge(bk_mailbox *m, int32_t n_rep, const float *part_dev, float *out_dev, uint32_t seqno) {
    if (!m || !part_dev || !out_dev) return fail(m ? m->ctx : nullptr, BK_ERR_INVALID, "bk_exchange_merge: null argument");
    bk_ctx *ctx = m->ctx;
    if (m->hd != kHd) return fail(ctx, BK_ERR_UNSUPPORTED, "bk_exchange_merge: rows of 256 values only");
    if (n_rep < 1 || n_rep > kMaxRep || m->n_rows % n_rep != 0)
        return fail(ctx, BK_ERR_INVALID, "bk_exchange_merge: the mailbox's rows are not a whole number of groups of n_rep");
    if (seqno == 0) return fail(ctx, BK_ERR_INVALID, "bk_exchange_merge: sequence numbers start at 1");
    for (int r = 0; r < m->world; r++)
        if (!m->peer[r]) return fail(ctx, BK_ERR_INVALID, "bk_exchange_merge: peers are not opened");
    bk_status st = bind_device(ctx);
    if (st != BK_OK) return st;
    DecodeArgs xa{};
    xa.n_head = m->n_rows;  // the mailbox's rows are the "heads" of this exchange, in groups of n_rep
    xa.out = out_dev;
    xa.xch_peer = m->d_peer;
    xa.xch_world = m->world;
    xa.xch_rank = m->rank;
    xa.xch_seqno = seqno;
    xa.xch_err = ctx->d_err;
    xa.xch_spin = ctx->xch_polls;
    exchange_merge_kernel<<<m->n_rows / n_rep, 256, (size_t)n_rep * kHd * sizeof(float), ctx->stream>>>(xa, n_rep, part_dev);
    ctx->launches++;
    BK_CUDA(ctx, cudaGetLastError());
    return BK_OK;
}

bk_status bk_attn_step_split(bk_cache *c, int32_t layer, int32_t seq, int32_t q_pos, const float *q_dev,
                             const float *k_dev, const float *v_dev, float *out_dev, bk_mailbox *m, uint32_t seqno) {
    if (!c || !m) return fail(c ? c->ctx : nullptr, BK_ERR_INVALID, "bk_attn_step_split: null argument");
    bk_ctx *ctx = c->ctx;
    if (layer < 0 || layer >= c->cfg.n_layers || seq < 0 || seq >= c->cfg.n_seqs)
        return fail(ctx, BK_ERR_INVALID, "bk_attn_step_split: bad layer/seq");
    const bool owner = k_dev != nullptr;
    if (owner && !v_dev) return fail(ctx, BK_ERR_INVALID, "bk_attn_step_split: k without v");
    int32_t &np = c->n_pos[c->slab(layer, seq)];
    if (!owner) return bk_decode_attn_split(c, layer, seq, np, q_pos, q_dev, out_dev, m, seqno);
    if (np >= c->cfg.n_ctx)
        return fail(ctx, BK_ERR_RANGE, "bk_attn_step_split: the local chunk is full (raise BONSAI_CTX)");
    if (m->ctx != ctx || m->n_rows != c->cfg.n_head || m->hd != c->cfg.hd || seqno == 0)
        return fail(ctx, BK_ERR_INVALID, "bk_attn_step_split: mailbox does not match, or sequence number 0");
    for (int r = 0; r < m->world; r++)
        if (!m->peer[r]) return fail(ctx, BK_ERR_INVALID, "bk_attn_step_split: peers are not opened");
    if (q_pos < 0 || q_pos >= c->rope->n_pos) return fail(ctx, BK_ERR_RANGE, "bk_attn_step_split: position beyond the rope table");
    // on caches that take the tensor-core kernels the row is stored by the decode launch itself
    DecodeArgs a;
    fill_decode_args(c, layer, 0, &a);
    const bool fused_append = decode_entry_uses_mma(ctx, a, np + 1);
    bk_status st = decode_with_exchange(c, layer, seq, np + 1, q_pos, q_dev, out_dev, m->d_peer, m->world, m->rank, seqno,
                                        k_dev, v_dev);
    if (st == BK_OK && fused_append) np += 1;  // (the other route went through bk_append, which counted it)
    return st;
}

}  // extern "C"
