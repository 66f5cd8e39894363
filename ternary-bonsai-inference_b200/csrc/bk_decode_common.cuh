// Tail shared by the decode kernels: merge the split-K chunks of one (sequence, kv head) and
// write the result.  A CTA that has reduced its chunk to (acc[NREP][256], M[NREP], L[NREP]) in
// shared memory (acc relative to M, exp2 domain) calls finish_item():
//   * more than one chunk: the CTA stores its triple in the partials buffer, takes a ticket
//     from the (sequence, kv head) counter and returns unless it is the last to arrive; the
//     last one re-reads every chunk's triple and combines them.  Nobody waits for anybody.
//   * planar V: the combined accumulator is still in Givens-rotated space and is rotated back
//     once here (src/forward.rs:349, shaders/attn_out_q.comp:85-91);
//   * output: acc / L (times sigmoid(gate) when the layer form of the step passes a gate), or
//     the unnormalised (acc, m, l) triple when the caller merges chunks held by other caches /
//     GPUs itself.
#pragma once

#include <cuda/atomic>
#include <math_constants.h>

#include "bk_device.cuh"
#include "bk_internal.h"
#include "bk_mma_common.cuh"

namespace bk {

constexpr int kFactorCap = 256;  // chunks whose rescale factors are cached in shared memory
constexpr int kDistSpin = 1 << 21;  // polls of the arrival counter before the slice combine gives up

// Per-CTA time stamps for tuning builds (-DBK_PHASE): stamp i of CTA b lands in g_phase[b][i].
#ifdef BK_PHASE
static __device__ unsigned long long g_phase[1024][16];
__device__ __forceinline__ unsigned long long phase_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define BK_STAMP(i)                                                                       \
    do {                                                                                  \
        if (threadIdx.x == 0 && blockIdx.x < 1024) g_phase[blockIdx.x][i] = phase_timer(); \
    } while (0)
#else
#define BK_STAMP(i)
#endif

// A free region of shared memory through which the last arriver streams the other chunks'
// triples (the tensor-core kernels pass their drained stage ring): the TMA engine copies them in
// rounds into the region's two halves, completion on the two mbarriers at `bar` (initialised by
// the caller with count 1 and not used for anything else).  addr = 0: no region, the combine reads
// the triples with ordinary loads.
struct FinishSmem {
    uint32_t addr = 0;    // shared-window address, 16-byte aligned
    uint32_t bytes = 0;
    uint32_t bar = 0;     // shared-window address of two consecutive mbarriers
    uint8_t *ptr = nullptr;  // the same region as a generic pointer
    int *err_flag = nullptr;
};

// Context split over the GPUs of one node: dims [d0, d0 + dn) of the (acc, m, l) rows of the n_rep q heads of
// kv head `kv`: send this rank's values to slot [rank] of every rank's mailbox, wait (bounded) for the same
// values of every rank in this rank's own mailbox, and write the log-sum-exp merge to a.out.
// A mailbox is [2 parities][world][n_head][hd + 2] eight-byte words (value bits, sequence number).  A word is
// stored with one 8-byte store, which arrives whole, so it validates itself: the receiver reads it until its
// second half is the call's sequence number.  Nothing else is needed - no arrival flags, no fence between data
// and flag, one trip over the link instead of three.  The CTA that holds coordinate 0 also sends the heads' m
// and l.  The word grid does not depend on how a rank has cut its work, so ranks whose launches have different
// shapes (or that send from the stand-alone exchange kernel) understand each other.  Slots alternate with the
// parity of the sequence number: a rank can be at most one call ahead of another (it needs the other's rows to
// finish a call), so a word is never overwritten before it was read.  vals: [n_rep][dn] in shared memory,
// relative to s_M (exp2 domain), not normalised.  Every thread of the CTA must call; on a time-out the
// affected outputs are zeros and the context's error word is raised.
// One mailbox word: value and sequence number in a single 8-byte store (never two 4-byte ones).
__device__ __forceinline__ void store_word(uint2 *p, float value, unsigned seqno) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};\n" ::"l"(p), "r"(__float_as_uint(value)), "r"(seqno) : "memory");
}

__device__ __forceinline__ void exchange_slice(const DecodeArgs &a, int n_rep, int slot, int kv, int d0, int dn,
                                               const float *vals, const float *s_M, const float *s_L, int *s_ok) {
    constexpr int kStride = kHd + 2;
    const int tid = threadIdx.x, nt = blockDim.x;
    const int world = a.xch_world, rank = a.xch_rank, n_rows = a.n_head, row0 = kv * n_rep;
    const unsigned seqno = a.xch_seqno, par = seqno & 1u;
    const size_t slot_w = (size_t)n_rows * kStride;
    (void)s_ok;
    BK_STAMP(10);
    for (int r = 0; r < world; r++) {
        uint2 *dst = reinterpret_cast<uint2 *>(a.xch_peer[r]) + ((size_t)par * world + rank) * slot_w + (size_t)row0 * kStride;
        for (int i = tid; i < n_rep * dn; i += nt) {
            const int rr = i / dn, d = i - rr * dn;
            store_word(dst + rr * kStride + d0 + d, vals[i], seqno);
        }
        if (d0 == 0 && tid < n_rep) {
            store_word(dst + tid * kStride + kHd, s_M[tid] * 0.6931471805599453f, seqno);  // log2 -> ln
            store_word(dst + tid * kStride + kHd + 1, s_L[tid], seqno);
        }
    }
    const uint2 *mbox = reinterpret_cast<const uint2 *>(a.xch_peer[rank]) + (size_t)par * world * slot_w + (size_t)row0 * kStride;
    bool first = true;
    for (int i = tid; i < n_rep * dn; i += nt) {
        const int rr = i / dn, d = d0 + (i - rr * dn);
        // every rank's (m, l, value): all loads of a round are issued together; words that have not arrived yet
        // are read again
        uint2 wm[kMaxWorld], wl[kMaxWorld], wx[kMaxWorld];
        unsigned pending = (world >= 32) ? 0xffffffffu : ((1u << world) - 1u);
        int polls = 0;
        bool ok = true;
        while (pending) {
#pragma unroll
            for (int r = 0; r < kMaxWorld; r++)
                if (pending >> r & 1u) {
                    const uint2 *p = mbox + (size_t)r * slot_w + (size_t)rr * kStride;
                    wm[r] = __ldcv(p + kHd);
                    wl[r] = __ldcv(p + kHd + 1);
                    wx[r] = __ldcv(p + d);
                }
#pragma unroll
            for (int r = 0; r < kMaxWorld; r++)
                if ((pending >> r & 1u) && wm[r].y == seqno && wl[r].y == seqno && wx[r].y == seqno) pending &= ~(1u << r);
            if (pending) {
                if (++polls > a.xch_spin) {  // a peer never sent: leave a mark and go on rather than hang
                    ok = false;
                    raise_error(a.xch_err, 3);
                    break;
                }
                if (polls > 2048) __nanosleep(64);  // the first microseconds without a pause: the ranks run in lock step
            }
        }
        if (first) {
            BK_STAMP(11);
            first = false;
        }
        float Mx = -CUDART_INF_F;
#pragma unroll
        for (int r = 0; r < kMaxWorld; r++)
            if (r < world && ok && __uint_as_float(wl[r].x) > 0.f) Mx = fmaxf(Mx, __uint_as_float(wm[r].x));
        float Ls = 0.f, sum = 0.f;
#pragma unroll
        for (int r = 0; r < kMaxWorld; r++)
            if (r < world && ok && __uint_as_float(wl[r].x) > 0.f) {
                const float f = expf(__uint_as_float(wm[r].x) - Mx);
                Ls = fmaf(__uint_as_float(wl[r].x), f, Ls);
                sum = fmaf(__uint_as_float(wx[r].x), f, sum);
            }
        a.out[((size_t)slot * a.n_head + row0 + rr) * kHd + d] = (ok && Ls > 0.f) ? sum / Ls : 0.f;
    }
    BK_STAMP(12);
}

// The slice form of the split-K combine.  When every CTA of a (sequence, kv head) is resident at
// the same time (the launcher sets DecodeArgs::dist only then), nobody leaves after publishing:
// each CTA waits (bounded) until all n_chunks triples are in the scratch and then combines ONE
// slice of the output - all heads of the group, `D` consecutive coordinates - from every chunk's
// triple: one L2 round trip of a few hundred 16-byte loads per CTA instead of one CTA walking
// through all the triples.  The slices are whole Givens pairs, so the inverse rotation, the
// division by l and the gate happen here too.  `red` is free shared memory (16-byte aligned, at
// least 16 KiB); s_f holds kFactorCap * NREP floats.  Returns false when the wait ran out.
template <int NREP>
__device__ __forceinline__ bool combine_slice(const DecodeArgs &a, int slot, int kv, int my_chunk, int n_chunks,
                                              const float *base /* first chunk's triple */, float *red, float *s_f,
                                              float *s_M, float *s_L, int *s_flag, unsigned *counter, bool v_planar,
                                              const float *givens, int *err_flag) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        cuda::atomic_ref<unsigned, cuda::thread_scope_device> cnt(*counter);
        int polls = 0, ok = 1;
        while (cnt.load(cuda::memory_order_acquire) < (unsigned)n_chunks) {
            if (++polls > kDistSpin) {  // never expected: leave a mark, write nothing
                ok = 0;
                raise_error(err_flag, 6);
                break;
            }
        }
        *s_flag = ok;
    }
    __syncthreads();
    BK_STAMP(7);
    if (!*s_flag) return false;
    int D4 = (kHd / 4 + n_chunks - 1) / n_chunks;  // 16-byte columns per head in a slice
    if (a.xch_peer) {  // context split: slices on the mailbox's octet grid, and of a size that divides the row
        int D8 = 8;
        while (D8 * n_chunks < kHd) D8 <<= 1;
        D4 = D8 >> 2;
    }
    const int D = 4 * D4, n_slices = (kHd + D - 1) / D;
    if (my_chunk >= n_slices) return true;
    const int d0 = my_chunk * D, d4 = min(D4, (kHd - d0) >> 2), dn = 4 * d4;
    const int n_col = NREP * d4;                     // 16-byte columns of this slice (<= 192 for two chunks)
    const int n_grp = max(1, 256 / n_col);           // thread groups; group g takes chunks g, g + n_grp, ...
    const bool act = tid < n_grp * n_col;
    const int grp = tid / n_col, col = tid - grp * n_col, r_col = col / d4, j_col = col - r_col * d4;
    // the data loads go out first: they and the (m, l) sweep below share one round trip
    constexpr int kPre = 4;
    float4 pre[kPre];
    const float *src = base + (size_t)r_col * kScratchStride + d0 + 4 * j_col;
#pragma unroll
    for (int u = 0; u < kPre; u++) {
        const int c = grp + u * n_grp;
        pre[u] = (act && c < n_chunks) ? __ldcg(reinterpret_cast<const float4 *>(src + (size_t)c * NREP * kScratchStride))
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float *gate = (a.gate && !a.partial) ? a.gate + ((size_t)slot * a.n_head + (size_t)kv * NREP) * a.gate_stride + d0 : nullptr;
    if (warp < NREP) {  // one warp per head: global max, every chunk's factor, the merged l
        const int r = warp;
        constexpr int kPer = kFactorCap / 32;
        float2 ml[kPer];
        float M = -CUDART_INF_F;
#pragma unroll
        for (int u = 0; u < kPer; u++) {
            const int c = lane + 32 * u;
            ml[u] = make_float2(-CUDART_INF_F, 0.f);
            if (c < n_chunks) ml[u] = __ldcg(reinterpret_cast<const float2 *>(base + ((size_t)c * NREP + r) * kScratchStride + kHd));
            M = fmaxf(M, ml[u].x);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
        float Lsum = 0.f;
#pragma unroll
        for (int u = 0; u < kPer; u++) {
            const int c = lane + 32 * u;
            const float f = ml[u].x > -CUDART_INF_F ? exp2f(ml[u].x - M) : 0.f;
            Lsum = fmaf(ml[u].y, f, Lsum);
            if (c < n_chunks) s_f[c * NREP + r] = f;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) Lsum += __shfl_xor_sync(0xffffffffu, Lsum, off);
        if (lane == 0) {
            s_M[r] = M;
            s_L[r] = Lsum;
        }
    }
    __syncthreads();
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    if (act) {
        for (int c0 = grp; c0 < n_chunks; c0 += kPre * n_grp) {
            if (c0 > grp) {
#pragma unroll
                for (int u = 0; u < kPre; u++) {
                    const int c = c0 + u * n_grp;
                    pre[u] = c < n_chunks ? __ldcg(reinterpret_cast<const float4 *>(src + (size_t)c * NREP * kScratchStride))
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int u = 0; u < kPre; u++) {
                const int c = c0 + u * n_grp;
                const float f = c < n_chunks ? s_f[c * NREP + r_col] : 0.f;
                if (f != 0.f) {  // an empty chunk's accumulator is never looked at
                    sum.x = fmaf(pre[u].x, f, sum.x);
                    sum.y = fmaf(pre[u].y, f, sum.y);
                    sum.z = fmaf(pre[u].z, f, sum.z);
                    sum.w = fmaf(pre[u].w, f, sum.w);
                }
            }
        }
        reinterpret_cast<float4 *>(red)[grp * n_col + col] = sum;
    }
    __syncthreads();
    float *res = red + (size_t)4 * n_grp * n_col;  // [NREP][dn], fixed summation order over the groups
    const int n_out = NREP * dn, nthr = (int)blockDim.x;  // (up to 768 outputs for a slice of half a row: loop)
    for (int i = tid; i < n_out; i += nthr) {
        const int r = i / dn, d = i - r * dn;
        float t = 0.f;
        for (int g2 = 0; g2 < n_grp; g2++) t += red[((size_t)g2 * n_col + r * d4 + (d >> 2)) * 4 + (d & 3)];
        res[i] = t;
    }
    __syncthreads();
    float *snd = res + n_out;  // context split: what this slice sends
    for (int i = tid; i < n_out; i += nthr) {
        const int r_o = i / dn, d_o = i - r_o * dn;
        float o = res[i];
        if (v_planar) {  // undo the Givens rotation: coordinate d0 + d and its partner (src/forward.rs:349)
            const int pr = (d0 + d_o) >> 1;
            const float c = givens[2 * pr], sn = givens[2 * pr + 1];
            float o0, o1;
            givens_inv(res[r_o * dn + (d_o & ~1)], res[r_o * dn + (d_o | 1)], c, sn, o0, o1);
            o = (d_o & 1) ? o1 : o0;
        }
        if (a.xch_peer) {
            snd[i] = o;
        } else if (a.partial) {
            a.out[((size_t)slot * a.n_head + (size_t)kv * NREP + r_o) * kPartStride + d0 + d_o] = o;
        } else {
            const float Ls = s_L[r_o];
            o = Ls > 0.f ? o / Ls : 0.f;
            // src/forward.rs:379-382 with src/kernels.rs:162: out *= 1 / (1 + exp(-gate))
            if (gate) o *= 1.0f / (1.0f + expf(-__ldg(gate + (size_t)r_o * a.gate_stride + d_o)));
            a.out[((size_t)slot * a.n_head + (size_t)kv * NREP + r_o) * kHd + d0 + d_o] = o;
        }
    }
    if (a.xch_peer) {  // context split: this slice goes to every rank and is merged with theirs
        __syncthreads();
        exchange_slice(a, NREP, slot, kv, d0, dn, snd, s_M, s_L, s_flag);
        return true;
    }
    if (a.partial && my_chunk == 0 && tid < NREP) {
        float *po = a.out + ((size_t)slot * a.n_head + (size_t)kv * NREP + tid) * kPartStride;
        po[kHd] = s_M[tid] * 0.6931471805599453f;  // log2 -> ln
        po[kHd + 1] = s_L[tid];
    }
    return true;
}

template <int NREP, bool STREAM = false>
__device__ __forceinline__ void finish_item(const DecodeArgs &a, int slot, int s, int kv, int item, int n_chunks,
                                            int first_item, float *s_acc /* [NREP][kHd] */, float *s_M, float *s_L,
                                            int *s_last, bool v_planar,
                                            const float *givens = nullptr /* shared-memory copy, if the caller has one */,
                                            FinishSmem fs = FinishSmem()) {
    __shared__ float s_f[kFactorCap * NREP];
    __shared__ float s_scale[8];
    // the first 256 threads work; a larger CTA's remaining threads only take part in the barriers
    const int tid = threadIdx.x, nt = 256;
    const bool act = threadIdx.x < 256;
    const int tid0 = act ? tid : (1 << 30);  // loop start that keeps idle threads out of strided loops
    const int warp = tid >> 5, lane = tid & 31;
    // gate values of this thread's outputs (coordinate tid of every head); the CTA that writes the
    // output fetches them as early as it knows it is the one, so they travel with the partials
    const float *gate = (a.gate && !a.partial && act)
                            ? a.gate + ((size_t)slot * a.n_head + (size_t)kv * NREP) * a.gate_stride + tid : nullptr;
    float gv[NREP];
    auto load_gate = [&]() {
#pragma unroll
        for (int r = 0; r < NREP; r++) gv[r] = gate ? __ldg(gate + (size_t)r * a.gate_stride) : 0.f;
    };
    if (n_chunks <= 1) load_gate();
    if (n_chunks > 1) {
        float *part = a.partials + ((size_t)item * NREP) * kScratchStride;
        for (int i = tid0; i < NREP * kHd; i += nt) {
            const int r = i / kHd, d = i - r * kHd;
            part[(size_t)r * kScratchStride + d] = s_acc[i];
        }
        if (tid < NREP) {
            part[(size_t)tid * kScratchStride + kHd] = s_M[tid];
            part[(size_t)tid * kScratchStride + kHd + 1] = s_L[tid];
        }
        // Publish: the barrier orders every thread's stores before thread 0's release, which
        // makes them visible to whoever later acquires the counter (cumulativity), so no thread
        // needs a full __threadfence().
        __syncthreads();
        if (tid == 0) {
            cuda::atomic_ref<unsigned, cuda::thread_scope_device> cnt(a.counters[s * a.n_kv + kv]);
            const unsigned ticket = cnt.fetch_add(1u, cuda::memory_order_acq_rel);
            *s_last = (ticket == (unsigned)(n_chunks - 1));
        }
        if (STREAM) asm volatile("fence.proxy.async;\n" ::: "memory");  // this thread's shared-memory traffic before the copies below
        __syncthreads();
        BK_STAMP(6);
        if (STREAM && a.dist && fs.ptr && fs.bytes >= 20480 && n_chunks <= kFactorCap) {
            // every CTA of this (sequence, kv head) stays and combines one slice of the output
            const float *base0 = a.partials + (size_t)first_item * NREP * kScratchStride;
            combine_slice<NREP>(a, slot, kv, item - first_item, n_chunks, base0, reinterpret_cast<float *>(fs.ptr), s_f, s_M,
                                s_L, s_last, &a.counters[s * a.n_kv + kv], v_planar, givens ? givens : a.givens, fs.err_flag);
            BK_STAMP(8);
            return;  // (the counter is cleared by the launch after the next one)
        }
        if (!*s_last) return;
        const float *base = a.partials + (size_t)first_item * NREP * kScratchStride;
        constexpr uint32_t kChunkBytes = NREP * kScratchStride * sizeof(float);
        const int cap = STREAM ? min((int)((fs.bytes / 2) / kChunkBytes), 32) : 0;  // chunks per half
        if (STREAM && cap >= 1 && fs.bytes >= (blockDim.x >> 6) * NREP * kHd * sizeof(float)) {
            // ---- streamed combine: chunks arrive through the TMA engine, two rounds in flight ------
            const int n_rounds = (n_chunks + cap - 1) / cap;
            const uint32_t half_bytes = (uint32_t)cap * kChunkBytes;
            auto issue_round = [&](int rd) {
                const int c0 = rd * cap, nc = min(cap, n_chunks - c0);
                const uint32_t bar = fs.bar + (uint32_t)(rd & 1) * 8u, dst = fs.addr + (uint32_t)(rd & 1) * half_bytes;
                mbar_expect_tx(bar, (uint32_t)nc * kChunkBytes);
                for (int c = 0; c < nc; c++)
                    tma_bulk(dst + (uint32_t)c * kChunkBytes, base + (size_t)(c0 + c) * NREP * kScratchStride, kChunkBytes, bar);
            };
            if (tid == 0) {
                // the other CTAs' stores (generic proxy, acquired through the ticket) before the async-proxy reads
                asm volatile("fence.proxy.async;\n" ::: "memory");
                issue_round(0);
                if (n_rounds > 1) issue_round(1);
            }
            load_gate();
            const int n_g = (int)blockDim.x >> 6, rg = tid >> 6, x = tid & 63;  // 64 threads span a row with float4
            float4 sum[NREP];
#pragma unroll
            for (int r = 0; r < NREP; r++) sum[r] = make_float4(0.f, 0.f, 0.f, 0.f);
            float M_run = -CUDART_INF_F, L_run = 0.f;  // warp r < NREP: running max and sum of head r
            for (int rd = 0; rd < n_rounds; rd++) {
                const int nc = min(cap, n_chunks - rd * cap);
                const uint32_t bar = fs.bar + (uint32_t)(rd & 1) * 8u, parity = (uint32_t)(rd >> 1) & 1u;
                int polls = 0;
                while (!mbar_try_wait(bar, parity)) {
                    if (++polls > kWaitPolls) {  // never expected; leave a mark and go on rather than hang
                        if (tid == 0) raise_error(fs.err_flag, 3);
                        break;
                    }
                }
                const float *H = reinterpret_cast<const float *>(fs.ptr + (size_t)(rd & 1) * half_bytes);
                if (warp < NREP) {  // one warp per head: this round's factors, online in the running max
                    const int r = warp;
                    const bool valid = lane < nc;
                    const float2 ml = valid ? *reinterpret_cast<const float2 *>(H + ((size_t)lane * NREP + r) * kScratchStride + kHd)
                                            : make_float2(-CUDART_INF_F, 0.f);
                    float mx = ml.x;
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
                    const float Mn = fmaxf(M_run, mx);
                    const float fc = ml.x > -CUDART_INF_F ? exp2f(ml.x - Mn) : 0.f;
                    const float keep = M_run > -CUDART_INF_F ? exp2f(M_run - Mn) : 0.f;
                    float ls = ml.y * fc;
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, off);
                    L_run = fmaf(L_run, keep, ls);
                    M_run = Mn;
                    if (valid) s_f[lane * NREP + r] = fc;
                    if (lane == 0) s_scale[r] = keep;
                }
                __syncthreads();
#pragma unroll
                for (int r = 0; r < NREP; r++) {
                    const float k = s_scale[r];
                    sum[r].x *= k; sum[r].y *= k; sum[r].z *= k; sum[r].w *= k;
                }
                for (int c = rg; c < nc; c += n_g) {
#pragma unroll
                    for (int r = 0; r < NREP; r++) {
                        const float4 v = reinterpret_cast<const float4 *>(H + ((size_t)c * NREP + r) * kScratchStride)[x];
                        const float f = s_f[c * NREP + r];
                        sum[r].x = fmaf(v.x, f, sum[r].x);
                        sum[r].y = fmaf(v.y, f, sum[r].y);
                        sum[r].z = fmaf(v.z, f, sum[r].z);
                        sum[r].w = fmaf(v.w, f, sum[r].w);
                    }
                }
                __syncthreads();  // this half and the factors are free again
                if (tid == 0 && rd + 2 < n_rounds) issue_round(rd + 2);
            }
            if (warp < NREP && lane == 0) {
                s_M[warp] = M_run;
                s_L[warp] = L_run;
            }
            // the groups' sums meet in the first half (every copy into it has been consumed), fixed order
            float4 *scratch = reinterpret_cast<float4 *>(fs.ptr);  // [n_g][NREP][64]
#pragma unroll
            for (int r = 0; r < NREP; r++) scratch[((size_t)rg * NREP + r) * 64 + x] = sum[r];
            __syncthreads();
            if (act) {
                const float *sf = reinterpret_cast<const float *>(fs.ptr);
#pragma unroll
                for (int r = 0; r < NREP; r++) {
                    float t = 0.f;
                    for (int g2 = 0; g2 < n_g; g2++) t += sf[((size_t)g2 * NREP + r) * kHd + tid];
                    s_acc[r * kHd + tid] = t;
                }
            }
            if (tid == 0) a.counters[s * a.n_kv + kv] = 0;  // ready for the next launch
            __syncthreads();
        } else {
        // 64 threads span one 256-float row with float4 loads; the four 64-thread groups take
        // every fourth chunk.  The (head, chunk) pairs of a thread form one flat list walked 24
        // independent 16-byte loads at a time.  The first batch is issued before the m/l sweep
        // below so that both travel in the same L2 round trip.
        const int rg = tid >> 6, x = tid & 63;
        const int per_rg = (n_chunks - rg + 3) / 4;  // chunks rg, rg+4, ...
        const int n_pairs = act ? per_rg * NREP : 0;
        constexpr int kBatch = (NREP == 6) ? 30 : 32;  // a multiple of NREP: slot u is always head u % NREP
        float4 v[kBatch];
        auto load_batch = [&](int i0) {
#pragma unroll
            for (int u = 0; u < kBatch; u++) {
                const int i = i0 + u, r = u % NREP;
                const int c = rg + 4 * (i / NREP);
                if (i < n_pairs)
                    v[u] = __ldcg(reinterpret_cast<const float4 *>(base + ((size_t)c * NREP + r) * kScratchStride) + x);
                else
                    v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        };
        load_batch(0);
        load_gate();
        // one warp per head: global max, the chunks' rescale factors and the merged l, from one
        // sweep over the (m, l) pairs
        if (warp < NREP) {
            const int r = warp;
            constexpr int kPer = kFactorCap / 32;  // (m, l) pairs a lane keeps in registers
            float2 ml[kPer];
            float M = -CUDART_INF_F;
#pragma unroll
            for (int u = 0; u < kPer; u++) {
                const int c = lane + 32 * u;
                ml[u] = make_float2(-CUDART_INF_F, 0.f);
                if (c < n_chunks)
                    ml[u] = __ldcg(reinterpret_cast<const float2 *>(base + ((size_t)c * NREP + r) * kScratchStride + kHd));
                M = fmaxf(M, ml[u].x);
            }
            for (int c = kFactorCap + lane; c < n_chunks; c += 32)  // beyond the cached range (rare)
                M = fmaxf(M, __ldcg(base + ((size_t)c * NREP + r) * kScratchStride + kHd));
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
            float Lsum = 0.f;
#pragma unroll
            for (int u = 0; u < kPer; u++) {
                const int c = lane + 32 * u;
                const float f = ml[u].x > -CUDART_INF_F ? exp2f(ml[u].x - M) : 0.f;
                Lsum = fmaf(ml[u].y, f, Lsum);
                if (c < n_chunks) s_f[c * NREP + r] = f;
            }
            for (int c = kFactorCap + lane; c < n_chunks; c += 32) {
                const float2 x2 = __ldcg(reinterpret_cast<const float2 *>(base + ((size_t)c * NREP + r) * kScratchStride + kHd));
                Lsum = fmaf(x2.y, x2.x > -CUDART_INF_F ? exp2f(x2.x - M) : 0.f, Lsum);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) Lsum += __shfl_xor_sync(0xffffffffu, Lsum, off);
            if (lane == 0) {
                s_M[r] = M;
                s_L[r] = Lsum;
            }
        }
        __syncthreads();
        float4 sum[NREP];
#pragma unroll
        for (int r = 0; r < NREP; r++) sum[r] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int i0 = 0; i0 < n_pairs; i0 += kBatch) {
            if (i0 > 0) load_batch(i0);
#pragma unroll
            for (int u = 0; u < kBatch; u++) {
                const int i = i0 + u, r = u % NREP;
                const int c = rg + 4 * (i / NREP);
                float f = 0.f;
                if (i < n_pairs) {
                    if (c < kFactorCap) f = s_f[c * NREP + r];
                    else {
                        const float mc = __ldcg(base + ((size_t)c * NREP + r) * kScratchStride + kHd);
                        f = mc > -CUDART_INF_F ? exp2f(mc - s_M[r]) : 0.f;
                    }
                }
                sum[r].x = fmaf(v[u].x, f, sum[r].x);
                sum[r].y = fmaf(v[u].y, f, sum[r].y);
                sum[r].z = fmaf(v[u].z, f, sum[r].z);
                sum[r].w = fmaf(v[u].w, f, sum[r].w);
            }
        }
        // fixed order over the four groups keeps the result deterministic
        for (int gsel = 0; gsel < 4; gsel++) {
            if (rg == gsel) {
#pragma unroll
                for (int r = 0; r < NREP; r++) {
                    float4 *dst = reinterpret_cast<float4 *>(s_acc + r * kHd) + x;
                    if (gsel == 0) *dst = sum[r];
                    else {
                        float4 o = *dst;
                        o.x += sum[r].x; o.y += sum[r].y; o.z += sum[r].z; o.w += sum[r].w;
                        *dst = o;
                    }
                }
            }
            __syncthreads();
        }
        if (tid == 0) a.counters[s * a.n_kv + kv] = 0;  // ready for the next launch
        __syncthreads();
        }
    }

    if (v_planar) {
        for (int i = tid0; i < NREP * (kHd / 2); i += nt) {
            const int r = i / (kHd / 2), pr = i - r * (kHd / 2);
            float o0, o1;
            const float *gv = givens ? givens : a.givens;
            givens_inv(s_acc[r * kHd + 2 * pr], s_acc[r * kHd + 2 * pr + 1], gv[2 * pr], gv[2 * pr + 1],
                       o0, o1);
            s_acc[r * kHd + 2 * pr] = o0;
            s_acc[r * kHd + 2 * pr + 1] = o1;
        }
        __syncthreads();
    }
    if (a.xch_peer) {
        // ---- context split: send this kv head's rows to every rank, wait for everybody's, merge ----
        __shared__ int s_ok;
        exchange_slice(a, NREP, slot, kv, 0, kHd, s_acc, s_M, s_L, &s_ok);
    } else if (a.partial) {
        float *out = a.out + ((size_t)slot * a.n_head + (size_t)kv * NREP) * kPartStride;
        for (int i = tid0; i < NREP * kHd; i += nt) {
            const int r = i / kHd, d = i - r * kHd;
            out[(size_t)r * kPartStride + d] = s_acc[i];
        }
        if (tid < NREP) {
            out[(size_t)tid * kPartStride + kHd] = s_M[tid] * 0.6931471805599453f;  // log2 -> ln
            out[(size_t)tid * kPartStride + kHd + 1] = s_L[tid];
        }
    } else {
        float *out = a.out + ((size_t)slot * a.n_head + (size_t)kv * NREP) * kHd;
        if (act) {
#pragma unroll
            for (int r = 0; r < NREP; r++) {
                const float Ls = s_L[r];
                float o = Ls > 0.f ? s_acc[r * kHd + tid] / Ls : 0.f;
                // src/forward.rs:379-382 with src/kernels.rs:162: out *= 1 / (1 + exp(-gate))
                if (gate) o *= 1.0f / (1.0f + expf(-gv[r]));
                out[r * kHd + tid] = o;
            }
        }
    }
}

}  // namespace bk
