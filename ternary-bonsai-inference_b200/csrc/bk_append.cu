// Fused KV append: IMROPE on K, then store K and V rows as f32, f16 or rotated Lloyd-Max
// ("planar") rows, one launch for any number of tokens.  Replaces rope_imrope.comp (k side),
// kv_store.comp, kv_store_f16.comp and kv_store_q.comp and follows the reference CPU path
// bit for bit (src/forward.rs:259-285, src/kvquant.rs:397-412, src/rope.rs:61-69).
//
// A CTA stages 32 vectors of 256 floats ((K|V, kv head) of consecutive tokens):
//   1. coalesced float4 loads into shared memory; K vectors rotate pairs (j, j + n_rot/2) with
//      the (cos, sin) row of the token's position from the host-built rope table;
//   2. planar rows: one warp adds the 256 squares of all 32 vectors, a vector per lane, each lane
//      in order (the reference's f32 sum is sequential, so each chain is; 32 run side by side);
//   3. the warps scale, Givens-rotate, find the nearest centroid (one read of a host-built cell table of the
//      decision thresholds, or a binary search and a neighbour check: the same index as the reference's
//      linear scan) and write `bits` bytes per lane;
//      f32/f16 rows leave as 128-bit stores.
// Traffic per token is the algorithmic minimum: 2*n_kv*1 KiB in, rows + norms out.
#include <atomic>

#include "bk_device.cuh"
#include "bk_internal.h"

namespace bk {

namespace {

constexpr int kVecPad = kHd + 4;  // floats per staged vector; +4 keeps float4 alignment and makes the
                                  // per-lane 128-bit reads of the norm pass conflict-free
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

// Eight consecutive coordinates of a staged vector for every lane without bank conflicts: two 128-bit reads
// in the staging layout (coordinates 4 l .. 4 l + 3 and 128 + 4 l .. + 3), then lanes 2m and 2m + 1 swap
// one of them: the even lane ends with group m (coordinates 8 m .. 8 m + 7), the odd one with group 16 + m.
// (Reading 8 consecutive floats per lane directly puts eight lanes on every bank.)  Returns the group.
__device__ __forceinline__ int load_group_of_8(const float *sx, int lane, float (&x)[8]) {
    const float4 a = reinterpret_cast<const float4 *>(sx)[lane], b = reinterpret_cast<const float4 *>(sx)[lane + 32];
    const bool odd = lane & 1;
    const float4 send = odd ? a : b;
    float4 recv;
    recv.x = __shfl_xor_sync(0xffffffffu, send.x, 1);
    recv.y = __shfl_xor_sync(0xffffffffu, send.y, 1);
    recv.z = __shfl_xor_sync(0xffffffffu, send.z, 1);
    recv.w = __shfl_xor_sync(0xffffffffu, send.w, 1);
    const float4 lo = odd ? recv : a, hi = odd ? b : recv;
    x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w;
    x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
    return odd ? 16 + (lane >> 1) : (lane >> 1);
}

// Rotate, quantize and pack the 8 coordinates of one lane; `n` is the vector's norm.
template <int BITS>
__device__ __forceinline__ void store_planar_row(const float *sx, int lane, float n, const float *givens,
                                                 const float *sbook, uint8_t *row) {
    const float inv = (n > 1e-12f) ? __fdiv_rn(1.0f, n) : 0.0f;
    float x[8];
    const int group = load_group_of_8(sx, lane, x);
    const float4 g0 = reinterpret_cast<const float4 *>(givens)[2 * group], g1 = reinterpret_cast<const float4 *>(givens)[2 * group + 1];
    const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    uint64_t packed = 0;
#pragma unroll
    for (int pr = 0; pr < 4; pr++) {
        const float a = __fmul_rn(x[2 * pr], inv), b = __fmul_rn(x[2 * pr + 1], inv);
        float r0, r1;
        givens_fwd(a, b, gv[2 * pr], gv[2 * pr + 1], r0, r1);
        packed |= (uint64_t)nearest_centroid_fast<BITS>(r0, sbook) << (BITS * (2 * pr));
        packed |= (uint64_t)nearest_centroid_fast<BITS>(r1, sbook) << (BITS * (2 * pr + 1));
    }
    store_group8<BITS>(row, group, packed);
}

// The same with the one-read centroid search (codebooks of up to 16 centroids; bk_device.cuh).
template <int BITS>
__device__ __forceinline__ void store_planar_row_thr(const float *sx, int lane, float n, const float *givens,
                                                     const float *sbook, const uint2 *tab, uint8_t *row) {
    const float inv = (n > 1e-12f) ? __fdiv_rn(1.0f, n) : 0.0f;
    float x[8];
    const int group = load_group_of_8(sx, lane, x);  // coordinates 8 group .. 8 group + 7
    const float4 g0 = reinterpret_cast<const float4 *>(givens)[2 * group], g1 = reinterpret_cast<const float4 *>(givens)[2 * group + 1];
    const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    uint32_t packed = 0;  // 8 indices of at most 4 bits
#pragma unroll
    for (int pr = 0; pr < 4; pr++) {
        const float a = __fmul_rn(x[2 * pr], inv), b = __fmul_rn(x[2 * pr + 1], inv);
        float r0, r1;
        givens_fwd(a, b, gv[2 * pr], gv[2 * pr + 1], r0, r1);
        packed |= nearest_centroid_thr<BITS>(r0, sbook, tab) << (BITS * (2 * pr));
        packed |= nearest_centroid_thr<BITS>(r1, sbook, tab) << (BITS * (2 * pr + 1));
    }
    store_group8<BITS>(row, group, (uint64_t)packed);
}

__device__ __forceinline__ void store_f32_row(const float *sx, int lane, uint8_t *row) {
    float4 *dst = reinterpret_cast<float4 *>(row);
    const float4 *src = reinterpret_cast<const float4 *>(sx);
    dst[lane] = src[lane];
    dst[lane + 32] = src[lane + 32];
}

__device__ __forceinline__ void store_f16_row(const float *sx, int lane, uint8_t *row) {
    float x[8];
    const int group = load_group_of_8(sx, lane, x);
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t lo = f32_to_half_ref(x[2 * i]);
        const uint32_t hi = f32_to_half_ref(x[2 * i + 1]);
        w[i] = lo | (hi << 16);
    }
    reinterpret_cast<uint4 *>(row)[group] = make_uint4(w[0], w[1], w[2], w[3]);
}

// A CTA takes 32 consecutive vectors of the launch (vector = token * 2*n_kv + j; j < n_kv: K head
// j, else V head j - n_kv).  Pass 1: each warp stages 8 vectors with float4 loads and ropes the K
// ones.  Pass 2: warp 0 adds the squares of all 32 vectors, one vector per lane, each lane in
// order (the reference's f32 sum is sequential, so the chain is; 32 chains run side by side).
// Pass 3: each warp scales, rotates, finds the nearest centroids of and stores its 8 vectors.
// kVecs = 32 for bulk calls (throughput: every lane of the norm pass works), 8 for small calls
// (latency: one vector per warp).
template <int BITS, int kVecs>
__global__ void __launch_bounds__(kThreads, kVecs == 32 ? 5 : 4) append_kernel(AppendArgs a) {
    extern __shared__ __align__(16) float smem[];
    float *sbook = smem + kVecs * kVecPad;  // centroids
    float *sgiv = sbook + 256;              // Givens table
    float *snorm = sgiv + kHd;              // the 32 norms
    [[maybe_unused]] uint2 *tab = reinterpret_cast<uint2 *>(snorm + 32);    // the 512 cells of the one-read centroid search
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kv = a.n_kv, per_tok = 2 * n_kv;
    const int n_vec = a.n_tokens * per_tok, v0 = blockIdx.x * kVecs;
    // vector -> (token, K|V head): a shift and a mask when 2 * n_kv is a power of two (it is for qwen35)
    const int tok_shift = (per_tok & (per_tok - 1)) == 0 ? __ffs(per_tok) - 1 : -1;
    auto tok_of = [&](int vec) { return tok_shift >= 0 ? vec >> tok_shift : vec / per_tok; };
    const bool planar = a.k_kind == ROW_PLANAR || a.v_kind == ROW_PLANAR;

    if (BITS > 0) {
        for (int i = threadIdx.x; i < (1 << BITS); i += kThreads) sbook[i] = a.book[i];
        for (int i = threadIdx.x; i < kHd; i += kThreads) sgiv[i] = a.givens[i];
        if constexpr (BITS >= 1 && BITS <= 4)  // built once per context on the host
            for (int i = threadIdx.x; i < 256; i += kThreads) reinterpret_cast<uint4 *>(tab)[i] = __ldg(reinterpret_cast<const uint4 *>(a.cell_tab) + i);
    }
    // k and v may come from the previous kernel in the stream: with programmatic dependent launch
    // only the table copies above run ahead of it.  Nothing after this kernel depends on more
    // than its completion, so dependents may be scheduled right away.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    // ---- pass 1: stage (and rope).  A warp owns vectors warp, warp + 8, ...; all of their global
    // loads (rows and rope entries) are issued before any is used, so the pass costs one round trip.
    constexpr int kPerWarp = kVecs / kWarps;
    float4 ra[kPerWarp], rb[kPerWarp];
    float2 rcs[kPerWarp];
    const int half = a.n_rot >> 1;
#pragma unroll
    for (int u = 0; u < kPerWarp; u++) {
        const int vec = v0 + warp + u * kWarps;
        ra[u] = rb[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        rcs[u] = make_float2(1.f, 0.f);
        if (vec < n_vec) {
            const int tok = tok_of(vec), j = vec - tok * per_tok;
            const bool is_v = j >= n_kv;
            const int kv = is_v ? j - n_kv : j;
            const float4 *src4 = reinterpret_cast<const float4 *>((is_v ? a.v : a.k) + ((size_t)tok * n_kv + kv) * kHd);
            ra[u] = __ldg(src4 + lane);
            rb[u] = __ldg(src4 + lane + 32);
            if (!is_v && lane < half) {  // n_rot <= 64: one rope entry per lane
                const int pos = a.desc ? a.desc[tok].z : a.pos0 + tok;
                rcs[u] = __ldg(a.rope + (size_t)pos * half + lane);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < kPerWarp; u++) {
        const int lv = warp + u * kWarps, vec = v0 + lv;
        if (vec >= n_vec) continue;
        float *sx = smem + lv * kVecPad;
        reinterpret_cast<float4 *>(sx)[lane] = ra[u];
        reinterpret_cast<float4 *>(sx)[lane + 32] = rb[u];
        const bool is_v = (vec - tok_of(vec) * per_tok) >= n_kv;
        if (!is_v) {
            __syncwarp();
            if (half <= 32) {
                if (lane < half) {
                    float x0 = sx[lane], x1 = sx[lane + half];
                    rope_pair(x0, x1, rcs[u]);
                    sx[lane] = x0;
                    sx[lane + half] = x1;
                }
            } else {  // wider rotations: entries beyond the prefetched 32 come straight from the table
                const int tok = tok_of(vec), pos = a.desc ? a.desc[tok].z : a.pos0 + tok;
                const float2 *cs = a.rope + (size_t)pos * half;
                for (int p = lane; p < half; p += 32) {
                    float x0 = sx[p], x1 = sx[p + half];
                    rope_pair(x0, x1, cs[p]);
                    sx[p] = x0;
                    sx[p + half] = x1;
                }
            }
        }
    }
    __syncthreads();
    // ---- pass 2: 32 sequential sums side by side ----------------------------------------------------
    if (planar && warp == 0 && lane < kVecs && v0 + lane < n_vec) {
        const float4 *x4 = reinterpret_cast<const float4 *>(smem + lane * kVecPad);
        float acc = 0.0f;
#pragma unroll 8
        for (int i = 0; i < kHd / 4; i++) {
            const float4 x = x4[i];
            acc = __fadd_rn(acc, __fmul_rn(x.x, x.x));
            acc = __fadd_rn(acc, __fmul_rn(x.y, x.y));
            acc = __fadd_rn(acc, __fmul_rn(x.z, x.z));
            acc = __fadd_rn(acc, __fmul_rn(x.w, x.w));
        }
        snorm[lane] = __fsqrt_rn(acc);
    }
    __syncthreads();
    // ---- pass 3: store --------------------------------------------------------------------------------
    for (int lv = warp; lv < kVecs; lv += kWarps) {
        const int vec = v0 + lv;
        if (vec >= n_vec) break;
        const int tok = tok_of(vec), j = vec - tok * per_tok;
        const bool is_v = j >= n_kv;
        const int kv = is_v ? j - n_kv : j;
        size_t seq_rows = 0;
        int row_idx;
        if (a.desc) {
            const int4 d = a.desc[tok];
            seq_rows = (size_t)d.x * a.seq_stride_rows;
            row_idx = d.y;
        } else {
            row_idx = a.row0 + tok;
        }
        const float *sx = smem + lv * kVecPad;
        const size_t r = seq_rows + (size_t)row_idx * n_kv + kv;
        const int kind = is_v ? a.v_kind : a.k_kind;
        uint8_t *row = (is_v ? a.v_rows + r * a.v_row_bytes : a.k_rows + r * a.k_row_bytes);
        if (kind == ROW_F32) {
            store_f32_row(sx, lane, row);
        } else if (kind == ROW_F16) {
            store_f16_row(sx, lane, row);
        } else {
            if constexpr (BITS > 0) {
                const float n = snorm[lv];
                if (lane == 0) (is_v ? a.v_norms : a.k_norms)[r] = n;
                if constexpr (BITS <= 4) store_planar_row_thr<BITS>(sx, lane, n, sgiv, sbook, tab, row);
                else store_planar_row<BITS>(sx, lane, n, sgiv, sbook, row);
            }
        }
    }
}


}  // namespace

bk_status launch_append(bk_ctx *ctx, const AppendArgs &a) {
    if (a.n_tokens <= 0) return BK_OK;
    const int threads = kThreads;
    const size_t n_vec = (size_t)a.n_tokens * 2 * a.n_kv;
    const bool bulk = n_vec > (size_t)8 * 2 * ctx->n_sms;  // more than two small CTAs per SM: go for throughput
    const int vecs = bulk ? 32 : 8;
    const size_t smem = (size_t)(vecs * kVecPad + 256 + kHd + 32) * sizeof(float) + 512 * sizeof(uint2);
    const unsigned grid = (unsigned)((n_vec + vecs - 1) / vecs);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see griddepcontrol.* in the kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t err = cudaSuccess;
    const bool planar = a.k_kind == ROW_PLANAR || a.v_kind == ROW_PLANAR;
    // The bulk kernel wants five CTAs of 39 KiB per SM: ask for the largest shared-memory carve-out (once per
    // kernel and process; a hint, so its result is not checked).
    auto launch_bulk = [&](auto *kernel) {
        static std::atomic<bool> hinted{false};
        if (!hinted.exchange(true)) cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        return cudaLaunchKernelEx(&cfg, kernel, a);
    };
    if (!planar) {
        err = bulk ? launch_bulk(append_kernel<0, 32>) : cudaLaunchKernelEx(&cfg, append_kernel<0, 8>, a);
    } else {
        const bool ok = dispatch_bits(a.bits, [&]<int B>() {
            err = bulk ? launch_bulk(append_kernel<B, 32>) : cudaLaunchKernelEx(&cfg, append_kernel<B, 8>, a);
        });
        if (!ok) return fail(ctx, BK_ERR_INVALID, "append: bits must be 1..8");
    }
    ctx->launches++;
    BK_CUDA(ctx, err);
    BK_CUDA(ctx, cudaGetLastError());
    return BK_OK;
}

}  // namespace bk
