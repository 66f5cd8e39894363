// Fused KV append: IMROPE on K, then store K and V rows as f32, f16 or rotated Lloyd-Max
// ("planar") rows, one launch for any number of tokens.  Replaces rope_imrope.comp (k side),
// kv_store.comp, kv_store_f16.comp and kv_store_q.comp and follows the reference CPU path
// bit for bit (src/forward.rs:259-285, src/kvquant.rs:397-412, src/rope.rs:61-69).
//
// One CTA per token, one warp per (K|V, kv head) vector of 256 floats:
//   1. coalesced float4 loads into shared memory; K warps rotate pairs (j, j + n_rot/2) with
//      the (cos, sin) row of the token's position from the host-built rope table;
//   2. planar rows: lane 0 of the warp adds the 256 squares in order (the reference's f32 sum
//      is sequential, so the chain is too), the warp then scales, Givens-rotates, finds the
//      nearest centroid for its 8 coordinates per lane and writes `bits` bytes per lane;
//   3. f32/f16 rows are written with 128-bit stores.
// Traffic per token is the algorithmic minimum: 2*n_kv*1 KiB in, rows + norms out.
#include "bk_device.cuh"
#include "bk_internal.h"

namespace bk {

namespace {

constexpr int kVecPad = kHd + 4;  // floats per staged vector; +4 keeps float4 alignment

template <int BITS>
__device__ __forceinline__ void store_planar_row(const float *sx, int lane, const float *givens,
                                                 const float *sbook, uint8_t *row, float *norm_out) {
    float n = 0.f;
    if (lane == 0) n = serial_norm(sx, kHd);
    n = __shfl_sync(0xffffffffu, n, 0);
    if (lane == 0) *norm_out = n;
    const float inv = (n > 1e-12f) ? __fdiv_rn(1.0f, n) : 0.0f;
    uint64_t packed = 0;
#pragma unroll
    for (int pr = 0; pr < 4; pr++) {
        const int i = lane * 4 + pr;  // pair index: coordinates 2i, 2i+1
        const float a = __fmul_rn(sx[2 * i], inv), b = __fmul_rn(sx[2 * i + 1], inv);
        const float c = givens[2 * i], s = givens[2 * i + 1];
        float r0, r1;
        givens_fwd(a, b, c, s, r0, r1);
        const uint64_t i0 = nearest_centroid(r0, sbook, 1 << BITS);
        const uint64_t i1 = nearest_centroid(r1, sbook, 1 << BITS);
        packed |= i0 << (BITS * (2 * pr));
        packed |= i1 << (BITS * (2 * pr + 1));
    }
    store_group8<BITS>(row, lane, packed);
}

__device__ __forceinline__ void store_f32_row(const float *sx, int lane, uint8_t *row) {
    float4 *dst = reinterpret_cast<float4 *>(row);
    const float4 *src = reinterpret_cast<const float4 *>(sx);
    dst[lane] = src[lane];
    dst[lane + 32] = src[lane + 32];
}

__device__ __forceinline__ void store_f16_row(const float *sx, int lane, uint8_t *row) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t lo = f32_to_half_ref(sx[lane * 8 + 2 * i]);
        const uint32_t hi = f32_to_half_ref(sx[lane * 8 + 2 * i + 1]);
        w[i] = lo | (hi << 16);
    }
    reinterpret_cast<uint4 *>(row)[lane] = make_uint4(w[0], w[1], w[2], w[3]);
}

template <int BITS>
__global__ void __launch_bounds__(512) append_kernel(AppendArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tok = blockIdx.x;
    const int n_kv = a.n_kv;
    const bool is_v = warp >= n_kv;
    const int kv = is_v ? warp - n_kv : warp;
    float *sx = smem + warp * kVecPad;
    float *sbook = smem + 2 * n_kv * kVecPad;  // centroids, shared by the CTA

    int row_idx, pos;
    size_t seq_rows = 0;
    if (a.desc) {
        const int4 d = a.desc[tok];
        seq_rows = (size_t)d.x * a.seq_stride_rows;
        row_idx = d.y;
        pos = d.z;
    } else {
        row_idx = a.row0 + tok;
        pos = a.pos0 + tok;
    }
    if (BITS > 0) {
        for (int i = threadIdx.x; i < (1 << BITS); i += blockDim.x) sbook[i] = a.book[i];
    }
    // k and v may come from the previous kernel in the stream: with programmatic dependent launch
    // only the codebook copy above runs ahead of it.  Nothing after this kernel depends on more
    // than its completion, so dependents may be scheduled right away.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    const float *src = (is_v ? a.v : a.k) + ((size_t)tok * n_kv + kv) * kHd;
    const float4 *src4 = reinterpret_cast<const float4 *>(src);
    reinterpret_cast<float4 *>(sx)[lane] = src4[lane];
    reinterpret_cast<float4 *>(sx)[lane + 32] = src4[lane + 32];
    __syncwarp();
    if (!is_v) {
        const int half = a.n_rot >> 1;
        const float2 *cs = a.rope + (size_t)pos * half;
        for (int j = lane; j < half; j += 32) {
            float x0 = sx[j], x1 = sx[j + half];
            rope_pair(x0, x1, cs[j]);
            sx[j] = x0;
            sx[j + half] = x1;
        }
        __syncwarp();
    }
    __syncthreads();  // the codebook copy

    const size_t r = seq_rows + (size_t)row_idx * n_kv + kv;
    const int kind = is_v ? a.v_kind : a.k_kind;
    uint8_t *row = (is_v ? a.v_rows + r * a.v_row_bytes : a.k_rows + r * a.k_row_bytes);
    if (kind == ROW_F32) {
        store_f32_row(sx, lane, row);
    } else if (kind == ROW_F16) {
        store_f16_row(sx, lane, row);
    } else {
        if constexpr (BITS > 0) {
            float *norms = is_v ? a.v_norms : a.k_norms;
            store_planar_row<BITS>(sx, lane, a.givens, sbook, row, norms + r);
        }
    }
}

}  // namespace

bk_status launch_append(bk_ctx *ctx, const AppendArgs &a) {
    if (a.n_tokens <= 0) return BK_OK;
    const int threads = 32 * 2 * a.n_kv;
    if (threads > 512) return fail(ctx, BK_ERR_UNSUPPORTED, "append: n_kv > 8");
    const size_t smem = (size_t)(2 * a.n_kv * kVecPad + 256) * sizeof(float);
    // Decode launches use nearly all of the SM's shared memory; asking for the same carve-out here
    // keeps the SM from being reconfigured between the append and the decode of every layer.
    static bool carveout_set[64] = {};
    if (ctx->device >= 0 && ctx->device < 64 && !carveout_set[ctx->device]) {
        dispatch_bits(a.bits > 0 ? a.bits : 4, [&]<int B>() {
            cudaFuncSetAttribute(append_kernel<B>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        });
        cudaFuncSetAttribute(append_kernel<0>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        carveout_set[ctx->device] = true;
    }
    const bool planar = a.k_kind == ROW_PLANAR || a.v_kind == ROW_PLANAR;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)a.n_tokens);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see griddepcontrol.* in the kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t err = cudaSuccess;
    if (!planar) {
        err = cudaLaunchKernelEx(&cfg, append_kernel<0>, a);
    } else {
        const bool ok = dispatch_bits(a.bits, [&]<int B>() { err = cudaLaunchKernelEx(&cfg, append_kernel<B>, a); });
        if (!ok) return fail(ctx, BK_ERR_INVALID, "append: bits must be 1..8");
    }
    ctx->launches++;
    BK_CUDA(ctx, err);
    BK_CUDA(ctx, cudaGetLastError());
    return BK_OK;
}

}  // namespace bk
