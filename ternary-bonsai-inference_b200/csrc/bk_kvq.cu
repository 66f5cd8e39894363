// GPU versions of the kvquant.rs / rope.rs / gguf.rs entry points, used for parity checks of
// the encode/decode format outside a cache.  Each mirrors one reference function and follows
// its f32 operation order, so results equal the reference CPU path bit for bit.
#include "bk_device.cuh"
#include "bk_internal.h"

namespace bk {

namespace {

// PlanarQuant::quantize, src/kvquant.rs:397-412.  One warp per vector.
template <int BITS>
__global__ void quantize_kernel(int n_vec, const float *x, const float *givens, const float *book, const uint2 *cell_tab,
                                uint8_t *packed, float *norms) {
    __shared__ __align__(16) float sx[4][kHd];
    __shared__ float sbook[256];
    __shared__ __align__(16) uint2 tab[BITS <= 4 ? 512 : 1];  // the cells of the one-read centroid search (up to 16 centroids)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int vec = blockIdx.x * 4 + warp;
    for (int i = threadIdx.x; i < (1 << BITS); i += blockDim.x) sbook[i] = book[i];
    if constexpr (BITS <= 4)
        for (int i = threadIdx.x; i < 512; i += blockDim.x) tab[i] = cell_tab[i];
    if (vec < n_vec) {
        const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)vec * kHd);
        reinterpret_cast<float4 *>(sx[warp])[lane] = src[lane];
        reinterpret_cast<float4 *>(sx[warp])[lane + 32] = src[lane + 32];
    }
    __syncthreads();
    if (vec >= n_vec) return;
    float n = 0.f;
    if (lane == 0) n = serial_norm(sx[warp], kHd);
    n = __shfl_sync(0xffffffffu, n, 0);
    if (lane == 0) norms[vec] = n;
    const float inv = (n > 1e-12f) ? __fdiv_rn(1.0f, n) : 0.0f;
    uint64_t word = 0;
#pragma unroll
    for (int pr = 0; pr < 4; pr++) {
        const int i = lane * 4 + pr;
        float r0, r1;
        givens_fwd(__fmul_rn(sx[warp][2 * i], inv), __fmul_rn(sx[warp][2 * i + 1], inv), givens[2 * i],
                   givens[2 * i + 1], r0, r1);
        if constexpr (BITS <= 4) {  // the search the bulk append uses
            word |= (uint64_t)nearest_centroid_thr<BITS>(r0, sbook, tab) << (BITS * (2 * pr));
            word |= (uint64_t)nearest_centroid_thr<BITS>(r1, sbook, tab) << (BITS * (2 * pr + 1));
        } else {
            word |= (uint64_t)nearest_centroid_fast<BITS>(r0, sbook) << (BITS * (2 * pr));
            word |= (uint64_t)nearest_centroid_fast<BITS>(r1, sbook) << (BITS * (2 * pr + 1));
        }
    }
    store_group8<BITS>(packed + (size_t)vec * 32 * BITS, lane, word);
}

// PlanarQuant::dequantize, src/kvquant.rs:415-428.  One thread per pair.
template <int BITS>
__global__ void dequantize_kernel(int n_vec, const uint8_t *packed, const float *norms, const float *givens,
                                  const float *book, float *out) {
    const int vec = blockIdx.x, pr = threadIdx.x;  // 128 threads
    const uint8_t *row = packed + (size_t)vec * 32 * BITS;
    const uint64_t g = load_group8<BITS>(row, pr >> 2);
    const int e = (pr & 3) * 2;
    const uint32_t mask = (1u << BITS) - 1u;
    const float a = book[(uint32_t)(g >> (BITS * e)) & mask];
    const float b = book[(uint32_t)(g >> (BITS * (e + 1))) & mask];
    float o0, o1;
    givens_inv(a, b, givens[2 * pr], givens[2 * pr + 1], o0, o1);
    const float n = norms[vec];
    out[(size_t)vec * kHd + 2 * pr] = __fmul_rn(o0, n);
    out[(size_t)vec * kHd + 2 * pr + 1] = __fmul_rn(o1, n);
}

// PlanarQuant::rotate / rotate_inv, src/kvquant.rs:373-394.
__global__ void rotate_kernel(int inverse, const float *x, const float *givens, float *out) {
    const int vec = blockIdx.x, pr = threadIdx.x;
    const float a = x[(size_t)vec * kHd + 2 * pr], b = x[(size_t)vec * kHd + 2 * pr + 1];
    float o0, o1;
    if (inverse) givens_inv(a, b, givens[2 * pr], givens[2 * pr + 1], o0, o1);
    else givens_fwd(a, b, givens[2 * pr], givens[2 * pr + 1], o0, o1);
    out[(size_t)vec * kHd + 2 * pr] = o0;
    out[(size_t)vec * kHd + 2 * pr + 1] = o1;
}

// PlanarQuant::dot_rotated_scratch, src/kvquant.rs:463-477: sequential f32 accumulation, so one
// thread walks a row (this is a parity entry point; the decode kernel is the fast path).
template <int BITS>
__global__ void dot_rotated_kernel(int n_vec, const float *q_rot, const uint8_t *packed, const float *norms,
                                   const float *book, float *out) {
    const int vec = blockIdx.x * blockDim.x + threadIdx.x;
    if (vec >= n_vec) return;
    const uint8_t *row = packed + (size_t)vec * 32 * BITS;
    const float *q = q_rot + (size_t)vec * kHd;
    const uint32_t mask = (1u << BITS) - 1u;
    float acc = 0.f;
    for (int g = 0; g < 32; g++) {
        const uint64_t w = load_group8<BITS>(row, g);
#pragma unroll
        for (int e = 0; e < 8; e++)
            acc = __fadd_rn(acc, __fmul_rn(q[g * 8 + e], book[(uint32_t)(w >> (BITS * e)) & mask]));
    }
    out[vec] = __fmul_rn(acc, norms[vec]);
}

// rope_imrope, src/rope.rs:9-70, for arbitrary (t, h, w, e) ids: pair j takes row band[j].
__global__ void rope_kernel(int hd, float *heads, const float2 *rows4, int n_dims, const int *band) {
    const int half = n_dims >> 1;
    float *h = heads + (size_t)blockIdx.x * hd;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float x0 = h[j], x1 = h[j + half];
        rope_pair(x0, x1, rows4[band[j] * half + j]);
        h[j] = x0;
        h[j + half] = x1;
    }
}

__global__ void f32_to_half_kernel(size_t n, const float *in, uint16_t *out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f32_to_half_ref(in[i]);
}
__global__ void half_to_f32_kernel(size_t n, const uint16_t *in, float *out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = half_bits_to_f32(in[i]);
}

}  // namespace

#define BK_LAUNCH_DONE(ctx)               \
    do {                                  \
        (ctx)->launches++;                \
        BK_CUDA((ctx), cudaGetLastError()); \
        return BK_OK;                     \
    } while (0)

bk_status launch_quantize(bk_ctx *ctx, int bits, int n_vec, const float *x, uint8_t *packed, float *norms) {
    if (n_vec <= 0) return BK_OK;
    const float *book = ctx->d_codebooks + (bits - 1) * kBookStride;
    if (!dispatch_bits(bits, [&]<int B>() {
            quantize_kernel<B><<<(n_vec + 3) / 4, 128, 0, ctx->stream>>>(n_vec, x, ctx->d_givens, book,
                                                                         B <= 4 ? ctx->d_cell_tabs + (B - 1) * 512 : nullptr, packed, norms);
        }))
        return fail(ctx, BK_ERR_INVALID, "bits must be 1..8");
    BK_LAUNCH_DONE(ctx);
}

bk_status launch_dequantize(bk_ctx *ctx, int bits, int n_vec, const uint8_t *packed, const float *norms,
                            float *out) {
    if (n_vec <= 0) return BK_OK;
    const float *book = ctx->d_codebooks + (bits - 1) * kBookStride;
    if (!dispatch_bits(bits, [&]<int B>() {
            dequantize_kernel<B><<<n_vec, 128, 0, ctx->stream>>>(n_vec, packed, norms, ctx->d_givens, book, out);
        }))
        return fail(ctx, BK_ERR_INVALID, "bits must be 1..8");
    BK_LAUNCH_DONE(ctx);
}

bk_status launch_rotate(bk_ctx *ctx, int n_vec, int inverse, const float *x, float *out) {
    if (n_vec <= 0) return BK_OK;
    rotate_kernel<<<n_vec, 128, 0, ctx->stream>>>(inverse, x, ctx->d_givens, out);
    BK_LAUNCH_DONE(ctx);
}

bk_status launch_dot_rotated(bk_ctx *ctx, int bits, int n_vec, const float *q_rot, const uint8_t *packed,
                             const float *norms, float *out) {
    if (n_vec <= 0) return BK_OK;
    const float *book = ctx->d_codebooks + (bits - 1) * kBookStride;
    if (!dispatch_bits(bits, [&]<int B>() {
            dot_rotated_kernel<B><<<(n_vec + 63) / 64, 64, 0, ctx->stream>>>(n_vec, q_rot, packed, norms, book, out);
        }))
        return fail(ctx, BK_ERR_INVALID, "bits must be 1..8");
    BK_LAUNCH_DONE(ctx);
}

bk_status launch_rope(bk_ctx *ctx, int n_heads, int hd, float *heads, const float2 *rows4, int n_dims,
                      const int *band) {
    if (n_heads <= 0) return BK_OK;
    rope_kernel<<<n_heads, 64, 0, ctx->stream>>>(hd, heads, rows4, n_dims, band);
    BK_LAUNCH_DONE(ctx);
}

bk_status launch_f32_to_half(bk_ctx *ctx, size_t n, const float *in, uint16_t *out) {
    if (n == 0) return BK_OK;
    f32_to_half_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(n, in, out);
    BK_LAUNCH_DONE(ctx);
}

bk_status launch_half_to_f32(bk_ctx *ctx, size_t n, const uint16_t *in, float *out) {
    if (n == 0) return BK_OK;
    half_to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(n, in, out);
    BK_LAUNCH_DONE(ctx);
}

}  // namespace bk
