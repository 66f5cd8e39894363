// Per-head RMSNorm rows (src/kernels.rs:97-122), bit for bit: the sum of squares runs in the
// reference's order, one lane per row walking a shared-memory copy of the row, and the row
// leaves as (x * scale) * w.  Used by bk_rms_norm_rows and, on caches that do not take the
// tensor-core decode path, by the layer form of the attention step for q (24 rows out of the
// interleaved [q | gate] projection output) and k (4 rows) in one launch; the tensor-core
// kernels do the same arithmetic themselves.
#include "bk_device.cuh"
#include "bk_internal.h"

namespace bk {

namespace {

constexpr int kWarps = 8;

__global__ void __launch_bounds__(kWarps * 32) rms_norm_rows_kernel(NormSeg s0, NormSeg s1, int row_len, float eps) {
    extern __shared__ float s_rows[];  // [kWarps][row_len]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int row = blockIdx.x * kWarps + warp;
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    if (row >= s0.n_rows + s1.n_rows) return;
    const NormSeg &sg = row < s0.n_rows ? s0 : s1;
    if (row >= s0.n_rows) row -= s0.n_rows;
    const float *src = sg.src + (size_t)row * sg.stride;
    float *sx = s_rows + (size_t)warp * row_len;
    for (int i = lane; i < row_len; i += 32) sx[i] = src[i];
    __syncwarp();
    float sc = 0.f;
    if (lane == 0) sc = rms_scale_ref(sx, row_len, eps);
    sc = __shfl_sync(0xffffffffu, sc, 0);
    float *dst = sg.dst + (size_t)row * row_len;
    for (int i = lane; i < row_len; i += 32) dst[i] = __fmul_rn(__fmul_rn(sx[i], sc), sg.w[i]);
}

}  // namespace

bk_status launch_rms_norm_rows(bk_ctx *ctx, const NormSeg &s0, const NormSeg &s1, int row_len, float eps) {
    const int n_rows = s0.n_rows + s1.n_rows;
    if (n_rows <= 0) return BK_OK;
    if (row_len < 1 || row_len > 1024) return fail(ctx, BK_ERR_UNSUPPORTED, "rms_norm_rows: row_len must be 1..1024");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((n_rows + kWarps - 1) / kWarps));
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = (size_t)kWarps * row_len * sizeof(float);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BK_CUDA(ctx, cudaLaunchKernelEx(&cfg, rms_norm_rows_kernel, s0, s1, row_len, eps));
    ctx->launches++;
    BK_CUDA(ctx, cudaGetLastError());
    return BK_OK;
}

}  // namespace bk
