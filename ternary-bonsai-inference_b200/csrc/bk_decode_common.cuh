// Tail shared by the decode kernels: merge the split-K chunks of one (sequence, kv head) and
// write the result.  A CTA that has reduced its chunk to (acc[NREP][256], M[NREP], L[NREP]) in
// shared memory (acc relative to M, exp2 domain) calls finish_item():
//   * more than one chunk: the CTA stores its triple in the partials buffer, takes a ticket
//     from the (sequence, kv head) counter and returns unless it is the last to arrive; the
//     last one re-reads every chunk's triple and combines them.  Nobody waits for anybody.
//   * planar V: the combined accumulator is still in Givens-rotated space and is rotated back
//     once here (src/forward.rs:349, shaders/attn_out_q.comp:85-91);
//   * output: acc / L, or the unnormalised (acc, m, l) triple when the caller merges chunks
//     held by other caches / GPUs itself.
#pragma once

#include <math_constants.h>

#include "bk_device.cuh"
#include "bk_internal.h"

namespace bk {

template <int NREP>
__device__ __forceinline__ void finish_item(const DecodeArgs &a, int s, int kv, int item, int n_chunks,
                                            int first_item, float *s_acc /* [NREP][kHd] */, float *s_M, float *s_L,
                                            int *s_last, bool v_planar) {
    const int tid = threadIdx.x, nt = blockDim.x;
    if (n_chunks > 1) {
        float *part = a.partials + ((size_t)item * NREP) * kPartStride;
        for (int i = tid; i < NREP * kHd; i += nt) {
            const int r = i / kHd, d = i - r * kHd;
            part[(size_t)r * kPartStride + d] = s_acc[i];
        }
        if (tid < NREP) {
            part[(size_t)tid * kPartStride + kHd] = s_M[tid];
            part[(size_t)tid * kPartStride + kHd + 1] = s_L[tid];
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned ticket = atomicAdd(&a.counters[s * a.n_kv + kv], 1u);
            *s_last = (ticket == (unsigned)(n_chunks - 1));
        }
        __syncthreads();
        if (!*s_last) return;
        __threadfence();
        const float *base = a.partials + (size_t)first_item * NREP * kPartStride;
        if (tid < NREP) {
            float M = -CUDART_INF_F;
            for (int c = 0; c < n_chunks; c++)
                M = fmaxf(M, __ldcg(base + ((size_t)c * NREP + tid) * kPartStride + kHd));
            float Lsum = 0.f;
            for (int c = 0; c < n_chunks; c++) {
                const float *pc = base + ((size_t)c * NREP + tid) * kPartStride;
                const float mc = __ldcg(pc + kHd);
                if (mc > -CUDART_INF_F) Lsum += __ldcg(pc + kHd + 1) * exp2f(mc - M);
            }
            s_M[tid] = M;
            s_L[tid] = Lsum;
        }
        __syncthreads();
        for (int i = tid; i < NREP * kHd; i += nt) {
            const int r = i / kHd, d = i - r * kHd;
            const float M = s_M[r];
            float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
            int c = 0;
            for (; c + 4 <= n_chunks; c += 4) {  // four independent loads in flight per thread
                const float *p0 = base + ((size_t)c * NREP + r) * kPartStride;
                const float *p1 = p0 + (size_t)NREP * kPartStride, *p2 = p1 + (size_t)NREP * kPartStride,
                            *p3 = p2 + (size_t)NREP * kPartStride;
                const float v0 = __ldcg(p0 + d), v1 = __ldcg(p1 + d), v2 = __ldcg(p2 + d), v3 = __ldcg(p3 + d);
                const float m0 = __ldcg(p0 + kHd), m1 = __ldcg(p1 + kHd), m2 = __ldcg(p2 + kHd), m3 = __ldcg(p3 + kHd);
                sum0 = fmaf(v0, m0 > -CUDART_INF_F ? exp2f(m0 - M) : 0.f, sum0);
                sum1 = fmaf(v1, m1 > -CUDART_INF_F ? exp2f(m1 - M) : 0.f, sum1);
                sum2 = fmaf(v2, m2 > -CUDART_INF_F ? exp2f(m2 - M) : 0.f, sum2);
                sum3 = fmaf(v3, m3 > -CUDART_INF_F ? exp2f(m3 - M) : 0.f, sum3);
            }
            for (; c < n_chunks; c++) {
                const float *pc = base + ((size_t)c * NREP + r) * kPartStride;
                const float mc = __ldcg(pc + kHd);
                sum0 = fmaf(__ldcg(pc + d), mc > -CUDART_INF_F ? exp2f(mc - M) : 0.f, sum0);
            }
            s_acc[i] = (sum0 + sum1) + (sum2 + sum3);
        }
        if (tid == 0) a.counters[s * a.n_kv + kv] = 0;  // ready for the next launch
        __syncthreads();
    }

    if (v_planar) {
        for (int i = tid; i < NREP * (kHd / 2); i += nt) {
            const int r = i / (kHd / 2), pr = i - r * (kHd / 2);
            float o0, o1;
            givens_inv(s_acc[r * kHd + 2 * pr], s_acc[r * kHd + 2 * pr + 1], a.givens[2 * pr], a.givens[2 * pr + 1],
                       o0, o1);
            s_acc[r * kHd + 2 * pr] = o0;
            s_acc[r * kHd + 2 * pr + 1] = o1;
        }
        __syncthreads();
    }
    if (a.partial) {
        float *out = a.out + ((size_t)s * a.n_head + (size_t)kv * NREP) * kPartStride;
        for (int i = tid; i < NREP * kHd; i += nt) {
            const int r = i / kHd, d = i - r * kHd;
            out[(size_t)r * kPartStride + d] = s_acc[i];
        }
        if (tid < NREP) {
            out[(size_t)tid * kPartStride + kHd] = s_M[tid] * 0.6931471805599453f;  // log2 -> ln
            out[(size_t)tid * kPartStride + kHd + 1] = s_L[tid];
        }
    } else {
        float *out = a.out + ((size_t)s * a.n_head + (size_t)kv * NREP) * kHd;
        for (int i = tid; i < NREP * kHd; i += nt) {
            const float Ls = s_L[i / kHd];
            out[i] = Ls > 0.f ? s_acc[i] / Ls : 0.f;
        }
    }
}

}  // namespace bk
