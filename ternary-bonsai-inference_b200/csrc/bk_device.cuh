// Device helpers shared by the append, decode and kvquant kernels.
//
// Everything that decides a stored bit (rope, norm, unit, rotate, nearest, pack, f32->f16) is
// written with explicit round-to-nearest intrinsics so that no FMA contraction or reassociation
// can change a result: the stored bytes must equal the reference CPU path's
// (src/kvquant.rs:357-412, src/rope.rs:61-69, src/gguf.rs:914-944), where Rust never fuses.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace bk {

// src/gguf.rs:914-944.  Round-to-nearest-even on the 13 dropped bits, except that the
// subnormal branch shifts first (sticky bits are lost) and exponents below -10 flush to zero.
// This differs from __float2half_rn only below 2^-14, and there the reference's rule wins.
__device__ __forceinline__ uint16_t f32_to_half_ref(float v) {
    const uint32_t b = __float_as_uint(v);
    const uint32_t sign = (b >> 16) & 0x8000u;
    const int exp = (int)((b >> 23) & 0xffu);
    const uint32_t man = b & 0x7fffffu;
    if (exp == 0xff) return (uint16_t)(sign | 0x7c00u | (man != 0 ? 0x200u : 0u));
    const int e = exp - 127 + 15;
    if (e >= 0x1f) return (uint16_t)(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        const uint32_t m = (man | 0x800000u) >> (uint32_t)(1 - e);
        const uint32_t half = m >> 13, rem = m & 0x1fffu;
        const uint32_t out = half + ((rem > 0x1000u || (rem == 0x1000u && (half & 1u))) ? 1u : 0u);
        return (uint16_t)(sign | out);
    }
    const uint32_t half = ((uint32_t)e << 10) | (man >> 13), rem = man & 0x1fffu;
    const uint32_t out = (half + ((rem > 0x1000u || (rem == 0x1000u && (half & 1u))) ? 1u : 0u)) & 0xffffu;
    return (uint16_t)(sign | out);
}

// src/gguf.rs:881-911: exact widening; the hardware conversion gives the same value for every
// finite and infinite input (NaN keeps a quiet payload, which nothing on this path compares).
__device__ __forceinline__ float half_bits_to_f32(uint16_t h) {
    return __half2float(__ushort_as_half(h));
}

// src/rope.rs:61-69 for one pair.
__device__ __forceinline__ void rope_pair(float &x0, float &x1, float2 cs) {
    const float a = __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
    const float b = __fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x));
    x0 = a;
    x1 = b;
}

// src/kvquant.rs:379-380 / 391-392 for one pair.
__device__ __forceinline__ void givens_fwd(float a, float b, float c, float s, float &o0, float &o1) {
    o0 = __fsub_rn(__fmul_rn(c, a), __fmul_rn(s, b));
    o1 = __fadd_rn(__fmul_rn(s, a), __fmul_rn(c, b));
}
__device__ __forceinline__ void givens_inv(float a, float b, float c, float s, float &o0, float &o1) {
    o0 = __fadd_rn(__fmul_rn(c, a), __fmul_rn(s, b));
    o1 = __fadd_rn(__fmul_rn(-s, a), __fmul_rn(c, b));
}

// src/kvquant.rs:357-370: ascending scan, strict '<', ties keep the lower index.
__device__ __forceinline__ uint32_t nearest_centroid(float v, const float *book, int n_levels) {
    uint32_t best = 0;
    float bd = fabsf(__fsub_rn(v, book[0]));
    for (int i = 1; i < n_levels; i++) {
        const float d = fabsf(__fsub_rn(v, book[i]));
        if (d < bd) {
            bd = d;
            best = (uint32_t)i;
        }
    }
    return best;
}

// The same index as nearest_centroid() in BITS + 2 steps instead of 2^BITS.  f32 subtraction is
// monotone, so along the ascending codebook |v - c_i| falls, then rises: the scan's answer is
// the last centroid <= v or its right neighbour, the left one on a tie (strict '<').  A plateau
// (equal rounded distances to two centroids on the same side) would need two centroids closer
// than an ulp of v; the context checks at creation that every codebook's gaps are above 1e-5,
// and rotated unit coordinates are below 2 in magnitude.  Non-finite v takes the scan.
template <int BITS>
__device__ __forceinline__ uint32_t nearest_centroid_fast(float v, const float *book) {
    if (!(fabsf(v) < 4.0f)) return nearest_centroid(v, book, 1 << BITS);
    int lo = 0;
#pragma unroll
    for (int step = 1 << (BITS - 1); step >= 1; step >>= 1)
        if (book[lo + step] <= v) lo += step;
    const int hi = min(lo + 1, (1 << BITS) - 1);
    const float d0 = fabsf(__fsub_rn(v, book[lo])), d1 = fabsf(__fsub_rn(v, book[hi]));
    return (uint32_t)((d1 < d0) ? hi : lo);
}

// The same index once more, for codebooks of up to 16 centroids, from ONE 8-byte read.  Along the ascending codebook the scan's answer is the number of
// thresholds T_i <= v, where T_i is the smallest float for which centroid i + 1 beats centroid i in the scan's
// own arithmetic (|v - c_{i+1}| < |v - c_i|, both differences rounded to f32; the predicate is monotone in v
// because f32 subtraction is).  The host finds every T_i by bisection over the floats, with the same rounded
// operations, and lays them out in 512 cells of width 2^-10 over [-0.25, 0.25) (clamped): cell k holds how many
// thresholds lie in lower cells and the one threshold inside it (+inf if none; the host checks that no cell
// holds two).  tab[cell] = (count, threshold bits).  Non-finite and huge v take the scan.
template <int BITS>
__device__ __forceinline__ uint32_t nearest_centroid_thr(float v, const float *book, const uint2 *tab) {
    static_assert(BITS <= 4, "the cell table covers codebooks of up to 16 centroids");
    if (!(fabsf(v) < 4.0f)) return nearest_centroid(v, book, 1 << BITS);
    const int cell = min(max(__float2int_rd(__fmul_rn(__fadd_rn(v, 0.25f), 1024.0f)), 0), 511);
    const uint2 e = tab[cell];
    return e.x + (v >= __uint_as_float(e.y) ? 1u : 0u);
}

// src/kvquant.rs:398: sequential f32 sum of squares then sqrt; 256 dependent adds by design.
__device__ __forceinline__ float serial_norm(const float *x, int n) {
    float acc = 0.0f;
#pragma unroll 16
    for (int i = 0; i < n; i++) acc = __fadd_rn(acc, __fmul_rn(x[i], x[i]));
    return __fsqrt_rn(acc);
}

// src/kernels.rs:112-116 (rms_norm_rows): sequential f32 sum of squares, then
// 1 / sqrt(ss / n + eps); the row is then (x * scale) * w, two roundings, left to right (:118).
__device__ __forceinline__ float rms_scale_ref(const float *x, int n, float eps) {
    float ss = 0.0f;
#pragma unroll 16
    for (int i = 0; i < n; i++) ss = __fadd_rn(ss, __fmul_rn(x[i], x[i]));
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)n), eps)));
}

// The `bits`-wide little-endian field stream of src/kvquant.rs:152-165 (for hd = 256 every
// pack_idx branch of the reference produces exactly this stream): 8 consecutive indices of a
// row occupy `bits` whole bytes starting at byte (first_index/8)*bits.
template <int BITS>
__device__ __forceinline__ uint64_t load_group8(const uint8_t *row, int group) {
    const uint8_t *p = row + group * BITS;
    if constexpr (BITS == 8) {
        const uint2 w = *reinterpret_cast<const uint2 *>(p);
        return ((uint64_t)w.y << 32) | w.x;
    } else if constexpr (BITS == 4) {
        return *reinterpret_cast<const uint32_t *>(p);
    } else if constexpr (BITS == 2) {
        return *reinterpret_cast<const uint16_t *>(p);
    } else if constexpr (BITS == 1) {
        return *p;
    } else {
        uint64_t v = 0;
#pragma unroll
        for (int i = 0; i < BITS; i++) v |= (uint64_t)p[i] << (8 * i);
        return v;
    }
}

template <int BITS>
__device__ __forceinline__ void store_group8(uint8_t *row, int group, uint64_t v) {
    uint8_t *p = row + group * BITS;
    if constexpr (BITS == 8) {
        *reinterpret_cast<uint2 *>(p) = make_uint2((uint32_t)v, (uint32_t)(v >> 32));
    } else if constexpr (BITS == 4) {
        *reinterpret_cast<uint32_t *>(p) = (uint32_t)v;
    } else if constexpr (BITS == 2) {
        *reinterpret_cast<uint16_t *>(p) = (uint16_t)v;
    } else if constexpr (BITS == 1) {
        *p = (uint8_t)v;
    } else {
#pragma unroll
        for (int i = 0; i < BITS; i++) p[i] = (uint8_t)(v >> (8 * i));
    }
}

// Run f.template operator()<BITS>() for a run-time width 1..8.
template <typename F>
__host__ inline bool dispatch_bits(int bits, F &&f) {
    switch (bits) {
        case 1: f.template operator()<1>(); return true;
        case 2: f.template operator()<2>(); return true;
        case 3: f.template operator()<3>(); return true;
        case 4: f.template operator()<4>(); return true;
        case 5: f.template operator()<5>(); return true;
        case 6: f.template operator()<6>(); return true;
        case 7: f.template operator()<7>(); return true;
        case 8: f.template operator()<8>(); return true;
        default: return false;
    }
}

}  // namespace bk
