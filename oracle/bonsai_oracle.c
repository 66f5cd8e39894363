/*
 * CPU oracle for the KV-cache path of herlangga72/ternary-bonsai-inference.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * reference's own single-threaded Rust CPU path (append + GQA decode
 * attention of the qwen35 full-attention layers).  It is the checker for the
 * CUDA library and the timed CPU baseline of the benchmark; the shipped
 * library never links, loads or calls it.
 *
 * Build flags that keep Rust's f32 semantics: -O2 -ffp-contract=off, no
 * fast-math (Rust neither fuses a*b+c nor reassociates float sums).  Every
 * `f32` of the reference is a `float` here, every `f64` a `double`, loops run
 * in the reference's order.  Transcendentals are the host libm's
 * (powf/cosf/sinf/expf/exp/cos/sin/sqrt), as they are for the Rust build.
 *
 * Pin status: the reference holds no golden byte vectors for this path.  Its
 * unit tests hold known answers for the f16 conversions, the mode parser, the
 * 3-bit pack layout, the softmax and the cache layout, and properties for the
 * codebook, the Givens table and the quantizer round trip; tests/ re-runs all
 * of those against this file.  Beyond them the bit pattern of quantized rows
 * is pinned only by a second, independent Python restatement
 * (tests/golden/gen_golden.py) that must agree with this file bit for bit:
 * "parity unpinned" against a running reference, because no Rust toolchain
 * exists on the build or test machines.
 *
 * Each function cites the reference lines it follows (paths inside the
 * reference project).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

#define OR_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* Lloyd-Max codebook: src/kvquant.rs:34-114                                */
/* ------------------------------------------------------------------------ */

/* src/kvquant.rs:34-44 (Abramowitz & Stegun 7.1.26) */
static double or_erf(double x) {
    double sign = (x < 0.0) ? -1.0 : 1.0;
    x = fabs(x);
    double t = 1.0 / (1.0 + 0.3275911 * x);
    double poly = ((((1.061405429 * t - 1.453152027) * t) + 1.421413741) * t - 0.284496736) * t
                  + 0.254829592;
    double y = 1.0 - poly * t * exp(-x * x);
    return sign * y;
}

/* src/kvquant.rs:46-48 */
static double or_norm_cdf(double x, double sigma) {
    return 0.5 * (1.0 + or_erf(x / (sigma * 1.4142135623730951)));
}

/* src/kvquant.rs:50-52 */
static double or_norm_pdf(double x, double sigma) {
    return exp(-(x * x) / (2.0 * sigma * sigma)) / (sigma * sqrt(2.0 * 3.14159265358979323846));
}

/* src/kvquant.rs:56-58 */
static double or_gauss_first_moment(double a, double b, double sigma) {
    return sigma * sigma * (or_norm_pdf(a, sigma) - or_norm_pdf(b, sigma));
}

/* src/kvquant.rs:62-99.  Writes 2^bits ascending centroids; returns the
 * number of iterations run (the 300 cap is part of the format: widths 4..8
 * never meet the 1e-12 exit). */
OR_API int or_solve_lloyd_max(double sigma, unsigned bits, float *out) {
    size_t n = (size_t)1 << bits;
    double lo = -3.5 * sigma, hi = 3.5 * sigma;
    double *c = malloc(n * sizeof(double));
    double *next = malloc(n * sizeof(double));
    double *edges = malloc((n + 1) * sizeof(double));
    for (size_t i = 0; i < n; i++) c[i] = lo + (hi - lo) * ((double)i + 0.5) / (double)n;
    double outer = 12.0 * sigma;
    int iters = 0;
    for (int it = 0; it < 300; it++) {
        iters++;
        edges[0] = -outer;
        for (size_t i = 0; i + 1 < n; i++) edges[i + 1] = (c[i] + c[i + 1]) / 2.0;
        edges[n] = outer;
        for (size_t i = 0; i < n; i++) {
            double a = edges[i], b = edges[i + 1];
            double mass = or_norm_cdf(b, sigma) - or_norm_cdf(a, sigma);
            if (mass > 1e-15) next[i] = or_gauss_first_moment(a, b, sigma) / mass;
            else next[i] = c[i];
        }
        double shift = 0.0;
        for (size_t i = 0; i < n; i++) {
            double d = fabs(next[i] - c[i]);
            if (d > shift) shift = d; /* f64::max fold from 0.0 */
        }
        memcpy(c, next, n * sizeof(double));
        if (shift < 1e-12) break;
    }
    for (size_t i = 0; i < n; i++) out[i] = (float)c[i];
    free(c); free(next); free(edges);
    return iters;
}

/* src/kvquant.rs:103-114: sigma = 1/sqrt(d), one book per width 1..8. */
OR_API void or_codebook(size_t d, unsigned bits, float *out) {
    double sigma = 1.0 / sqrt((double)d);
    or_solve_lloyd_max(sigma, bits, out);
}

/* src/kvquant.rs:856-880 (diagnostic used by the reference's distortion test) */
OR_API float or_expected_distortion(size_t d, unsigned bits) {
    double sigma = 1.0 / sqrt((double)d);
    size_t n = (size_t)1 << bits;
    float *c = malloc(n * sizeof(float));
    double *edges = malloc((n + 1) * sizeof(double));
    or_codebook(d, bits, c);
    double outer = 12.0 * sigma;
    edges[0] = -outer;
    for (size_t i = 0; i + 1 < n; i++) edges[i + 1] = ((double)c[i] + (double)c[i + 1]) / 2.0;
    edges[n] = outer;
    double dist = 0.0;
    for (size_t i = 0; i < n; i++) {
        double a = edges[i], b = edges[i + 1], c0 = (double)c[i];
        double mass = or_norm_cdf(b, sigma) - or_norm_cdf(a, sigma);
        double m1 = or_gauss_first_moment(a, b, sigma);
        double m2 = sigma * sigma * (mass + a * or_norm_pdf(a, sigma) - b * or_norm_pdf(b, sigma));
        dist += m2 - 2.0 * c0 * m1 + c0 * c0 * mass;
    }
    free(c); free(edges);
    return (float)dist;
}

/* ------------------------------------------------------------------------ */
/* Givens table: src/kvquant.rs:120-145                                     */
/* ------------------------------------------------------------------------ */

/* src/kvquant.rs:120-126 */
OR_API uint64_t or_splitmix64(uint64_t *state) {
    *state += 0x9E3779B97F4A7C15ULL;
    uint64_t z = *state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

/* src/kvquant.rs:131-145: out holds ceil(d/2) (cos, sin) pairs, interleaved. */
OR_API void or_givens_table(size_t d, float *out) {
    size_t n_groups = (d + 1) / 2;
    uint64_t state = 42;
    for (size_t g = 0; g < n_groups; g++) {
        uint64_t r = or_splitmix64(&state);
        double u = (double)(r >> 11) / (double)((uint64_t)1 << 53);
        double t = u * 6.283185307179586;
        out[2 * g] = (float)cos(t);
        out[2 * g + 1] = (float)sin(t);
    }
}

/* ------------------------------------------------------------------------ */
/* Bit packing: src/kvquant.rs:152-319                                      */
/* ------------------------------------------------------------------------ */

/* src/kvquant.rs:184-186 */
OR_API size_t or_packed_bytes(size_t n, unsigned bits) { return (n * bits + 7) / 8; }

/* src/kvquant.rs:152-165 */
OR_API void or_pack_bits(const uint8_t *idx, size_t n, unsigned bits, uint8_t *out) {
    memset(out, 0, or_packed_bytes(n, bits));
    size_t bitpos = 0;
    for (size_t k = 0; k < n; k++) {
        size_t byte = bitpos >> 3;
        unsigned off = (unsigned)(bitpos & 7);
        uint32_t v = (uint32_t)idx[k] & ((1u << bits) - 1);
        out[byte] |= (uint8_t)((v << off) & 0xff);
        if (off + bits > 8) out[byte + 1] |= (uint8_t)(v >> (8 - off));
        bitpos += bits;
    }
}

/* src/kvquant.rs:168-181 */
OR_API void or_unpack_bits(const uint8_t *packed, unsigned bits, size_t n, uint8_t *out) {
    uint32_t mask = (1u << bits) - 1;
    size_t bitpos = 0;
    for (size_t k = 0; k < n; k++) {
        size_t byte = bitpos >> 3;
        unsigned off = (unsigned)(bitpos & 7);
        uint32_t v = (uint32_t)packed[byte] >> off;
        if (off + bits > 8) v |= (uint32_t)packed[byte + 1] << (8 - off);
        out[k] = (uint8_t)(v & mask);
        bitpos += bits;
    }
}

/* src/kvquant.rs:191-202 */
static void or_pack_groups3(const uint8_t *idx, size_t n, uint8_t *out) {
    size_t groups = n / 8;
    for (size_t g = 0; g < groups; g++) {
        uint32_t v = 0;
        for (int k = 0; k < 8; k++) v |= ((uint32_t)idx[g * 8 + k] & 0x7) << (3 * k);
        out[3 * g] = (uint8_t)v;
        out[3 * g + 1] = (uint8_t)(v >> 8);
        out[3 * g + 2] = (uint8_t)(v >> 16);
    }
}

/* src/kvquant.rs:205-215 */
static void or_unpack_groups3(const uint8_t *packed, size_t n, uint8_t *out) {
    size_t groups = n / 8;
    for (size_t g = 0; g < groups; g++) {
        uint32_t v = (uint32_t)packed[3 * g] | (uint32_t)packed[3 * g + 1] << 8
                     | (uint32_t)packed[3 * g + 2] << 16;
        for (int k = 0; k < 8; k++) out[g * 8 + k] = (uint8_t)((v >> (3 * k)) & 0x7);
    }
}

/* src/kvquant.rs:221-236: single-plane layouts for widths 1, 2, 4 only.
 * Returns the plane's field width (== bits) and byte count, or 0. */
static unsigned or_plane_layout(size_t n, unsigned bits, size_t *plane_bytes) {
    size_t total = or_packed_bytes(n, bits);
    size_t pb;
    switch (bits) {
        case 1: pb = (n + 7) / 8; break;
        case 2: pb = (n + 3) / 4; break;
        case 4: pb = (n + 1) / 2; break;
        default: return 0;
    }
    if (pb > total) return 0;
    *plane_bytes = pb;
    return bits;
}

/* src/kvquant.rs:267-291 */
static void or_pack_planes(const uint8_t *idx, size_t n, unsigned bits, uint8_t *out) {
    size_t pbytes;
    unsigned fb = or_plane_layout(n, bits, &pbytes);
    if (!fb) { or_pack_bits(idx, n, bits, out); return; }
    memset(out, 0, or_packed_bytes(n, bits));
    size_t poff = 0;
    unsigned fshift = 0;
    /* the layout vector of the reference has exactly one (field, bytes) entry */
    uint32_t mask = (1u << fb) - 1;
    size_t cpb = 8 / fb;
    for (size_t b = 0; b < pbytes; b++) {
        uint32_t byte = 0;
        for (size_t k = 0; k < cpb; k++) {
            size_t i = b * cpb + k;
            if (i >= n) break;
            byte |= (((uint32_t)idx[i] >> fshift) & mask) << (fb * (unsigned)k);
        }
        out[poff + b] = (uint8_t)byte;
    }
}

/* src/kvquant.rs:294-319 */
static void or_unpack_planes(const uint8_t *packed, size_t n, unsigned bits, uint8_t *out) {
    size_t pbytes;
    unsigned fb = or_plane_layout(n, bits, &pbytes);
    if (!fb) { or_unpack_bits(packed, bits, n, out); return; }
    memset(out, 0, n);
    size_t poff = 0;
    unsigned fshift = 0;
    uint32_t mask = (1u << fb) - 1;
    size_t cpb = 8 / fb;
    for (size_t b = 0; b < pbytes; b++) {
        uint32_t byte = packed[poff + b];
        for (size_t k = 0; k < cpb; k++) {
            size_t i = b * cpb + k;
            if (i >= n) break;
            out[i] |= (uint8_t)(((byte >> (fb * (unsigned)k)) & mask) << fshift);
        }
    }
}

/* src/kvquant.rs:241-249 */
OR_API void or_pack_idx(const uint8_t *idx, size_t n, unsigned bits, uint8_t *out) {
    size_t pb;
    if (bits == 3 && n % 8 == 0) or_pack_groups3(idx, n, out);
    else if (or_plane_layout(n, bits, &pb)) or_pack_planes(idx, n, bits, out);
    else or_pack_bits(idx, n, bits, out);
}

/* src/kvquant.rs:252-260 */
OR_API void or_unpack_idx(const uint8_t *packed, size_t n, unsigned bits, uint8_t *out) {
    size_t pb;
    if (bits == 3 && n % 8 == 0) or_unpack_groups3(packed, n, out);
    else if (or_plane_layout(n, bits, &pb)) or_unpack_planes(packed, n, bits, out);
    else or_unpack_bits(packed, bits, n, out);
}

/* ------------------------------------------------------------------------ */
/* PlanarQuant: src/kvquant.rs:325-478                                      */
/* ------------------------------------------------------------------------ */

typedef struct {
    size_t hd, n_groups, hd_padded;
    unsigned bits;
    float *cb;     /* 2^bits centroids, codebook(hd, bits) */
    float *givens; /* n_groups (cos, sin) pairs */
} or_pq;

/* src/kvquant.rs:336-345; returns NULL where the reference asserts. */
OR_API or_pq *or_pq_new(size_t hd, unsigned bits) {
    if (bits < 1 || bits > 8) return NULL;
    or_pq *p = calloc(1, sizeof(or_pq));
    p->hd = hd;
    p->bits = bits;
    p->n_groups = (hd + 1) / 2;
    p->hd_padded = p->n_groups * 2;
    p->cb = malloc(((size_t)1 << bits) * sizeof(float));
    p->givens = malloc(p->n_groups * 2 * sizeof(float));
    or_codebook(hd, bits, p->cb);
    or_givens_table(hd, p->givens);
    return p;
}

OR_API void or_pq_free(or_pq *p) {
    if (!p) return;
    free(p->cb); free(p->givens); free(p);
}

/* src/kvquant.rs:348-350 */
OR_API size_t or_pq_packed_len(const or_pq *p) { return or_packed_bytes(p->hd_padded, p->bits); }

/* src/kvquant.rs:357-370: strict '<' ascending scan, ties keep the lower index */
static uint8_t or_pq_nearest(const or_pq *p, float v) {
    const float *c = p->cb;
    size_t n = (size_t)1 << p->bits;
    size_t best = 0;
    float bd = fabsf(v - c[0]);
    for (size_t i = 1; i < n; i++) {
        float d = fabsf(v - c[i]);
        if (d < bd) { bd = d; best = i; }
    }
    return (uint8_t)best;
}

/* src/kvquant.rs:373-382; x has x_len valid entries, the rest read as 0 */
OR_API void or_pq_rotate(const or_pq *p, const float *x, size_t x_len, float *out) {
    for (size_t i = 0; i < p->n_groups; i++) {
        float c = p->givens[2 * i], s = p->givens[2 * i + 1];
        float a = (2 * i < x_len) ? x[2 * i] : 0.0f;
        float b = (2 * i + 1 < x_len) ? x[2 * i + 1] : 0.0f;
        out[2 * i] = c * a - s * b;
        out[2 * i + 1] = s * a + c * b;
    }
}

/* src/kvquant.rs:385-394 */
OR_API void or_pq_rotate_inv(const or_pq *p, const float *x, size_t x_len, float *out) {
    for (size_t i = 0; i < p->n_groups; i++) {
        float c = p->givens[2 * i], s = p->givens[2 * i + 1];
        float a = (2 * i < x_len) ? x[2 * i] : 0.0f;
        float b = (2 * i + 1 < x_len) ? x[2 * i + 1] : 0.0f;
        out[2 * i] = c * a + s * b;
        out[2 * i + 1] = -s * a + c * b;
    }
}

/* src/kvquant.rs:441-450 */
static void or_pq_rotate_inv_inplace(const or_pq *p, float *x) {
    for (size_t i = 0; i < p->n_groups; i++) {
        float c = p->givens[2 * i], s = p->givens[2 * i + 1];
        float a = x[2 * i], b = x[2 * i + 1];
        x[2 * i] = c * a + s * b;
        x[2 * i + 1] = -s * a + c * b;
    }
}

/* src/kvquant.rs:397-412 */
OR_API void or_pq_quantize(const or_pq *p, const float *x, uint8_t *packed, float *norm) {
    float sum = 0.0f;
    for (size_t i = 0; i < p->hd; i++) sum += x[i] * x[i];
    float n = sqrtf(sum);
    *norm = n;
    float inv = (n > 1e-12f) ? 1.0f / n : 0.0f;
    float *rot = calloc(p->hd_padded, sizeof(float));
    float *unit = calloc(p->hd_padded, sizeof(float));
    uint8_t *idx = calloc(p->hd_padded, 1);
    for (size_t i = 0; i < p->hd; i++) unit[i] = x[i] * inv;
    or_pq_rotate(p, unit, p->hd_padded, rot);
    for (size_t i = 0; i < p->hd_padded; i++) idx[i] = or_pq_nearest(p, rot[i]);
    or_pack_idx(idx, p->hd_padded, p->bits, packed);
    free(rot); free(unit); free(idx);
}

/* src/kvquant.rs:415-428 */
OR_API void or_pq_dequantize(const or_pq *p, const uint8_t *packed, float norm, float *out) {
    uint8_t *idx = calloc(p->hd_padded, 1);
    float *rot = calloc(p->hd_padded, sizeof(float));
    float *un = calloc(p->hd_padded, sizeof(float));
    or_unpack_idx(packed, p->hd_padded, p->bits, idx);
    for (size_t i = 0; i < p->hd_padded; i++) rot[i] = p->cb[idx[i]];
    or_pq_rotate_inv(p, rot, p->hd_padded, un);
    for (size_t i = 0; i < p->hd; i++) out[i] = un[i] * norm;
    free(idx); free(rot); free(un);
}

/* src/kvquant.rs:431-437 */
static void or_pq_unpack_centroids_into(const or_pq *p, const uint8_t *packed, uint8_t *idx,
                                        float *out) {
    or_unpack_idx(packed, p->hd_padded, p->bits, idx);
    for (size_t i = 0; i < p->hd_padded; i++) out[i] = p->cb[idx[i]];
}

/* src/kvquant.rs:463-477 */
static float or_pq_dot_rotated_scratch(const or_pq *p, const float *q_rot, const uint8_t *packed,
                                       float norm, uint8_t *idx) {
    or_unpack_idx(packed, p->hd_padded, p->bits, idx);
    float acc = 0.0f;
    for (size_t i = 0; i < p->hd; i++) acc += q_rot[i] * p->cb[idx[i]];
    return acc * norm;
}

/* src/kvquant.rs:455-458 */
OR_API float or_pq_dot_rotated(const or_pq *p, const float *q_rot, const uint8_t *packed,
                               float norm) {
    uint8_t *idx = calloc(p->hd_padded, 1);
    float r = or_pq_dot_rotated_scratch(p, q_rot, packed, norm, idx);
    free(idx);
    return r;
}

OR_API const float *or_pq_codebook_ptr(const or_pq *p) { return p->cb; }
OR_API const float *or_pq_givens_ptr(const or_pq *p) { return p->givens; }

/* ------------------------------------------------------------------------ */
/* Mode selection: src/kvquant.rs:486-567                                   */
/* ------------------------------------------------------------------------ */

enum { OR_MODE_F32 = 0, OR_MODE_F16 = 1, OR_MODE_PLANAR = 2 };

/* parse::<u32>() of Rust: optional leading '+', then one or more ASCII
 * digits, nothing else; overflow is an error. */
static int or_parse_u32(const char *s, size_t len, uint32_t *out) {
    size_t i = 0;
    if (len == 0) return 0;
    if (s[0] == '+') i = 1;
    if (i >= len) return 0;
    uint64_t v = 0;
    for (; i < len; i++) {
        if (s[i] < '0' || s[i] > '9') return 0;
        v = v * 10 + (uint64_t)(s[i] - '0');
        if (v > 0xffffffffULL) return 0;
    }
    *out = (uint32_t)v;
    return 1;
}

/* src/kvquant.rs:515-543.  Unknown or out-of-range values fall back to f32. */
OR_API void or_parse_mode(const char *s, int *mode, int *bits, int *v_quant) {
    *mode = OR_MODE_F32; *bits = 0; *v_quant = 0;
    size_t len = strlen(s);
    if (len == 0 || strcmp(s, "f32") == 0) return;
    if (strcmp(s, "f16") == 0 || strcmp(s, "fp16") == 0 || strcmp(s, "half") == 0) {
        *mode = OR_MODE_F16;
        return;
    }
    int k_only = 0;
    if (s[len - 1] == 'k') { k_only = 1; len--; }
    const char *rest = NULL;
    size_t rest_len = 0;
    if (len >= 6 && strncmp(s, "planar", 6) == 0) { rest = s + 6; rest_len = len - 6; }
    else if (len >= 3 && strncmp(s, "iso", 3) == 0) { rest = s + 3; rest_len = len - 3; }
    if (!rest) return;
    uint32_t b;
    if (!or_parse_u32(rest, rest_len, &b)) return;
    if (b < 1 || b > 8) return;
    *mode = OR_MODE_PLANAR;
    *bits = (int)b;
    *v_quant = !k_only;
}

/* ------------------------------------------------------------------------ */
/* IMROPE: src/rope.rs:9-70                                                 */
/* ------------------------------------------------------------------------ */

OR_API void or_rope_imrope(float *head, int64_t p_t, int64_t p_h, int64_t p_w, int64_t p_e,
                           size_t n_dims, const int32_t sections[4], float freq_base) {
    int64_t sect_dims = (int64_t)sections[0] + sections[1] + sections[2] + sections[3];
    float theta_scale = powf(freq_base, -2.0f / (float)n_dims);
    float th = (float)p_t, hh = (float)p_h, wh = (float)p_w, eh = (float)p_e;
    int64_t s0 = sections[0], s1 = sections[1], s2 = sections[2];
    float *cache = calloc(n_dims, sizeof(float));
    for (size_t i0 = 0; i0 < n_dims; i0 += 2) {
        int64_t sector = ((int64_t)i0 / 2) % sect_dims;
        float theta;
        if (sector % 3 == 1 && sector < 3 * s1) theta = hh;
        else if (sector % 3 == 2 && sector < 3 * s2) theta = wh;
        else if (sector % 3 == 0 && sector < 3 * s0) theta = th;
        else theta = eh;
        cache[i0] = cosf(theta);
        cache[i0 + 1] = sinf(theta);
        th *= theta_scale; hh *= theta_scale; wh *= theta_scale; eh *= theta_scale;
    }
    size_t half = n_dims / 2;
    for (size_t j = 0; j < half; j++) {
        float c = cache[2 * j], s = cache[2 * j + 1];
        float x0 = head[j], x1 = head[j + half];
        head[j] = x0 * c - x1 * s;
        head[j + half] = x0 * s + x1 * c;
    }
    free(cache);
}

/* ------------------------------------------------------------------------ */
/* f16 conversions: src/gguf.rs:881-944                                     */
/* ------------------------------------------------------------------------ */

/* src/gguf.rs:881-911 */
OR_API float or_half_to_f32(uint16_t h) {
    uint32_t sign = (h >> 15) & 1, exp = (h >> 10) & 0x1f, man = h & 0x3ff, bits;
    if (exp == 0) {
        if (man == 0) bits = sign << 31;
        else {
            int32_t e = 127 - 15 + 1;
            uint32_t m = man;
            while ((m & 0x400) == 0) { m <<= 1; e -= 1; }
            m &= 0x3ff;
            bits = (sign << 31) | ((uint32_t)e << 23) | (m << 13);
        }
    } else if (exp == 0x1f) {
        bits = (sign << 31) | 0x7f800000u | (man << 13);
    } else {
        bits = (sign << 31) | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* src/gguf.rs:914-944.  Round-to-nearest-even, except that the subnormal
 * branch shifts before it rounds (sticky bits are lost) and e < -10 flushes
 * to signed zero. */
OR_API uint16_t or_f32_to_half(float v) {
    uint32_t b;
    memcpy(&b, &v, 4);
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000);
    int32_t exp = (int32_t)((b >> 23) & 0xff);
    uint32_t man = b & 0x7fffff;
    if (exp == 0xff) {
        uint16_t m = man != 0 ? 0x200 : 0;
        return sign | 0x7c00 | m;
    }
    int32_t e = exp - 127 + 15;
    if (e >= 0x1f) return sign | 0x7c00;
    if (e <= 0) {
        if (e < -10) return sign;
        uint32_t m = (man | 0x800000) >> (uint32_t)(1 - e);
        uint16_t half = (uint16_t)(m >> 13);
        uint32_t rem = m & 0x1fff;
        uint16_t out = half + ((rem > 0x1000 || (rem == 0x1000 && (half & 1) == 1)) ? 1 : 0);
        return sign | out;
    }
    uint16_t half = (uint16_t)(((uint32_t)e << 10) | (man >> 13));
    uint32_t rem = man & 0x1fff;
    uint16_t out = (uint16_t)(half + ((rem > 0x1000 || (rem == 0x1000 && (half & 1) == 1)) ? 1 : 0));
    return sign | out;
}

/* ------------------------------------------------------------------------ */
/* softmax: src/kernels.rs:175-202                                          */
/* ------------------------------------------------------------------------ */

/* Returns -1 where the reference returns Err (length not a multiple). */
OR_API int or_softmax_rows(const float *x, size_t len, size_t row_len, float *out) {
    if (row_len == 0 || len % row_len != 0) return -1;
    for (size_t r = 0; r < len / row_len; r++) {
        const float *src = x + r * row_len;
        float *dst = out + r * row_len;
        float max = -INFINITY;
        for (size_t i = 0; i < row_len; i++)
            if (src[i] > max) max = src[i];
        double sum = 0.0;
        for (size_t i = 0; i < row_len; i++) {
            float e = expf(src[i] - max);
            dst[i] = e;
            sum += (double)e;
        }
        float inv = 1.0f / (float)sum;
        for (size_t i = 0; i < row_len; i++) dst[i] *= inv;
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* AttnCache + the attention step: src/forward.rs:30-140, 247-375           */
/* ------------------------------------------------------------------------ */

typedef struct {
    size_t n_layer, n_kv, hd, n_kv_elems, n_head, n_rot;
    int32_t sections[4];
    float freq_base;
    int mode, bits, v_quant;
    or_pq *pq, *pqv;
    /* per layer growable stores (src/forward.rs:30-51) */
    float **k, **v; size_t *k_len, *v_len, *k_cap, *v_cap;
    uint16_t **k16, **v16; size_t *k16_len, *v16_len, *k16_cap, *v16_cap;
    uint8_t **kq, **vq; size_t *kq_len, *vq_len, *kq_cap, *vq_cap;
    float **kn, **vn; size_t *kn_len, *vn_len, *kn_cap, *vn_cap;
} or_cache;

static void *or_grow(void *p, size_t *cap, size_t need, size_t elem) {
    if (need <= *cap) return p;
    size_t nc = *cap ? *cap : 1024;
    while (nc < need) nc *= 2;
    *cap = nc;
    return realloc(p, nc * elem);
}

#define OR_ALLOC_ARR(c, name, T) \
    c->name = calloc(n_layer, sizeof(T *)); \
    c->name##_len = calloc(n_layer, sizeof(size_t)); \
    c->name##_cap = calloc(n_layer, sizeof(size_t));

/* src/forward.rs:54-75 with the qwen35 constants passed in explicitly. */
OR_API or_cache *or_cache_new(size_t n_layer, size_t n_head, size_t n_kv, size_t hd, size_t n_rot,
                              const int32_t sections[4], float freq_base, int mode, int bits,
                              int v_quant) {
    or_cache *c = calloc(1, sizeof(or_cache));
    c->n_layer = n_layer; c->n_head = n_head; c->n_kv = n_kv; c->hd = hd;
    c->n_kv_elems = n_kv * hd; c->n_rot = n_rot; c->freq_base = freq_base;
    memcpy(c->sections, sections, sizeof(c->sections));
    c->mode = mode; c->bits = bits; c->v_quant = v_quant;
    if (mode == OR_MODE_PLANAR) {
        c->pq = or_pq_new(hd, (unsigned)bits);
        if (v_quant) c->pqv = or_pq_new(hd, (unsigned)bits);
    }
    OR_ALLOC_ARR(c, k, float) OR_ALLOC_ARR(c, v, float)
    OR_ALLOC_ARR(c, k16, uint16_t) OR_ALLOC_ARR(c, v16, uint16_t)
    OR_ALLOC_ARR(c, kq, uint8_t) OR_ALLOC_ARR(c, vq, uint8_t)
    OR_ALLOC_ARR(c, kn, float) OR_ALLOC_ARR(c, vn, float)
    return c;
}

#define OR_FREE_ARR(c, name) \
    for (size_t i = 0; i < c->n_layer; i++) free(c->name[i]); \
    free(c->name); free(c->name##_len); free(c->name##_cap);

OR_API void or_cache_free(or_cache *c) {
    if (!c) return;
    OR_FREE_ARR(c, k) OR_FREE_ARR(c, v) OR_FREE_ARR(c, k16) OR_FREE_ARR(c, v16)
    OR_FREE_ARR(c, kq) OR_FREE_ARR(c, vq) OR_FREE_ARR(c, kn) OR_FREE_ARR(c, vn)
    or_pq_free(c->pq); or_pq_free(c->pqv);
    free(c);
}

/* Decoder::reset clears the per-layer stores (src/forward.rs:640-656). */
OR_API void or_cache_reset(or_cache *c) {
    for (size_t i = 0; i < c->n_layer; i++) {
        c->k_len[i] = c->v_len[i] = c->k16_len[i] = c->v16_len[i] = 0;
        c->kq_len[i] = c->vq_len[i] = c->kn_len[i] = c->vn_len[i] = 0;
    }
}

/* src/forward.rs:78-86 */
OR_API size_t or_cache_n_pos(const or_cache *c, size_t il) {
    if (c->pq) return c->kn_len[il] / c->n_kv;
    if (c->mode == OR_MODE_F16) return c->k16_len[il] / c->n_kv_elems;
    return c->k_len[il] / c->n_kv_elems;
}

#define OR_PUSH(c, name, il, src, count, T) do { \
    c->name[il] = or_grow(c->name[il], &c->name##_cap[il], c->name##_len[il] + (count), sizeof(T)); \
    memcpy(c->name[il] + c->name##_len[il], (src), (count) * sizeof(T)); \
    c->name##_len[il] += (count); } while (0)

/* src/forward.rs:90-95 */
static void or_cache_append(or_cache *c, size_t il, const float *krow, const float *vrow) {
    OR_PUSH(c, k, il, krow, c->n_kv_elems, float);
    OR_PUSH(c, v, il, vrow, c->n_kv_elems, float);
}

/* src/forward.rs:99-111 */
static void or_cache_append_k_quantized(or_cache *c, size_t il, const float *krow) {
    size_t plen = or_pq_packed_len(c->pq);
    uint8_t *packed = malloc(plen);
    for (size_t kv = 0; kv < c->n_kv; kv++) {
        float norm = 0.0f;
        or_pq_quantize(c->pq, krow + kv * c->hd, packed, &norm);
        OR_PUSH(c, kq, il, packed, plen, uint8_t);
        OR_PUSH(c, kn, il, &norm, 1, float);
    }
    free(packed);
}

/* src/forward.rs:114-117 */
static void or_cache_append_v(or_cache *c, size_t il, const float *vrow) {
    OR_PUSH(c, v, il, vrow, c->n_kv_elems, float);
}

/* src/forward.rs:120-125 */
static void or_cache_append_f16(or_cache *c, size_t il, const float *krow, const float *vrow) {
    size_t n = c->n_kv_elems;
    uint16_t *tmp = malloc(n * sizeof(uint16_t));
    for (size_t i = 0; i < n; i++) tmp[i] = or_f32_to_half(krow[i]);
    OR_PUSH(c, k16, il, tmp, n, uint16_t);
    for (size_t i = 0; i < n; i++) tmp[i] = or_f32_to_half(vrow[i]);
    OR_PUSH(c, v16, il, tmp, n, uint16_t);
    free(tmp);
}

/* src/forward.rs:128-139 */
static void or_cache_append_v_quantized(or_cache *c, size_t il, const float *vrow) {
    size_t plen = or_pq_packed_len(c->pqv);
    uint8_t *packed = malloc(plen);
    for (size_t kv = 0; kv < c->n_kv; kv++) {
        float norm = 0.0f;
        or_pq_quantize(c->pqv, vrow + kv * c->hd, packed, &norm);
        OR_PUSH(c, vq, il, packed, plen, uint8_t);
        OR_PUSH(c, vn, il, &norm, 1, float);
    }
    free(packed);
}

/* The store half of the step, src/forward.rs:259-285: IMROPE on each kv head
 * of the (already RMS-normed) k with all four position ids = pos, then append
 * by mode.  v is stored as given.  k is not modified (a copy is roped). */
OR_API void or_append_token(or_cache *c, size_t il, const float *k_in, const float *v_in,
                            size_t pos) {
    float *k = malloc(c->n_kv_elems * sizeof(float));
    memcpy(k, k_in, c->n_kv_elems * sizeof(float));
    for (size_t kv = 0; kv < c->n_kv; kv++)
        or_rope_imrope(k + kv * c->hd, (int64_t)pos, (int64_t)pos, (int64_t)pos, (int64_t)pos,
                       c->n_rot, c->sections, c->freq_base);
    if (c->pq) {
        or_cache_append_k_quantized(c, il, k);
        if (c->pqv) or_cache_append_v_quantized(c, il, v_in);
        else or_cache_append_v(c, il, v_in);
    } else if (c->mode == OR_MODE_F16) {
        or_cache_append_f16(c, il, k, v_in);
    } else {
        or_cache_append(c, il, k, v_in);
    }
    free(k);
}

/* src/forward.rs:181-183 */
static float or_dot(const float *a, const float *b, size_t n) {
    float s = 0.0f;
    for (size_t i = 0; i < n; i++) s += a[i] * b[i];
    return s;
}

/* src/forward.rs:186-191 */
static float or_dot_f16(const float *a, const uint16_t *b, size_t n) {
    float s = 0.0f;
    for (size_t i = 0; i < n; i++) s += a[i] * or_half_to_f32(b[i]);
    return s;
}

/* One q-head of src/forward.rs:297-375.  `q` is that head's roped query. */
static void or_attend_head(const or_cache *c, size_t il, size_t hq, const float *qh, size_t n_pos,
                           float *out_head) {
    size_t hd = c->hd, n_kv = c->n_kv, n_rep = c->n_head / c->n_kv, nke = c->n_kv_elems;
    size_t hdp = ((hd + 1) / 2) * 2;
    float scale = 1.0f / sqrtf((float)hd);
    float *scores = malloc(n_pos * sizeof(float));
    float *probs = malloc(n_pos * sizeof(float));
    float *head_out = calloc(hdp, sizeof(float));
    float *qrot = calloc(hdp, sizeof(float));
    float *vrot = calloc(hdp, sizeof(float));
    uint8_t *vidx = calloc(hdp, 1);
    size_t kv = hq / n_rep, kv_off = kv * hd;

    if (c->pq) {
        size_t plen = or_pq_packed_len(c->pq);
        or_pq_rotate(c->pq, qh, hd, qrot);
        for (size_t j = 0; j < n_pos; j++) {
            const uint8_t *row = c->kq[il] + (j * n_kv + kv) * plen;
            float norm = c->kn[il][j * n_kv + kv];
            scores[j] = or_pq_dot_rotated_scratch(c->pq, qrot, row, norm, vidx) * scale;
        }
    } else if (c->mode == OR_MODE_F16) {
        for (size_t j = 0; j < n_pos; j++)
            scores[j] = or_dot_f16(qh, c->k16[il] + j * nke + kv_off, hd) * scale;
    } else {
        for (size_t j = 0; j < n_pos; j++)
            scores[j] = or_dot(qh, c->k[il] + j * nke + kv_off, hd) * scale;
    }
    or_softmax_rows(scores, n_pos, n_pos, probs);

    if (c->pqv) {
        size_t plen = or_pq_packed_len(c->pqv);
        for (size_t j = 0; j < n_pos; j++) {
            float pj = probs[j];
            if (pj == 0.0f) continue;
            float norm = c->vn[il][j * n_kv + kv];
            or_pq_unpack_centroids_into(c->pqv, c->vq[il] + (j * n_kv + kv) * plen, vidx, vrot);
            float w = pj * norm;
            for (size_t d = 0; d < hd; d++) head_out[d] += w * vrot[d];
        }
        or_pq_rotate_inv_inplace(c->pqv, head_out);
    } else if (c->mode == OR_MODE_F16) {
        for (size_t j = 0; j < n_pos; j++) {
            float pj = probs[j];
            if (pj == 0.0f) continue;
            const uint16_t *vj = c->v16[il] + j * nke + kv_off;
            for (size_t d = 0; d < hd; d++) head_out[d] += pj * or_half_to_f32(vj[d]);
        }
    } else {
        for (size_t j = 0; j < n_pos; j++) {
            float pj = probs[j];
            if (pj == 0.0f) continue;
            const float *vj = c->v[il] + j * nke + kv_off;
            for (size_t d = 0; d < hd; d++) head_out[d] += pj * vj[d];
        }
    }
    memcpy(out_head, head_out, hd * sizeof(float));
    free(scores); free(probs); free(head_out); free(qrot); free(vrot); free(vidx);
}

/* The attend half of the step, src/forward.rs:247-258 and 287-375: IMROPE on
 * each q head at q_pos, then GQA attention over the first n_pos cached
 * positions (the reference always uses n_pos = pos + 1, q_pos = pos).
 * `threads` <= 1 runs the reference's single-threaded head loop; larger
 * values spread the independent q-heads over POSIX threads, which changes no
 * result because heads share no state. */
typedef struct {
    const or_cache *c; size_t il, n_pos, nh, hd; const float *q; float *out;
    size_t next; pthread_mutex_t mu;
} or_head_job;

static void *or_head_worker(void *arg) {
    or_head_job *j = arg;
    for (;;) {
        pthread_mutex_lock(&j->mu);
        size_t hq = j->next++;
        pthread_mutex_unlock(&j->mu);
        if (hq >= j->nh) break;
        or_attend_head(j->c, j->il, hq, j->q + hq * j->hd, j->n_pos, j->out + hq * j->hd);
    }
    return NULL;
}

OR_API int or_attend(const or_cache *c, size_t il, const float *q_in, size_t q_pos, size_t n_pos,
                     float *out, int threads) {
    if (n_pos == 0 || n_pos > or_cache_n_pos(c, il)) return -1;
    size_t nh = c->n_head, hd = c->hd;
    float *q = malloc(nh * hd * sizeof(float));
    memcpy(q, q_in, nh * hd * sizeof(float));
    for (size_t h = 0; h < nh; h++)
        or_rope_imrope(q + h * hd, (int64_t)q_pos, (int64_t)q_pos, (int64_t)q_pos, (int64_t)q_pos,
                       c->n_rot, c->sections, c->freq_base);
    if (threads <= 1) {
        for (size_t hq = 0; hq < nh; hq++) or_attend_head(c, il, hq, q + hq * hd, n_pos, out + hq * hd);
    } else {
        if ((size_t)threads > nh) threads = (int)nh;
        or_head_job job = {c, il, n_pos, nh, hd, q, out, 0, PTHREAD_MUTEX_INITIALIZER};
        pthread_t *tid = malloc((size_t)threads * sizeof(pthread_t));
        int started = 0;
        for (int t = 0; t < threads; t++)
            if (pthread_create(&tid[started], NULL, or_head_worker, &job) == 0) started++;
        if (started == 0) or_head_worker(&job);
        for (int t = 0; t < started; t++) pthread_join(tid[t], NULL);
        free(tid);
    }
    free(q);
    return 0;
}

/* Whole step as src/forward.rs:247-375 runs it: rope, store at index pos
 * (which must equal the number of cached tokens), attend over pos + 1. */
OR_API int or_attn_step(or_cache *c, size_t il, const float *q, const float *k, const float *v,
                        size_t pos, float *out, int threads) {
    if (or_cache_n_pos(c, il) != pos) return -2; /* debug_assert at src/forward.rs:285 */
    or_append_token(c, il, k, v, pos);
    return or_attend(c, il, q, pos, pos + 1, out, threads);
}

/* rms_norm_rows, src/kernels.rs:97-122: rows of row_len sharing one weight;
 * sequential f32 sum of squares, scale = 1 / sqrt(ss / row_len + eps),
 * dst = src * scale * w (left to right).  -1 on the reference's two error
 * cases (weight length, ragged x). */
OR_API int or_rms_norm_rows(const float *x, size_t x_len, const float *w, size_t w_len, size_t row_len, float eps,
                            float *out) {
    if (w_len != row_len) return -1;
    if (row_len == 0 || x_len % row_len != 0) return -1;
    for (size_t r = 0; r < x_len / row_len; r++) {
        const float *src = x + r * row_len;
        float *dst = out + r * row_len;
        float ss = 0.0f;
        for (size_t i = 0; i < row_len; i++) ss += src[i] * src[i];
        float scale = 1.0f / sqrtf(ss / (float)row_len + eps);
        for (size_t i = 0; i < row_len; i++) dst[i] = src[i] * scale * w[i];
    }
    return 0;
}

/* sigmoid, src/kernels.rs:162-164. */
OR_API float or_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

/* full_attention_layer between the projections and the output projection,
 * src/forward.rs:237-382: split [q | gate] per head (:237-241), per-head
 * RMSNorm of q and k (:242-245), then the step above (:247-375), then
 * out *= sigmoid(gate) (:379-382).  qfull [n_head][2*hd]. */
OR_API int or_attn_layer_step(or_cache *c, size_t il, const float *qfull, const float *kraw, const float *vraw,
                              const float *q_norm_w, const float *k_norm_w, float eps, size_t pos, float *out,
                              int threads) {
    size_t nh = c->n_head, hd = c->hd;
    float *q = malloc(nh * hd * sizeof(float)), *gate = malloc(nh * hd * sizeof(float));
    float *qn = malloc(nh * hd * sizeof(float)), *kn = malloc(c->n_kv_elems * sizeof(float));
    for (size_t h = 0; h < nh; h++) {
        memcpy(q + h * hd, qfull + h * 2 * hd, hd * sizeof(float));
        memcpy(gate + h * hd, qfull + h * 2 * hd + hd, hd * sizeof(float));
    }
    or_rms_norm_rows(q, nh * hd, q_norm_w, hd, hd, eps, qn);
    or_rms_norm_rows(kraw, c->n_kv_elems, k_norm_w, hd, hd, eps, kn);
    int rc = or_attn_step(c, il, qn, kn, vraw, pos, out, threads);
    if (rc == 0)
        for (size_t i = 0; i < nh * hd; i++) out[i] *= or_sigmoid(gate[i]);
    free(q); free(gate); free(qn); free(kn);
    return rc;
}

/* Read-only views of the stores, for byte comparison with the device cache. */
OR_API const float *or_cache_k(const or_cache *c, size_t il) { return c->k[il]; }
OR_API const float *or_cache_v(const or_cache *c, size_t il) { return c->v[il]; }
OR_API const uint16_t *or_cache_k16(const or_cache *c, size_t il) { return c->k16[il]; }
OR_API const uint16_t *or_cache_v16(const or_cache *c, size_t il) { return c->v16[il]; }
OR_API const uint8_t *or_cache_kq(const or_cache *c, size_t il) { return c->kq[il]; }
OR_API const uint8_t *or_cache_vq(const or_cache *c, size_t il) { return c->vq[il]; }
OR_API const float *or_cache_kn(const or_cache *c, size_t il) { return c->kn[il]; }
OR_API const float *or_cache_vn(const or_cache *c, size_t il) { return c->vn[il]; }

/* ------------------------------------------------------------------------ */
/* Test inputs                                                              */
/* ------------------------------------------------------------------------ */

/* xorshift generator shared by the reference's tests and self-checks:
 * src/bin/bonsai-vk.rs:32-42, src/kvquant.rs:581-589.  Values in [-1, 1). */
OR_API void or_rand_floats(uint64_t seed, size_t n, float *out) {
    uint64_t x = seed | 1;
    for (size_t i = 0; i < n; i++) {
        x ^= x << 13;
        x ^= x >> 7;
        x ^= x << 17;
        out[i] = ((float)(x >> 40) / (float)((uint64_t)1 << 24)) * 2.0f - 1.0f;
    }
}

OR_API int or_max_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

/* ---- PQ2_0 ternary rows (src/kernels.rs:204-330, 333-420, 631-650) ---------------------- */

/* pq2_row_bytes, src/kernels.rs:208-211. */
OR_API size_t or_pq2_row_bytes(size_t ne0) { return ((ne0 + 127) / 128) * 34; }

/* decode_pq2_0_row, src/kernels.rs:213-229: (code - 1) * scale, codes two bits each, least
 * significant first, one f16 scale per 128. */
OR_API void or_pq2_decode_row(const uint8_t *raw, size_t ne0, float *out) {
    size_t n = 0;
    for (size_t block = 0; block < (ne0 + 127) / 128; block++) {
        const uint8_t *b = raw + block * 34;
        const float scale = or_half_to_f32((uint16_t)(b[0] | (b[1] << 8)));
        for (size_t j = 0; j < 128 && block * 128 + j < ne0; j++) {
            const int code = (b[2 + j / 4] >> ((j % 4) * 2)) & 3;
            out[n++] = (float)(code - 1) * scale;
        }
    }
}

/* row_dot_scalar, src/kernels.rs:633-650: per block a sequential f32 sum of x * (code - 1), then
 * acc += scale * block_acc.  (The reference's AVX2 path, 652-760, is the same sum in another
 * order; its own test bounds the difference by 1e-4 relative, src/kernels.rs:855-906.) */
static float pq2_row_dot(const uint8_t *raw, size_t ne0, const float *x) {
    float acc = 0.0f;
    for (size_t block = 0; block < (ne0 + 127) / 128; block++) {
        const uint8_t *b = raw + block * 34;
        const float scale = or_half_to_f32((uint16_t)(b[0] | (b[1] << 8)));
        const size_t start = block * 128, end = start + 128 < ne0 ? start + 128 : ne0;
        float block_acc = 0.0f;
        for (size_t j = start; j < end; j++) {
            const int code = (b[2 + (j - start) / 4] >> (((j - start) % 4) * 2)) & 3;
            block_acc += x[j] * (float)(code - 1);
        }
        acc += scale * block_acc;
    }
    return acc;
}

/* dot_pq2_0_row, src/kernels.rs:234-263: the dot against the DECODED row (weights scaled first),
 * another rounding order the reference ships; -1 when the row is outside the payload. */
OR_API int or_pq2_dot_row(const uint8_t *payload, size_t payload_len, size_t ne0, size_t row, const float *x, float *out) {
    const size_t rb = or_pq2_row_bytes(ne0);
    if ((row + 1) * rb > payload_len) return -1;
    float *w = (float *)malloc(ne0 * sizeof(float));
    or_pq2_decode_row(payload + row * rb, ne0, w);
    float acc = 0.0f;
    for (size_t j = 0; j < ne0; j++) acc += x[j] * w[j];
    free(w);
    *out = acc;
    return 0;
}

/* pq2_matvec_range / pq2_matmul_n, src/kernels.rs:265-330, 333-420 (scalar row dot):
 * y[t * n_rows + r] = x[t] . W[base_row + r].  -1: rows outside the payload. */
OR_API int or_pq2_matmul(const uint8_t *payload, size_t payload_len, size_t ne0, size_t base_row, size_t n_rows, const float *x,
                         size_t n_tok, float *y) {
    const size_t rb = or_pq2_row_bytes(ne0);
    if ((base_row + n_rows) * rb > payload_len) return -1;
    for (size_t r = 0; r < n_rows; r++)
        for (size_t t = 0; t < n_tok; t++) y[t * n_rows + r] = pq2_row_dot(payload + (base_row + r) * rb, ne0, x + t * ne0);
    return 0;
}
