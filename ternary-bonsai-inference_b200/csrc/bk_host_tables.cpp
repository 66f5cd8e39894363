// Host set-up tables of the KV path: Lloyd-Max codebooks, the Givens table and the IMROPE
// cos/sin rows.  The reference computes all three on the CPU as well (the GPU build uploads the
// first two, src/gdev.rs:360-368; its shader recomputes the rope angle with pow(), which
// differs from the CPU's iterated product, and the CPU path is the one stored bytes must
// match).  These are one-time tables, not a compute fallback: the per-token work is on the GPU.
//
// Built with -ffp-contract=off; double where the reference uses f64, float where it uses f32,
// the host libm for exp/cos/sin/powf/cosf/sinf as in the reference's build.
#include <math.h>
#include <stdint.h>

#include <algorithm>
#include <thread>
#include <vector>

#include "bk_internal.h"

namespace bk {

namespace {

// A&S 7.1.26 as written at src/kvquant.rs:34-44.
double erf_as(double x) {
    const double sign = x < 0.0 ? -1.0 : 1.0;
    x = fabs(x);
    const double t = 1.0 / (1.0 + 0.3275911 * x);
    const double p =
        ((((1.061405429 * t - 1.453152027) * t) + 1.421413741) * t - 0.284496736) * t + 0.254829592;
    return sign * (1.0 - p * t * exp(-x * x));
}
double cdf(double x, double s) { return 0.5 * (1.0 + erf_as(x / (s * 1.4142135623730951))); }
double pdf(double x, double s) {
    return exp(-(x * x) / (2.0 * s * s)) / (s * sqrt(2.0 * 3.14159265358979323846));
}

uint64_t splitmix_next(uint64_t &state) {
    state += 0x9E3779B97F4A7C15ULL;
    uint64_t z = state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

}  // namespace

// src/kvquant.rs:62-114.  The 300-iteration cap is part of the format (widths 4..8 stop there).
void host_codebook(int hd, int bits, float *out) {
    const double sigma = 1.0 / sqrt((double)hd);
    const int n = 1 << bits;
    std::vector<double> c(n), nx(n), edge(n + 1);
    const double lo = -3.5 * sigma, hi = 3.5 * sigma, outer = 12.0 * sigma;
    for (int i = 0; i < n; i++) c[i] = lo + (hi - lo) * ((double)i + 0.5) / (double)n;
    for (int it = 0; it < 300; it++) {
        edge[0] = -outer;
        for (int i = 0; i + 1 < n; i++) edge[i + 1] = (c[i] + c[i + 1]) / 2.0;
        edge[n] = outer;
        double shift = 0.0;
        for (int i = 0; i < n; i++) {
            const double a = edge[i], b = edge[i + 1];
            const double mass = cdf(b, sigma) - cdf(a, sigma);
            nx[i] = mass > 1e-15 ? (sigma * sigma * (pdf(a, sigma) - pdf(b, sigma))) / mass : c[i];
            shift = std::max(shift, fabs(nx[i] - c[i]));
        }
        c.swap(nx);
        if (shift < 1e-12) break;
    }
    for (int i = 0; i < n; i++) out[i] = (float)c[i];
}

// src/kvquant.rs:131-145: splitmix64 from state 42, angle in f64, (cos, sin) narrowed to f32.
void host_givens(int hd, float *out) {
    uint64_t state = 42;
    for (int g = 0; g < (hd + 1) / 2; g++) {
        const uint64_t r = splitmix_next(state);
        const double u = (double)(r >> 11) / (double)(1ULL << 53);
        const double t = u * 6.283185307179586;
        out[2 * g] = (float)cos(t);
        out[2 * g + 1] = (float)sin(t);
    }
}

// src/rope.rs:37-49: which position id pair j rotates with.
int host_rope_band(int j, const int32_t sections[4]) {
    const int64_t sect_dims = (int64_t)sections[0] + sections[1] + sections[2] + sections[3];
    const int64_t sector = sect_dims > 0 ? (int64_t)j % sect_dims : 0;
    if (sector % 3 == 1 && sector < 3 * (int64_t)sections[1]) return 1;
    if (sector % 3 == 2 && sector < 3 * (int64_t)sections[2]) return 2;
    if (sector % 3 == 0 && sector < 3 * (int64_t)sections[0]) return 0;
    return 3;
}

// src/rope.rs:23-57: the angle of pair j is the f32 position multiplied j times by
// theta_scale = powf(base, -2/n_dims), each product rounded to f32; then libm cosf/sinf.
void host_rope_rows(int64_t pos0, int64_t n_pos, int n_rot, float freq_base, float2 *out) {
    const int half = n_rot / 2;
    if (half <= 0 || n_pos <= 0) return;
    const float theta_scale = powf(freq_base, -2.0f / (float)n_rot);
    auto work = [=](int64_t a, int64_t b) {
        for (int64_t p = a; p < b; p++) {
            float th = (float)(pos0 + p);
            float2 *row = out + p * half;
            for (int j = 0; j < half; j++) {
                row[j].x = cosf(th);
                row[j].y = sinf(th);
                th *= theta_scale;
            }
        }
    };
    unsigned nt = std::thread::hardware_concurrency();
    if (nt == 0) nt = 1;
    nt = (unsigned)std::min<int64_t>(nt, std::max<int64_t>(1, n_pos / 4096));
    if (nt <= 1) {
        work(0, n_pos);
        return;
    }
    std::vector<std::thread> th;
    const int64_t per = (n_pos + nt - 1) / nt;
    for (unsigned t = 0; t < nt; t++) {
        const int64_t a = t * per, b = std::min<int64_t>(n_pos, a + per);
        if (a < b) th.emplace_back(work, a, b);
    }
    for (auto &t : th) t.join();
}

}  // namespace bk
