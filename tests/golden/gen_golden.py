#!/usr/bin/env python3
"""Generate tests/golden/kvpath_golden.npz.

A second restatement of the reference's CPU KV-cache path, written in plain
Python over numpy float32 scalars and independent of oracle/bonsai_oracle.c
(it shares no code with it).  The C oracle must reproduce every array in the
fixture bit for bit; two restatements that agree are the strongest pin that
exists for this path, since the reference (Rust) cannot be built where the
tests run and holds no byte-level golden vectors of its own.

Transcendentals go through the host's glibc via ctypes (cosf/sinf/powf/expf
and the f64 exp/cos/sin/sqrt), the same library the Rust build calls.

Reference lines restated (paths inside the reference project):
  src/kvquant.rs:34-145   erf, Lloyd-Max codebook, splitmix64, Givens table
  src/kvquant.rs:152-165  little-endian bitstream packing (for hd = 256 every
                          pack_idx branch yields these bytes)
  src/kvquant.rs:357-412  nearest, rotate, quantize
  src/rope.rs:9-70        IMROPE
  src/gguf.rs:881-944     f16 conversions
  src/kernels.rs:175-202  softmax_rows
  src/forward.rs:247-375  the attention step
  src/bin/bonsai-vk.rs:32-42  rand_floats

Run:  python tests/golden/gen_golden.py     (about a minute)
"""
import ctypes
import math
import os
import struct

import numpy as np

F = np.float32
libm = ctypes.CDLL("libm.so.6")
for _n in ("cosf", "sinf", "expf"):
    getattr(libm, _n).restype = ctypes.c_float
    getattr(libm, _n).argtypes = [ctypes.c_float]
libm.powf.restype = ctypes.c_float
libm.powf.argtypes = [ctypes.c_float, ctypes.c_float]


def cosf(x): return F(libm.cosf(float(x)))
def sinf(x): return F(libm.sinf(float(x)))
def expf(x): return F(libm.expf(float(x)))
def powf(x, y): return F(libm.powf(float(x), float(y)))


HD, N_KV, N_HEAD, N_ROT = 256, 4, 24, 64
SECTIONS = (11, 11, 10, 0)
FREQ_BASE = F(1e7)


# -- kvquant.rs:34-114 ------------------------------------------------------
def erf(x):
    sign = -1.0 if x < 0.0 else 1.0
    x = abs(x)
    t = 1.0 / (1.0 + 0.3275911 * x)
    y = 1.0 - (((((1.061405429 * t - 1.453152027) * t) + 1.421413741) * t - 0.284496736) * t
               + 0.254829592) * t * math.exp(-x * x)
    return sign * y


def norm_cdf(x, s): return 0.5 * (1.0 + erf(x / (s * math.sqrt(2.0))))
def norm_pdf(x, s): return math.exp(-(x * x) / (2.0 * s * s)) / (s * math.sqrt(2.0 * math.pi))
def first_moment(a, b, s): return s * s * (norm_pdf(a, s) - norm_pdf(b, s))


def solve_lloyd_max(sigma, bits):
    n = 1 << bits
    lo, hi = -3.5 * sigma, 3.5 * sigma
    c = [lo + (hi - lo) * (i + 0.5) / n for i in range(n)]
    outer = 12.0 * sigma
    iters = 0
    for _ in range(300):
        iters += 1
        edges = [-outer] + [(c[i] + c[i + 1]) / 2.0 for i in range(n - 1)] + [outer]
        nxt = []
        for i in range(n):
            a, b = edges[i], edges[i + 1]
            mass = norm_cdf(b, sigma) - norm_cdf(a, sigma)
            nxt.append(first_moment(a, b, sigma) / mass if mass > 1e-15 else c[i])
        shift = max(abs(x - y) for x, y in zip(nxt, c))
        c = nxt
        if shift < 1e-12:
            break
    return np.array(c, dtype=np.float64).astype(np.float32), iters


def codebook(d, bits):
    return solve_lloyd_max(1.0 / math.sqrt(float(d)), bits)


# -- kvquant.rs:120-145 -----------------------------------------------------
M64 = (1 << 64) - 1


def splitmix64(state):
    state = (state + 0x9E3779B97F4A7C15) & M64
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
    return state, z ^ (z >> 31)


def givens_table(d):
    state = 42
    out = np.zeros(((d + 1) // 2, 2), dtype=np.float32)
    for g in range(out.shape[0]):
        state, r = splitmix64(state)
        u = (r >> 11) / float(1 << 53)
        t = u * math.tau
        out[g, 0] = F(math.cos(t))
        out[g, 1] = F(math.sin(t))
    return out


# -- bonsai-vk.rs:32-42 -----------------------------------------------------
def rand_floats(seed, n):
    x = (seed | 1) & M64
    out = np.zeros(n, dtype=np.float32)
    for i in range(n):
        x ^= (x << 13) & M64
        x ^= x >> 7
        x ^= (x << 17) & M64
        out[i] = F(F(F(x >> 40) / F(1 << 24)) * F(2.0)) - F(1.0)
    return out


# -- kvquant.rs:152-165 -----------------------------------------------------
def pack_bits(idx, bits):
    nbytes = (len(idx) * bits + 7) // 8
    out = [0] * (nbytes + 1)
    bp = 0
    for v in idx:
        b, off = bp >> 3, bp & 7
        v &= (1 << bits) - 1
        out[b] |= (v << off) & 0xFF
        if off + bits > 8:
            out[b + 1] |= (v >> (8 - off)) & 0xFF
        bp += bits
    return np.array(out[:nbytes], dtype=np.uint8)


def unpack_bits(packed, bits, n):
    out = []
    bp = 0
    mask = (1 << bits) - 1
    for _ in range(n):
        b, off = bp >> 3, bp & 7
        v = int(packed[b]) >> off
        if off + bits > 8:
            v |= int(packed[b + 1]) << (8 - off)
        out.append(v & mask)
        bp += bits
    return out


# -- kvquant.rs:357-412 -----------------------------------------------------
def rotate(x, giv):
    out = np.zeros(len(x), dtype=np.float32)
    for i in range(len(x) // 2):
        c, s = F(giv[i, 0]), F(giv[i, 1])
        a, b = F(x[2 * i]), F(x[2 * i + 1])
        out[2 * i] = F(c * a) - F(s * b)
        out[2 * i + 1] = F(s * a) + F(c * b)
    return out


def rotate_inv(x, giv):
    out = np.zeros(len(x), dtype=np.float32)
    for i in range(len(x) // 2):
        c, s = F(giv[i, 0]), F(giv[i, 1])
        a, b = F(x[2 * i]), F(x[2 * i + 1])
        out[2 * i] = F(c * a) + F(s * b)
        out[2 * i + 1] = F(F(-s) * a) + F(c * b)
    return out


def nearest(v, cb):
    best, bd = 0, abs(F(v - cb[0]))
    for i in range(1, len(cb)):
        d = abs(F(v - cb[i]))
        if d < bd:
            bd, best = d, i
    return best


def quantize(x, cb, giv, bits):
    acc = F(0.0)
    for v in x:
        acc = F(acc + F(F(v) * F(v)))
    n = F(np.sqrt(acc))
    inv = F(F(1.0) / n) if n > F(1e-12) else F(0.0)
    unit = np.array([F(F(v) * inv) for v in x], dtype=np.float32)
    rot = rotate(unit, giv)
    idx = [nearest(F(v), cb) for v in rot]
    return pack_bits(idx, bits), n


# -- rope.rs:9-70 -----------------------------------------------------------
def rope_imrope(head, p_t, p_h, p_w, p_e, n_dims, sections, freq_base):
    head = head.copy()
    sect_dims = sum(sections)
    theta_scale = powf(freq_base, F(-2.0) / F(n_dims))
    th, hh, wh, eh = F(p_t), F(p_h), F(p_w), F(p_e)
    s0, s1, s2 = sections[0], sections[1], sections[2]
    cache = np.zeros(n_dims, dtype=np.float32)
    for i0 in range(0, n_dims, 2):
        sector = (i0 // 2) % sect_dims
        if sector % 3 == 1 and sector < 3 * s1:
            theta = hh
        elif sector % 3 == 2 and sector < 3 * s2:
            theta = wh
        elif sector % 3 == 0 and sector < 3 * s0:
            theta = th
        else:
            theta = eh
        cache[i0], cache[i0 + 1] = cosf(theta), sinf(theta)
        th, hh, wh, eh = F(th * theta_scale), F(hh * theta_scale), F(wh * theta_scale), F(eh * theta_scale)
    half = n_dims // 2
    for j in range(half):
        c, s = F(cache[2 * j]), F(cache[2 * j + 1])
        x0, x1 = F(head[j]), F(head[j + half])
        head[j] = F(x0 * c) - F(x1 * s)
        head[j + half] = F(x0 * s) + F(x1 * c)
    return head


# -- gguf.rs:881-944 --------------------------------------------------------
def half_to_f32(h):
    sign, exp, man = (h >> 15) & 1, (h >> 10) & 0x1F, h & 0x3FF
    if exp == 0:
        if man == 0:
            bits = sign << 31
        else:
            e, m = 127 - 15 + 1, man
            while m & 0x400 == 0:
                m <<= 1
                e -= 1
            bits = (sign << 31) | (e << 23) | ((m & 0x3FF) << 13)
    elif exp == 0x1F:
        bits = (sign << 31) | 0x7F800000 | (man << 13)
    else:
        bits = (sign << 31) | ((exp + 127 - 15) << 23) | (man << 13)
    return struct.unpack("<f", struct.pack("<I", bits))[0]


def f32_to_half(v):
    b = struct.unpack("<I", struct.pack("<f", float(v)))[0]
    sign, exp, man = (b >> 16) & 0x8000, (b >> 23) & 0xFF, b & 0x7FFFFF
    if exp == 0xFF:
        return sign | 0x7C00 | (0x200 if man else 0)
    e = exp - 127 + 15
    if e >= 0x1F:
        return sign | 0x7C00
    if e <= 0:
        if e < -10:
            return sign
        m = (man | 0x800000) >> (1 - e)
        half, rem = m >> 13, m & 0x1FFF
        return sign | (half + (1 if rem > 0x1000 or (rem == 0x1000 and half & 1) else 0))
    half, rem = (e << 10) | (man >> 13), man & 0x1FFF
    return sign | ((half + (1 if rem > 0x1000 or (rem == 0x1000 and half & 1) else 0)) & 0xFFFF)


# -- kernels.rs:175-202 -----------------------------------------------------
def softmax_row(x):
    mx = F(-np.inf)
    for v in x:
        if v > mx:
            mx = F(v)
    e = np.zeros(len(x), dtype=np.float32)
    total = 0.0
    for i, v in enumerate(x):
        e[i] = expf(F(v) - mx)
        total += float(e[i])
    inv = F(1.0) / F(total)
    return np.array([F(v * inv) for v in e], dtype=np.float32)


# -- forward.rs:247-375 -----------------------------------------------------
def attention_steps(mode, bits, v_quant, n_tokens, seed, inputs=None):
    """Run n_tokens decode steps from an empty cache; return per-step outputs and the cache.
    `inputs(pos)` may supply the step's (q, k, v) instead of the seeded generator."""
    cb = codebook(HD, bits)[0] if mode == "planar" else None
    giv = givens_table(HD)
    kstore, vstore, knorm, vnorm = [], [], [], []
    outs = []
    scale = F(1.0) / F(np.sqrt(F(HD)))
    for pos in range(n_tokens):
        if inputs is not None:
            q, k, v = inputs(pos)
        else:
            q = rand_floats(seed + 3 * pos, N_HEAD * HD)
            k = rand_floats(seed + 3 * pos + 1, N_KV * HD)
            v = rand_floats(seed + 3 * pos + 2, N_KV * HD)
        q = np.concatenate([rope_imrope(q[h * HD:(h + 1) * HD], pos, pos, pos, pos, N_ROT, SECTIONS, FREQ_BASE)
                            for h in range(N_HEAD)])
        k = np.concatenate([rope_imrope(k[h * HD:(h + 1) * HD], pos, pos, pos, pos, N_ROT, SECTIONS, FREQ_BASE)
                            for h in range(N_KV)])
        for kv in range(N_KV):
            kr, vr = k[kv * HD:(kv + 1) * HD], v[kv * HD:(kv + 1) * HD]
            if mode == "planar":
                p, n = quantize(kr, cb, giv, bits)
                kstore.append(p); knorm.append(n)
                if v_quant:
                    p, n = quantize(vr, cb, giv, bits)
                    vstore.append(p); vnorm.append(n)
                else:
                    vstore.append(vr.copy())
            elif mode == "f16":
                kstore.append(np.array([f32_to_half(x) for x in kr], dtype=np.uint16))
                vstore.append(np.array([f32_to_half(x) for x in vr], dtype=np.uint16))
            else:
                kstore.append(kr.copy()); vstore.append(vr.copy())
        n_pos = pos + 1
        out = np.zeros(N_HEAD * HD, dtype=np.float32)
        for hq in range(N_HEAD):
            qh = q[hq * HD:(hq + 1) * HD]
            kv = hq // (N_HEAD // N_KV)
            scores = np.zeros(n_pos, dtype=np.float32)
            if mode == "planar":
                qrot = rotate(qh, giv)
            for j in range(n_pos):
                row = kstore[j * N_KV + kv]
                acc = F(0.0)
                if mode == "planar":
                    idx = unpack_bits(row, bits, HD)
                    for i in range(HD):
                        acc = F(acc + F(qrot[i] * cb[idx[i]]))
                    acc = F(acc * knorm[j * N_KV + kv])
                elif mode == "f16":
                    for i in range(HD):
                        acc = F(acc + F(qh[i] * F(half_to_f32(int(row[i])))))
                else:
                    for i in range(HD):
                        acc = F(acc + F(qh[i] * row[i]))
                scores[j] = F(acc * scale)
            probs = softmax_row(scores)
            ho = np.zeros(HD, dtype=np.float32)
            for j in range(n_pos):
                pj = F(probs[j])
                if pj == 0.0:
                    continue
                row = vstore[j * N_KV + kv]
                if mode == "planar" and v_quant:
                    idx = unpack_bits(row, bits, HD)
                    w = F(pj * vnorm[j * N_KV + kv])
                    for d in range(HD):
                        ho[d] = F(ho[d] + F(w * cb[idx[d]]))
                elif mode == "f16":
                    for d in range(HD):
                        ho[d] = F(ho[d] + F(pj * F(half_to_f32(int(row[d])))))
                else:
                    for d in range(HD):
                        ho[d] = F(ho[d] + F(pj * row[d]))
            if mode == "planar" and v_quant:
                # rotate_inv_inplace: (c*a + s*b, -s*a + c*b)
                ho = rotate_inv(ho, giv)
            out[hq * HD:(hq + 1) * HD] = ho
        outs.append(out)
    return np.stack(outs), kstore, vstore, knorm, vnorm


def main():
    g = {}
    # codebooks and iteration counts for every width
    for bits in range(1, 9):
        cb, iters = codebook(HD, bits)
        g[f"codebook_b{bits}"] = cb.view(np.uint32)
        g[f"codebook_iters_b{bits}"] = np.array([iters], dtype=np.int32)
    giv = givens_table(HD)
    g["givens"] = giv.view(np.uint32)
    state, r0 = splitmix64(42)
    g["splitmix_first"] = np.array([r0], dtype=np.uint64)

    # rand_floats
    g["rand_0x1010"] = rand_floats(0x1010, 64).view(np.uint32)

    # f16 conversions: specials, boundary cases and a sweep
    vals = [0.0, -0.0, 1.0, -2.0, 0.5, 65504.0, 65520.0, 1e5, -1e5, float("inf"), float("-inf"),
            6.1035156e-5, 6.0975552e-5, 5.9604645e-8, 2.9802322e-8, 2.9802326e-8, 8.940697e-8,
            1e-8, 3.0e-5, 3.00001e-5, 1.0009766, 1.0004883, 1.0014648, 0.1, -0.3333, 20.0, 19.99]
    xs = rand_floats(0x5151, 400)
    vals += [float(F(x) * F(10.0)) for x in xs[:200]] + [float(F(x) * F(1e-4)) for x in xs[200:]]
    vin = np.array(vals, dtype=np.float32)
    g["f16_in"] = vin.view(np.uint32)
    g["f16_out"] = np.array([f32_to_half(v) for v in vin], dtype=np.uint16)
    hs = np.array([0x0000, 0x0001, 0x03FF, 0x0400, 0x3C00, 0xC000, 0x3800, 0x7BFF, 0x7C00, 0xFC00,
                   0x8001, 0x0200, 0x1234, 0xABCD], dtype=np.uint16)
    g["half_in"] = hs
    g["half_out"] = np.array([half_to_f32(int(h)) for h in hs], dtype=np.float32).view(np.uint32)

    # rope: text positions and one mixed-position case (sections matter there)
    head = rand_floats(0x7777, 2 * HD)
    rope_pos = [(0, 0, 0, 0), (5, 5, 5, 5), (17, 17, 17, 17), (37, 37, 37, 37), (4096, 4096, 4096, 4096),
                (131071, 131071, 131071, 131071), (262143, 262143, 262143, 262143), (3, 5, 7, 0)]
    g["rope_in"] = head.view(np.uint32)
    g["rope_pos"] = np.array(rope_pos, dtype=np.int64)
    g["rope_out"] = np.stack([
        np.concatenate([rope_imrope(head[h * HD:(h + 1) * HD], *p, N_ROT, SECTIONS, FREQ_BASE) for h in range(2)])
        for p in rope_pos]).view(np.uint32)

    # quantize: every width, vectors of several scales incl. an outlier channel and zeros
    qx = rand_floats(0xBEEF, 6 * HD).reshape(6, HD).copy()
    qx[1] *= F(16.0)
    qx[2, 17] *= F(20.0); qx[2, 200] *= F(20.0)
    qx[3] *= F(1e-3)
    qx[4] = 0.0
    qx[5] *= F(1e-14)
    g["quant_in"] = qx.view(np.uint32)
    for bits in range(1, 9):
        cb, _ = codebook(HD, bits)
        rows, norms = [], []
        for r in range(qx.shape[0]):
            p, n = quantize(qx[r], cb, giv, bits)
            rows.append(p); norms.append(n)
        g[f"quant_bytes_b{bits}"] = np.stack(rows)
        g[f"quant_norm_b{bits}"] = np.array(norms, dtype=np.float32).view(np.uint32)

    # softmax
    sx = np.array([1.0, 2.0, 3.0, -np.inf, 0.0, 0.0, 0.0, 0.0], dtype=np.float32)
    g["softmax_in"] = sx
    g["softmax_out"] = np.concatenate([softmax_row(sx[:4]), softmax_row(sx[4:])]).view(np.uint32)

    # attention steps from an empty cache, 3 tokens, every store mode
    for tag, (mode, bits, vq) in {"f32": ("f32", 0, False), "f16": ("f16", 0, False),
                                  "planar4": ("planar", 4, True), "planar3": ("planar", 3, True),
                                  "planar4k": ("planar", 4, False)}.items():
        outs, ks, vs, kn, vn = attention_steps(mode, bits, vq, 3, 0xA000)
        g[f"attn_{tag}_out"] = outs.view(np.uint32)
        g[f"attn_{tag}_k"] = np.stack(ks)
        g[f"attn_{tag}_v"] = np.stack(vs)
        if kn:
            g[f"attn_{tag}_kn"] = np.array(kn, dtype=np.float32).view(np.uint32)
        if vn:
            g[f"attn_{tag}_vn"] = np.array(vn, dtype=np.float32).view(np.uint32)
        print("attention", tag, "done", flush=True)

    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kvpath_golden.npz")
    np.savez_compressed(out, **g)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
