#!/usr/bin/env python3
"""Golden vectors for the layer form of the attention step (q|gate split, per-head RMSNorm,
attention, sigmoid gate), from a Python restatement that shares no code with the C oracle:

  src/kernels.rs:97-122   rms_norm_rows (sequential f32 sum, 1/sqrt(ss/n + eps), x*scale*w)
  src/kernels.rs:162-164  sigmoid
  src/forward.rs:237-245  split [q | gate] per head, RMSNorm of q and k
  src/forward.rs:379-382  out *= sigmoid(gate)

The attention core in between is gen_golden.attention_steps.  Every f32 operation is a numpy
float32 scalar operation; exp comes from the C library through ctypes, like the reference's.
Writes layer_golden.npz beside this file.  Run:  python tests/golden/gen_layer_golden.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from gen_golden import HD, N_HEAD, N_KV, F, attention_steps, expf, rand_floats  # noqa: E402

EPS = F(1e-6)


def rms_norm_rows(x, w, row_len, eps):
    out = np.zeros(len(x), dtype=np.float32)
    for r in range(len(x) // row_len):
        src = x[r * row_len:(r + 1) * row_len]
        ss = F(0.0)
        for v in src:
            ss = F(ss + F(v * v))
        scale = F(F(1.0) / F(np.sqrt(F(F(ss / F(row_len)) + eps))))
        for i in range(row_len):
            out[r * row_len + i] = F(F(src[i] * scale) * w[i])
    return out


def sigmoid(x):
    return F(F(1.0) / F(F(1.0) + expf(F(-x))))


def layer_steps(mode, bits, v_quant, n_tokens, seed):
    qw = F(1.0) + F(0.25) * rand_floats(seed + 101, HD)
    kw = F(1.0) + F(0.25) * rand_floats(seed + 102, HD)
    qfulls, kraws, vraws, gates = [], [], [], []

    def inputs(pos):
        qfull = F(3.0) * rand_floats(seed + 3 * pos, N_HEAD * 2 * HD)
        kraw = F(2.0) * rand_floats(seed + 3 * pos + 1, N_KV * HD)
        vraw = rand_floats(seed + 3 * pos + 2, N_KV * HD)
        q = np.concatenate([qfull[h * 2 * HD:h * 2 * HD + HD] for h in range(N_HEAD)])
        gate = np.concatenate([qfull[h * 2 * HD + HD:(h + 1) * 2 * HD] for h in range(N_HEAD)])
        qfulls.append(qfull); kraws.append(kraw); vraws.append(vraw); gates.append(gate)
        return rms_norm_rows(q, qw, HD, EPS), rms_norm_rows(kraw, kw, HD, EPS), vraw

    outs, ks, vs, kn, vn = attention_steps(mode, bits, v_quant, n_tokens, seed, inputs=inputs)
    gated = np.zeros_like(outs)
    for t in range(n_tokens):
        for i in range(N_HEAD * HD):
            gated[t, i] = F(outs[t, i] * sigmoid(gates[t][i]))
    return dict(qw=qw, kw=kw, qfull=np.stack(qfulls), kraw=np.stack(kraws), vraw=np.stack(vraws), out=gated,
                k=np.stack(ks), v=np.stack(vs), kn=np.array(kn, dtype=np.float32), vn=np.array(vn, dtype=np.float32))


def main():
    g = {}
    # the reference's own unit-test vector (src/kernels.rs:790-811) and seeded head-sized rows
    x = np.array([1.0, 2.0, 3.0, 4.0, 0.5, -0.5, 2.0, -3.0], dtype=np.float32)
    w = np.array([0.5, 1.0, 1.5, 2.0], dtype=np.float32)
    g["rms_small_x"], g["rms_small_w"] = x, w
    g["rms_small_out"] = rms_norm_rows(x, w, 4, EPS).view(np.uint32)
    xr = F(5.0) * rand_floats(0x5151, 6 * HD)
    xr[2 * HD:3 * HD] = 0.0            # a zero row: scale = 1/sqrt(eps)
    xr[3 * HD:4 * HD] *= F(1e-20)      # squares underflow
    wr = F(1.0) + F(0.5) * rand_floats(0x5252, HD)
    g["rms_rows_x"], g["rms_rows_w"] = xr.view(np.uint32), wr.view(np.uint32)
    g["rms_rows_out"] = rms_norm_rows(xr, wr, HD, EPS).view(np.uint32)
    sx = np.array([0.0, -1000.0, 1000.0, 1.0, -1.0, 0.3, -7.5, 20.0, -88.0, -104.0], dtype=np.float32)
    g["sigmoid_in"] = sx
    g["sigmoid_out"] = np.array([sigmoid(v) for v in sx], dtype=np.float32).view(np.uint32)
    for tag, (mode, bits, vq) in {"planar4": ("planar", 4, True), "f16": ("f16", 0, False)}.items():
        r = layer_steps(mode, bits, vq, 3, 0xB000)
        for key, val in r.items():
            g[f"layer_{tag}_{key}"] = val.view(np.uint32) if val.dtype == np.float32 else val
        print("layer", tag, "done", flush=True)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "layer_golden.npz")
    np.savez_compressed(out, **g)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
