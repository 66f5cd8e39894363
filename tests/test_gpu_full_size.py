"""Parity at the benchmark's full sizes (one layer), through the C ABI.

Config 3: planar4 cache at context 131072, N(0,1) K/V with 1 % of the channels x20.  The whole
cache is built by the fused append in bulk calls; the checks are (a) stored bytes of sampled
rows against the oracle's encoder, (b) the decode output against the oracle over the full
context (a few seconds of CPU), (c) size-independent properties: attending over the two halves
separately and merging gives the whole; appending in bulk calls or token by token stores the
same rows.  Config 2's f16 cache at 32768 and config 1's f32 cache at 4096 get the same
treatment at their sizes.
"""
import numpy as np
import pytest

from oracle_lib import MODE_F16, MODE_F32, MODE_PLANAR

pytestmark = pytest.mark.gpu

HD, NKV, NH = 256, 4, 24


def synth(rng, n):
    k = rng.standard_normal((n, NKV, HD), dtype=np.float32)
    v = rng.standard_normal((n, NKV, HD), dtype=np.float32)
    ch = rng.choice(HD, size=3, replace=False)
    k[:, :, ch] *= np.float32(20.0)
    v[:, :, ch] *= np.float32(20.0)
    return k, v


def close(got, want):
    err = float(np.max(np.abs(got.astype(np.float64) - want)))
    return err, err / max(float(np.max(np.abs(want))), 1e-30)


@pytest.mark.parametrize("tag,mode,bits,vq,n_ctx", [("planar4", MODE_PLANAR, 4, True, 131072),
                                                   ("f16", MODE_F16, 0, False, 32768),
                                                   ("f32", MODE_F32, 0, False, 4097)])
def test_full_size_layer(bk, gpu_ctx, oracle, tag, mode, bits, vq, n_ctx):
    rng = np.random.default_rng(2024)
    k, v = synth(rng, n_ctx)
    q = rng.standard_normal((NH, HD), dtype=np.float32)
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_ctx=n_ctx)
    for p0 in range(0, n_ctx, 8192):
        cache.append(0, k[p0:p0 + 8192], v[p0:p0 + 8192])
    assert cache.n_pos(0) == n_ctx

    # (a) + (b): the oracle builds the same cache (every row) and attends over all of it
    ref = oracle.cache(mode, bits, vq)
    for p in range(n_ctx):
        ref.append(0, k[p], v[p], p)
    sample = np.unique(np.concatenate([rng.integers(0, n_ctx, 61), [0, n_ctx - 1, n_ctx // 2]]))
    rd = ref.dump(0)
    for p in sample:
        gd = cache.dump_kv(0, n_pos=1, pos0=int(p))
        for key, val in rd.items():
            assert np.array_equal(gd[key][0].view(np.uint8), val[p].view(np.uint8)), (key, int(p))
    # checksum of checksums over every stored byte
    whole = cache.dump_kv(0)
    for key, val in rd.items():
        assert int(whole[key].view(np.uint8).astype(np.uint64).sum()) == int(val.view(np.uint8).astype(np.uint64).sum()), key
    got = cache.attend(0, q)[0]
    want = ref.attend(0, q, n_ctx - 1, n_ctx, threads=16)
    err, rel = close(got, want)
    assert err <= 1e-3 and rel <= 1e-3, (tag, err, rel)

    # (c) split invariance: two halves + log-sum-exp merge == whole
    half = n_ctx // 2
    lo = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_ctx=half, rope_positions=n_ctx)
    hi = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_ctx=n_ctx - half, rope_positions=n_ctx)
    lo.upload_kv(0, {key: val[:half] for key, val in whole.items()})
    hi.upload_kv(0, {key: val[half:] for key, val in whole.items()})
    lo.set_n_pos(0, 0, half)
    hi.set_n_pos(0, 0, n_ctx - half)
    parts = np.stack([lo.attend(0, q, q_pos=[n_ctx - 1], partial=True)[0],
                      hi.attend(0, q, q_pos=[n_ctx - 1], partial=True)[0]])
    dparts, dout = gpu_ctx.to_device(parts), gpu_ctx.alloc(NH * HD * 4)
    gpu_ctx.check(gpu_ctx.lib.bk_lse_merge(gpu_ctx.h, 2, NH, HD, dparts.ptr, dout.ptr))
    merged = dout.download((NH, HD), np.float32)
    err2, rel2 = close(merged, got.astype(np.float64))
    assert err2 <= 2e-4 and rel2 <= 2e-4, (tag, err2, rel2)
    for c in (cache, lo, hi):
        c.close()


def test_bulk_and_single_appends_store_the_same_rows(bk, gpu_ctx):
    rng = np.random.default_rng(7)
    k, v = synth(rng, 4096)
    a = bk.AttnCache(gpu_ctx, bk.parse_mode("planar4"), n_layers=1, n_ctx=4096)
    b = bk.AttnCache(gpu_ctx, bk.parse_mode("planar4"), n_layers=1, n_ctx=4096)
    a.append(0, k, v)                                  # one call of 4096 tokens
    for n0, n1 in ((0, 1), (1, 3), (3, 100), (100, 101), (101, 4096)):
        b.append(0, k[n0:n1], v[n0:n1])                # ragged calls, incl. single tokens
    da, db = a.dump_kv(0), b.dump_kv(0)
    for key in da:
        assert np.array_equal(da[key].view(np.uint8), db[key].view(np.uint8)), key
    a.close()
    b.close()
