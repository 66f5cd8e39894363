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
    assert err2 <= 2e-4 and rel2 <= 3e-4, (tag, err2, rel2)  # two GPU results, each ~1e-4 from the oracle
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


def test_config4_batched_step_64_sequences(bk, gpu_ctx, oracle):
    """Config 4 at full size, one layer: 64 independent planar4 sequences, contexts U[2048,16384]
    (seeded), one bk_attn_step_batch step.  The new row of EVERY sequence is bit-compared with the
    oracle's encoder and the rows before it must be untouched (byte checksums before and after);
    for a seeded sample of 8 sequences the oracle rebuilds the whole cache (every stored byte
    compared) and runs the step (outputs at 1e-3); the other sequences' outputs are cross-checked
    against single-sequence decode calls.  Oracle: src/forward.rs:247-375 per sequence."""
    rng = np.random.default_rng(4)
    n_seqs = 64
    lens = rng.integers(2048, 16385, n_seqs)
    pool_k, pool_v = synth(rng, int(lens.max()) + 1024)
    offs = [(int(i) * 131) % 1000 for i in range(n_seqs)]   # every sequence is its own slice of the pool
    n_ctx = int(lens.max()) + 1
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode("planar4"), n_layers=1, n_seqs=n_seqs, n_ctx=n_ctx)
    for i in range(n_seqs):
        cache.append(0, pool_k[offs[i]:offs[i] + lens[i]], pool_v[offs[i]:offs[i] + lens[i]], seq=i)

    def checksums(seq, n):
        d = cache.dump_kv(0, n_pos=n, seq=seq)
        return {key: int(val.view(np.uint8).astype(np.uint64).sum()) for key, val in d.items()}

    before = [checksums(i, int(lens[i])) for i in range(n_seqs)]
    k_new = rng.standard_normal((n_seqs, NKV, HD), dtype=np.float32)
    v_new = rng.standard_normal((n_seqs, NKV, HD), dtype=np.float32)
    q = rng.standard_normal((n_seqs, NH, HD), dtype=np.float32)
    dq, dk, dv = gpu_ctx.to_device(q), gpu_ctx.to_device(k_new), gpu_ctx.to_device(v_new)
    dout = gpu_ctx.alloc(n_seqs * NH * HD * 4)
    launches = gpu_ctx.launch_count
    cache.step_batch_device(0, dq.ptr, dk.ptr, dv.ptr, dout.ptr, n_seqs)
    out = dout.download((n_seqs, NH, HD), np.float32)
    assert gpu_ctx.launch_count - launches == 1          # all 64 appends and decodes in one launch

    sample = set(int(x) for x in rng.choice(n_seqs, 8, replace=False))
    worst = 0.0
    for i in range(n_seqs):
        n = int(lens[i])
        assert cache.n_pos(0, i) == n + 1
        assert checksums(i, n) == before[i], f"rows of sequence {i} changed"
        one = oracle.cache(MODE_PLANAR, 4, True)            # the new row alone: rope position n
        one.append(0, k_new[i], v_new[i], n)
        got_row, want_row = cache.dump_kv(0, n_pos=1, seq=i, pos0=n), one.dump(0)
        for key, val in want_row.items():
            assert np.array_equal(got_row[key][0].view(np.uint8), val[0].view(np.uint8)), (key, i)
        if i in sample:
            ref = oracle.cache(MODE_PLANAR, 4, True)
            for p in range(n):
                ref.append(0, pool_k[offs[i] + p], pool_v[offs[i] + p], p)
            want = ref.step(0, q[i], k_new[i], v_new[i], n, threads=16)
            whole, rd = cache.dump_kv(0, seq=i), ref.dump(0)
            for key, val in rd.items():
                assert np.array_equal(whole[key].view(np.uint8), val.view(np.uint8)), (key, i)
            err, rel = close(out[i], want.astype(np.float64))
            assert err <= 1e-3 and rel <= 1e-3, (i, n, err, rel)
            worst = max(worst, err)
        else:
            alone = cache.attend(0, q[i:i + 1], seq_ids=[i])[0]
            err, rel = close(out[i], alone.astype(np.float64))
            assert err <= 3e-4 and rel <= 3e-4, (i, n, err, rel)
    cache.close()


def test_config5_context_262144_and_chunk_merges(bk, gpu_ctx, oracle):
    """Config 5 on one GPU, one layer: a planar4 cache of 262144 rows.  bk_attn_step (fused append +
    decode) against the oracle at the full depth, then the context cut into 2, 4 and 8 chunks held
    by separate caches, each scanned with bk_decode_attn_partial and merged with bk_lse_merge: the
    merge must give the whole (what the per-GPU chunks of the split-context configuration compute).
    Oracle: src/forward.rs:287-375."""
    rng = np.random.default_rng(5)
    n_ctx = 262144
    k, v = synth(rng, n_ctx)
    q = rng.standard_normal((NH, HD), dtype=np.float32)
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode("planar4"), n_layers=1, n_ctx=n_ctx)
    ref = oracle.cache(MODE_PLANAR, 4, True)
    for p0 in range(0, n_ctx - 1, 8192):
        p1 = min(p0 + 8192, n_ctx - 1)
        cache.append(0, k[p0:p1], v[p0:p1])
    for p in range(n_ctx - 1):
        ref.append(0, k[p], v[p], p)
    got = bk.full_attention_step(cache, 0, q, k[n_ctx - 1], v[n_ctx - 1], n_ctx - 1)
    want = ref.step(0, q, k[n_ctx - 1], v[n_ctx - 1], n_ctx - 1, threads=16)
    err, rel = close(got, want.astype(np.float64))
    assert err <= 1e-3 and rel <= 1e-3, (err, rel)
    whole, rd = cache.dump_kv(0), ref.dump(0)
    for key, val in rd.items():   # every stored byte, the fused append's row included
        assert np.array_equal(whole[key].view(np.uint8), val.view(np.uint8)), key
    for parts in (2, 4, 8):
        bounds = [n_ctx * i // parts for i in range(parts + 1)]
        rows = []
        for b, e in zip(bounds[:-1], bounds[1:]):
            c = bk.AttnCache(gpu_ctx, bk.parse_mode("planar4"), n_layers=1, n_ctx=e - b, rope_positions=n_ctx)
            c.upload_kv(0, {key: val[b:e] for key, val in whole.items()})
            c.set_n_pos(0, 0, e - b)
            rows.append(c.attend(0, q, q_pos=[n_ctx - 1], partial=True)[0])
            c.close()
        dparts, dout = gpu_ctx.to_device(np.stack(rows)), gpu_ctx.alloc(NH * HD * 4)
        gpu_ctx.check(gpu_ctx.lib.bk_lse_merge(gpu_ctx.h, parts, NH, HD, dparts.ptr, dout.ptr))
        merged = dout.download((NH, HD), np.float32)
        err2, rel2 = close(merged, got.astype(np.float64))
        assert err2 <= 2e-4 and rel2 <= 5e-4, (parts, err2, rel2)   # two GPU results, each about 1e-4 from the oracle
        err3, rel3 = close(merged, want.astype(np.float64))
        assert err3 <= 1e-3 and rel3 <= 1e-3, (parts, err3, rel3)
    cache.close()
