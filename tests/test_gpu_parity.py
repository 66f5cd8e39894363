"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Bars: stored bytes (packed indices, norm bits, f16 bits, f32 bits) are bit-exact; attention
outputs are within max-abs 1e-3 and max-abs / max|reference| 1e-3 (the reference's own `rel`
measure, src/bin/bonsai-golden.rs:150-166) of the oracle's f32 path.
"""
import numpy as np
import pytest

from oracle_lib import MODE_F16, MODE_F32, MODE_PLANAR

pytestmark = pytest.mark.gpu

HD, NKV, NH = 256, 4, 24
ABS_TOL = 1e-3
REL_TOL = 1e-3

MODES = [("f32", MODE_F32, 0, False), ("f16", MODE_F16, 0, False), ("planar4", MODE_PLANAR, 4, True),
         ("planar3", MODE_PLANAR, 3, True), ("planar4k", MODE_PLANAR, 4, False), ("planar8", MODE_PLANAR, 8, True),
         ("planar1", MODE_PLANAR, 1, True), ("planar2", MODE_PLANAR, 2, True), ("planar5", MODE_PLANAR, 5, True),
         ("planar6k", MODE_PLANAR, 6, False), ("planar7", MODE_PLANAR, 7, True)]


def bits_of(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_close(got, want, what=""):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    max_abs = np.max(np.abs(got - want))
    scale = max(np.max(np.abs(want)), 1e-30)
    assert max_abs <= ABS_TOL and max_abs / scale <= REL_TOL, f"{what}: max_abs {max_abs:.3e}, rel {max_abs / scale:.3e}"


def synth_kv(rng, n, outliers=True):
    """N(0,1) rows with 1 % of the 256 channels (3 of them, seeded) scaled x20."""
    k = rng.standard_normal((n, NKV, HD)).astype(np.float32)
    v = rng.standard_normal((n, NKV, HD)).astype(np.float32)
    if outliers:
        ch = rng.choice(HD, size=3, replace=False)
        k[:, :, ch] *= np.float32(20.0)
        v[:, :, ch] *= np.float32(20.0)
    return k, v


def compare_dumps(gpu_dump, ref_dump):
    assert sorted(gpu_dump) == sorted(ref_dump)
    for key, ref in ref_dump.items():
        got = gpu_dump[key]
        assert got.shape == ref.shape, key
        if ref.dtype == np.float32:
            assert np.array_equal(bits_of(got), bits_of(ref)), f"{key}: f32 bits differ"
        else:
            assert np.array_equal(got, ref), f"{key}: bytes differ"


# ---------------------------------------------------------------------------
# kvquant.rs entry points
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("bits", range(1, 9))
def test_quantize_bytes_and_norm_bits(bk, gpu_ctx, oracle, golden, bits):
    pq = bk.PlanarQuant(HD, bits, gpu_ctx)
    opq = oracle.pq(HD, bits)
    rng = np.random.default_rng(100 + bits)
    x = np.concatenate([golden["quant_in"].view(np.float32),
                        oracle.rand_floats(11, 64 * HD).reshape(64, HD),
                        synth_kv(rng, 40)[0].reshape(-1, HD)])
    packed, norms = pq.quantize(x)
    for r in range(x.shape[0]):
        p_ref, n_ref = opq.quantize(x[r])
        assert np.array_equal(packed[r], p_ref), (bits, r)
        assert bits_of(norms[r]) == bits_of(n_ref), (bits, r)
    g = golden["quant_in"].shape[0]
    assert np.array_equal(packed[:g], golden[f"quant_bytes_b{bits}"])
    assert np.array_equal(bits_of(norms[:g]), golden[f"quant_norm_b{bits}"])


@pytest.mark.parametrize("bits", [1, 3, 4, 7, 8])
def test_dequantize_rotate_dot_rotated_exact(bk, gpu_ctx, oracle, bits):
    pq, opq = bk.PlanarQuant(HD, bits, gpu_ctx), oracle.pq(HD, bits)
    x = oracle.rand_floats(23 + bits, 8 * HD).reshape(8, HD)
    q = oracle.rand_floats(57 + bits, 8 * HD).reshape(8, HD)
    packed, norms = pq.quantize(x)
    deq, rot, inv = pq.dequantize(packed, norms), pq.rotate(q), pq.rotate_inv(q)
    dots = pq.dot_rotated(rot, packed, norms)
    for r in range(8):
        assert np.array_equal(bits_of(deq[r]), bits_of(opq.dequantize(packed[r], norms[r])))
        assert np.array_equal(bits_of(rot[r]), bits_of(opq.rotate(q[r])))
        assert np.array_equal(bits_of(inv[r]), bits_of(opq.rotate_inv(q[r])))
        assert bits_of(dots[r]) == bits_of(opq.dot_rotated(rot[r], packed[r], norms[r]))


def test_reference_unit_tests_through_the_abi(bk, gpu_ctx, oracle):
    """src/kvquant.rs:631-667, 723-738 run against the GPU entry points."""
    p = bk.PlanarQuant(HD, 4, gpu_ctx)
    x = oracle.rand_floats(7, HD)
    assert np.max(np.abs(p.rotate_inv(p.rotate(x)) - x)) < 1e-5            # givens_is_orthogonal
    xs = oracle.rand_floats(11, 64 * HD).reshape(64, HD)                   # quantize_roundtrip_error_is_small
    packed, norms = p.quantize(xs)
    y = p.dequantize(packed, norms)
    rel = np.sqrt(((xs - y) ** 2).sum(1)) / np.maximum(np.sqrt((xs * xs).sum(1)), 1e-9)
    assert rel.max() < 0.12
    s = oracle.rand_floats(23, 2 * HD)                                      # dot_rotated_matches_dequantized_dot
    k, q = s[:HD], s[HD:]
    pk, nk = p.quantize(k)
    a = p.dot_rotated(p.rotate(q), pk, nk)
    assert abs(a - float(np.dot(q.astype(np.float64), p.dequantize(pk, nk).astype(np.float64)))) < 1e-4


def test_rope_bits(bk, gpu_ctx, oracle, golden):
    head = golden["rope_in"].view(np.float32).reshape(2, HD)
    for pos, want in zip(golden["rope_pos"], golden["rope_out"]):
        got = bk.rope_imrope(head, *[int(p) for p in pos], ctx=gpu_ctx)
        assert np.array_equal(bits_of(got.ravel()), want), pos
    # the reference's check_rope recipe (src/bin/bonsai-vk.rs:237-269): 24 heads, pos 37
    heads = oracle.rand_floats(0x7777, NH * HD).reshape(NH, HD)
    got = bk.rope_imrope(heads, 37, 37, 37, 37, ctx=gpu_ctx)
    for h in range(NH):
        assert np.array_equal(bits_of(got[h]), bits_of(oracle.rope(heads[h], 37, 37, 37, 37)))
    # other geometry: n_dims 8, sections [2,1,1,0], base 1e4 (the reference's mini config)
    small = oracle.rand_floats(0x99, 3 * 16).reshape(3, 16)
    got = bk.rope_imrope(small, 3, 5, 7, 2, n_dims=8, sections=(2, 1, 1, 0), freq_base=1e4, ctx=gpu_ctx)
    for h in range(3):
        want = oracle.rope(small[h], 3, 5, 7, 2, n_dims=8, sections=np.array([2, 1, 1, 0], np.int32), freq_base=1e4)
        assert np.array_equal(bits_of(got[h]), bits_of(want))


def test_f16_conversions(bk, gpu_ctx, oracle, golden):
    vin = golden["f16_in"].view(np.float32)
    assert np.array_equal(bk.f32_to_half(vin, gpu_ctx), golden["f16_out"])
    back = bk.half_to_f32(golden["half_in"], gpu_ctx)
    assert np.array_equal(bits_of(back), golden["half_out"])
    # every f16 bit pattern widens like the reference (NaNs: only NaN-ness is compared)
    allh = np.arange(65536, dtype=np.uint16)
    got = bk.half_to_f32(allh, gpu_ctx)
    ref = np.array([oracle.lib.or_half_to_f32(int(h)) for h in allh], np.float32)
    nan = np.isnan(ref)
    assert np.array_equal(np.isnan(got), nan) and np.array_equal(bits_of(got[~nan]), bits_of(ref[~nan]))
    # the reference's subnormal rule (shift, then round) on a dense sweep below 2^-14
    rng = np.random.default_rng(5)
    tiny = (rng.standard_normal(20000) * 2.0 ** rng.integers(-30, -12, 20000)).astype(np.float32)
    ref = np.array([oracle.lib.or_f32_to_half(float(v)) for v in tiny], np.uint16)
    assert np.array_equal(bk.f32_to_half(tiny, gpu_ctx), ref)


# ---------------------------------------------------------------------------
# append: stored bytes are bit-exact
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("tag,mode,bits,vq", MODES)
def test_append_bytes_bit_exact(bk, gpu_ctx, oracle, tag, mode, bits, vq):
    n = 70
    rng = np.random.default_rng(7)
    k, v = synth_kv(rng, n)
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=2, n_seqs=1, n_ctx=128)
    ref = oracle.cache(mode, bits, vq)
    for p in range(n):
        ref.append(0, k[p], v[p], p)
    # tokens 0..9 one call each, then a bulk call of 60 (both routes must give the same rows)
    for p in range(10):
        cache.append(1, k[p], v[p])
    cache.append(1, k[10:], v[10:])
    assert cache.n_pos(1) == n and cache.n_pos(0) == 0
    compare_dumps(cache.dump_kv(1), ref.dump(0))
    cache.close()


def test_append_golden_rows(bk, gpu_ctx, oracle, golden):
    """Rows stored by three decode steps equal the independent restatement's fixture."""
    for tag in ("f32", "f16", "planar4", "planar3", "planar4k"):
        cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_ctx=16)
        want = golden[f"attn_{tag}_out"]
        for pos in range(want.shape[0]):
            q = oracle.rand_floats(0xA000 + 3 * pos, NH * HD)
            k = oracle.rand_floats(0xA000 + 3 * pos + 1, NKV * HD)
            v = oracle.rand_floats(0xA000 + 3 * pos + 2, NKV * HD)
            out = bk.full_attention_step(cache, 0, q, k, v, pos)
            assert_close(out.ravel(), want[pos].view(np.float32), f"{tag} step {pos}")
        d = cache.dump_kv(0)
        n = want.shape[0]
        gk, gv = golden[f"attn_{tag}_k"], golden[f"attn_{tag}_v"]
        if tag.startswith("planar"):
            assert np.array_equal(d["kq"].reshape(n * NKV, -1), gk)
            assert np.array_equal(bits_of(d["kn"].ravel()), golden[f"attn_{tag}_kn"])
            if tag.endswith("k"):
                assert np.array_equal(bits_of(d["v"].reshape(n * NKV, -1)), bits_of(gv))
            else:
                assert np.array_equal(d["vq"].reshape(n * NKV, -1), gv)
                assert np.array_equal(bits_of(d["vn"].ravel()), golden[f"attn_{tag}_vn"])
        elif tag == "f16":
            assert np.array_equal(d["k16"].reshape(n * NKV, -1), gk) and np.array_equal(d["v16"].reshape(n * NKV, -1), gv)
        else:
            assert np.array_equal(bits_of(d["k"].reshape(n * NKV, -1)), bits_of(gk))
        cache.close()


def test_append_special_vectors(bk, gpu_ctx, oracle):
    """Zero vectors, tiny norms (inv = 0 branch), huge norms, f16 overflow and subnormals."""
    k = np.zeros((6, NKV, HD), np.float32)
    v = np.zeros((6, NKV, HD), np.float32)
    r = oracle.rand_floats(0x42, 6 * NKV * HD).reshape(6, NKV, HD)
    k[1], v[1] = r[1] * np.float32(1e-14), r[1] * np.float32(1e-20)
    k[2], v[2] = r[2] * np.float32(1e18), r[2] * np.float32(7e4)
    k[3], v[3] = r[3] * np.float32(3e-6), r[3] * np.float32(6e-8)
    k[4], v[4] = r[4], -r[4]
    k[5, :, 0], v[5, :, 255] = 1.0, -1.0
    for tag, mode, bits, vq in MODES[:5]:
        cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_ctx=8)
        ref = oracle.cache(mode, bits, vq)
        for p in range(6):
            ref.append(0, k[p], v[p], p)
        cache.append(0, k, v)
        compare_dumps(cache.dump_kv(0), ref.dump(0))
        cache.close()


def test_append_at_far_positions(bk, gpu_ctx, oracle):
    """Rope positions up to the 262144-token training context; rows land at the next index."""
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode("planar4"), n_layers=1, n_ctx=8, rope_positions=262144)
    ref = oracle.cache(MODE_PLANAR, 4, True)
    rng = np.random.default_rng(3)
    k, v = synth_kv(rng, 4)
    for i, pos in enumerate([0, 4096, 131071, 262143]):
        ref.append(0, k[i], v[i], pos)
        cache.append(0, k[i], v[i], pos=pos)
    compare_dumps(cache.dump_kv(0), ref.dump(0))
    cache.close()


def test_append_batch_many_sequences(bk, gpu_ctx, oracle):
    """One token for each of several sequences per launch, ragged lengths."""
    n_seqs = 5
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode("planar3"), n_layers=2, n_seqs=n_seqs, n_ctx=16)
    refs = [oracle.cache(MODE_PLANAR, 3, True) for _ in range(n_seqs)]
    rng = np.random.default_rng(11)
    lens = [3, 0, 7, 1, 5]
    for s, n in enumerate(lens):  # ragged prefill
        if n:
            k, v = synth_kv(rng, n)
            cache.append(1, k, v, seq=s)
            for p in range(n):
                refs[s].append(0, k[p], v[p], p)
    for _ in range(3):  # three batched steps over a subset, in a scrambled order
        ids = [4, 0, 2, 1]
        k, v = synth_kv(rng, len(ids))
        dk, dv = gpu_ctx.to_device(k), gpu_ctx.to_device(v)
        cache.append_batch_device(1, dk.ptr, dv.ptr, len(ids), seq_ids=ids)
        gpu_ctx.synchronize()
        for i, s in enumerate(ids):
            refs[s].append(0, k[i], v[i], refs[s].n_pos(0))
    for s in range(n_seqs):
        assert cache.n_pos(1, s) == refs[s].n_pos(0)
        if refs[s].n_pos(0):
            compare_dumps(cache.dump_kv(1, seq=s), refs[s].dump(0))
    cache.close()


def test_context_exhaustion_is_an_error(bk, gpu_ctx):
    """src/gdev.rs:907-912: a position beyond n_ctx fails instead of wrapping."""
    cache = bk.AttnCache(gpu_ctx, bk.F32, n_layers=1, n_ctx=4)
    z = np.zeros((4, NKV, HD), np.float32)
    cache.append(0, z, z)
    with pytest.raises(bk.BonsaiKvError) as e:
        cache.append(0, z[0], z[0])
    assert e.value.status == bk._abi.BK_ERR_RANGE and "BONSAI_CTX" in str(e.value)
    with pytest.raises(bk.BonsaiKvError):
        cache.step(0, np.zeros(NH * HD, np.float32), z[0], z[0], 4)
    cache.reset()
    assert cache.n_pos(0) == 0
    with pytest.raises(bk.BonsaiKvError) as e:  # the step must target the next row
        cache.step(0, np.zeros(NH * HD, np.float32), z[0], z[0], 2)
    assert e.value.status == bk._abi.BK_ERR_INVALID
    cache.close()


def test_unsupported_geometry_is_refused(bk, gpu_ctx):
    with pytest.raises(bk.BonsaiKvError) as e:
        bk.AttnCache(gpu_ctx, bk.F32, n_layers=1, n_ctx=4, hd=128)
    assert e.value.status == bk._abi.BK_ERR_UNSUPPORTED
    with pytest.raises(bk.BonsaiKvError):
        bk.AttnCache(gpu_ctx, bk.KvMode("planar", 9, True), n_layers=1, n_ctx=4)


def test_snapshot_roundtrip(bk, gpu_ctx):
    """dump_kv -> upload_kv into a fresh cache gives identical rows and identical attention."""
    rng = np.random.default_rng(21)
    k, v = synth_kv(rng, 50)
    q = rng.standard_normal((NH, HD)).astype(np.float32)
    a = bk.AttnCache(gpu_ctx, bk.parse_mode("planar4"), n_layers=1, n_ctx=64)
    a.append(0, k, v)
    rows = a.dump_kv(0)
    b = bk.AttnCache(gpu_ctx, bk.parse_mode("planar4"), n_layers=1, n_ctx=64)
    b.upload_kv(0, rows)
    b.set_n_pos(0, 0, 50)
    compare_dumps(b.dump_kv(0), rows)
    assert np.array_equal(a.attend(0, q), b.attend(0, q))
    a.close()
    b.close()


# ---------------------------------------------------------------------------
# decode attention
# ---------------------------------------------------------------------------

def run_both(bk, gpu_ctx, oracle, tag, mode, bits, vq, n_pos_list, seed=0, outliers=True, n_ctx=None):
    """Prefill several sequences, attend once per sequence on both paths, compare."""
    rng = np.random.default_rng(seed)
    n_seqs = len(n_pos_list)
    n_ctx = n_ctx or max(max(n_pos_list), 1)
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_seqs=n_seqs, n_ctx=n_ctx)
    q = rng.standard_normal((n_seqs, NH, HD)).astype(np.float32)
    want = np.zeros((n_seqs, NH, HD), np.float32)
    for s, n in enumerate(n_pos_list):
        if n == 0:
            continue
        k, v = synth_kv(rng, n, outliers)
        cache.append(0, k, v, seq=s)
        ref = oracle.cache(mode, bits, vq)
        for p in range(n):
            ref.append(0, k[p], v[p], p)
        want[s] = ref.attend(0, q[s], n - 1, n, threads=8)
    got = cache.attend(0, q, n_seqs=n_seqs)
    cache.close()
    return got, want


@pytest.mark.parametrize("tag,mode,bits,vq", MODES)
def test_decode_matches_oracle(bk, gpu_ctx, oracle, tag, mode, bits, vq):
    got, want = run_both(bk, gpu_ctx, oracle, tag, mode, bits, vq, [600], seed=1)
    assert_close(got, want, tag)


@pytest.mark.parametrize("n_pos", [1, 2, 7, 8, 9, 37, 63, 64, 65, 127, 129, 1000])
def test_decode_ragged_lengths(bk, gpu_ctx, oracle, n_pos):
    for tag, mode, bits, vq in MODES[:3]:
        got, want = run_both(bk, gpu_ctx, oracle, tag, mode, bits, vq, [n_pos], seed=n_pos)
        assert_close(got, want, f"{tag} n_pos={n_pos}")


def test_decode_long_context_split_k(bk, gpu_ctx, oracle):
    """Enough positions for many chunks per kv head (the partials + last-arriver combine)."""
    for tag, mode, bits, vq in [MODES[2], MODES[1]]:
        got, want = run_both(bk, gpu_ctx, oracle, tag, mode, bits, vq, [20000], seed=9)
        assert_close(got, want, tag)


def test_decode_batch_of_ragged_sequences(bk, gpu_ctx, oracle):
    lens = [300, 0, 1, 4097, 64, 129, 2050]
    for tag, mode, bits, vq in [MODES[2], MODES[0]]:
        got, want = run_both(bk, gpu_ctx, oracle, tag, mode, bits, vq, lens, seed=4)
        assert np.all(got[1] == 0.0)
        assert_close(got, want, tag)


def test_decode_more_sequences_than_one_launch_carries(bk, gpu_ctx, oracle):
    lens = [5 + (i * 7) % 40 for i in range(70)]
    got, want = run_both(bk, gpu_ctx, oracle, "planar4", MODE_PLANAR, 4, True, lens, seed=8)
    assert_close(got, want)


def test_decode_peaked_softmax(bk, gpu_ctx, oracle):
    """One position dominates (score gap ~ 90): the running-max rescale path."""
    rng = np.random.default_rng(2)
    n = 300
    k, v = synth_kv(rng, n, outliers=False)
    q = rng.standard_normal((NH, HD)).astype(np.float32)
    for tag, mode, bits, vq in MODES[:3]:
        cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_ctx=n)
        ref = oracle.cache(mode, bits, vq)
        kk = k.copy()
        kk[200] *= np.float32(6.0)
        # rope at position 0 for q too, so that q.k[200] really is large for every head group
        for kvh in range(NKV):
            kk[200, kvh] = q[kvh * 6] * np.float32(6.0)
        for p in range(n):
            ref.append(0, kk[p], v[p], 0)
        for p in range(n):
            cache.append(0, kk[p], v[p], pos=0)
        got = cache.attend(0, q, q_pos=[0])[0]
        want = ref.attend(0, q, 0, n)
        assert_close(got, want, tag)
        cache.close()


def test_attn_step_sequence(bk, gpu_ctx, oracle):
    """64 successive decode steps (append + attend) as one sequence, f16 cache."""
    rng = np.random.default_rng(12)
    n0, steps = 500, 64
    k, v = synth_kv(rng, n0 + steps)
    q = rng.standard_normal((steps, NH, HD)).astype(np.float32)
    cache = bk.AttnCache(gpu_ctx, bk.F16, n_layers=1, n_ctx=n0 + steps)
    ref = oracle.cache(MODE_F16)
    cache.append(0, k[:n0], v[:n0])
    for p in range(n0):
        ref.append(0, k[p], v[p], p)
    for t in range(steps):
        got = bk.full_attention_step(cache, 0, q[t], k[n0 + t], v[n0 + t], n0 + t)
        want = ref.step(0, q[t], k[n0 + t], v[n0 + t], n0 + t, threads=8)
        assert_close(got, want, f"step {t}")
    compare_dumps(cache.dump_kv(0), ref.dump(0))
    cache.close()


def test_check_attn_recipe(bk, gpu_ctx, oracle):
    """src/bin/bonsai-vk.rs:315-372 through the one-shot entry point: 24/4/256, n_pos 37, 1e-4."""
    q = oracle.rand_floats(0x1010, NH * HD)
    kc = oracle.rand_floats(0x2020, 37 * NKV * HD)
    vc = oracle.rand_floats(0x3030, 37 * NKV * HD)
    got = bk.attn_step(gpu_ctx, q, kc, vc, 37, NH, NKV, HD)
    k3, v3, q2 = kc.reshape(37, NKV, HD).astype(np.float64), vc.reshape(37, NKV, HD).astype(np.float64), q.reshape(NH, HD)
    for h in range(NH):
        s = (k3[:, h // 6, :] @ q2[h].astype(np.float64)) / 16.0
        p = np.exp(s - s.max())
        want = (p / p.sum()) @ v3[:, h // 6, :]
        assert np.max(np.abs(got[h] - want)) < 1e-4
    with pytest.raises(bk.BonsaiKvError):  # size validation like the reference
        bk.attn_step(gpu_ctx, q[:-1], kc, vc, 37, NH, NKV, HD)


def test_partials_merge_equals_whole(bk, gpu_ctx, oracle):
    """Context split: attend over two halves held by two caches, merge with bk_lse_merge."""
    rng = np.random.default_rng(31)
    n = 1500
    cut = 700
    k, v = synth_kv(rng, n)
    q = rng.standard_normal((NH, HD)).astype(np.float32)
    mode = bk.parse_mode("planar4")
    whole = bk.AttnCache(gpu_ctx, mode, n_layers=1, n_ctx=n)
    whole.append(0, k, v)
    want = whole.attend(0, q, q_pos=[n - 1])[0]
    lo = bk.AttnCache(gpu_ctx, mode, n_layers=1, n_ctx=cut, rope_positions=n)
    hi = bk.AttnCache(gpu_ctx, mode, n_layers=1, n_ctx=n - cut, rope_positions=n)
    lo.append(0, k[:cut], v[:cut], pos=0)
    hi.append(0, k[cut:], v[cut:], pos=cut)
    parts = np.stack([lo.attend(0, q, q_pos=[n - 1], partial=True)[0], hi.attend(0, q, q_pos=[n - 1], partial=True)[0]])
    dparts = gpu_ctx.to_device(parts)
    dout = gpu_ctx.alloc(NH * HD * 4)
    gpu_ctx.check(gpu_ctx.lib.bk_lse_merge(gpu_ctx.h, 2, NH, HD, dparts.ptr, dout.ptr))
    got = dout.download((NH, HD), np.float32)
    assert np.max(np.abs(got - want)) < 5e-5   # two tensor-core results over different splits
    ref = oracle.cache(MODE_PLANAR, 4, True)
    for p in range(n):
        ref.append(0, k[p], v[p], p)
    assert_close(got, ref.attend(0, q, n - 1, n, threads=8))
    for c in (whole, lo, hi):
        c.close()


@pytest.mark.parametrize("env", [{"BONSAI_KV_GENERIC": "1"}, {}])
def test_planar4_kernel_variants(bk, oracle, monkeypatch, env):
    """The 4-bit cache has two decode kernels behind the same entry point: the tensor-core
    path (default for 128 positions and more; launches with a sequence below 2048 rows in its precise
    form) and the generic f32 path (BONSAI_KV_GENERIC=1, read when the context is created).  All must
    meet the bar, on lengths that hit ragged tiles, single chunks and many chunks."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    ctx = bk.Context(0)
    for lens in ([1], [17], [127, 128, 129], [2047], [2048], [2049], [2063, 2064, 2065], [5000], [40000, 3, 2500]):
        got, want = run_both(bk, ctx, oracle, "planar4", MODE_PLANAR, 4, True, lens, seed=sum(lens))
        assert_close(got, want, f"{env} {lens}")
    ctx.close()


def test_planar4_tensor_core_path_other_group_sizes(bk, gpu_ctx, oracle):
    """GQA groups of 1, 2 and 4 q heads per kv head through the tensor-core path, 8 through the
    generic one."""
    rng = np.random.default_rng(77)
    n = 2500
    for n_head, n_kv in ((4, 4), (8, 4), (8, 2), (16, 2)):
        k = rng.standard_normal((n, n_kv, HD)).astype(np.float32)
        v = rng.standard_normal((n, n_kv, HD)).astype(np.float32)
        q = rng.standard_normal((n_head, HD)).astype(np.float32)
        cache = bk.AttnCache(gpu_ctx, bk.parse_mode("planar4"), n_layers=1, n_ctx=n, n_head=n_head, n_kv=n_kv)
        cache.append(0, k, v)
        ref = oracle.cache(MODE_PLANAR, 4, True, n_head=n_head, n_kv=n_kv)
        for p in range(n):
            ref.append(0, k[p], v[p], p)
        want = ref.attend(0, q, n - 1, n, threads=8)
        got = cache.attend(0, q)[0]
        assert_close(got, want, f"{n_head}/{n_kv}")
        cache.close()


def test_fused_step_on_long_planar4_cache(bk, gpu_ctx, oracle):
    """On a long 4-bit cache the attention step is one launch (append fused into the decode):
    the rows it stores and its outputs must match the oracle step by step."""
    rng = np.random.default_rng(41)
    n0, steps = 2600, 12
    k, v = synth_kv(rng, n0 + steps)
    q = rng.standard_normal((steps, NH, HD)).astype(np.float32)
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode("planar4"), n_layers=1, n_ctx=n0 + steps)
    ref = oracle.cache(MODE_PLANAR, 4, True)
    cache.append(0, k[:n0], v[:n0])
    for p in range(n0):
        ref.append(0, k[p], v[p], p)
    for t in range(steps):
        launches = gpu_ctx.launch_count
        got = bk.full_attention_step(cache, 0, q[t], k[n0 + t], v[n0 + t], n0 + t)
        assert gpu_ctx.launch_count - launches == 1
        want = ref.step(0, q[t], k[n0 + t], v[n0 + t], n0 + t, threads=8)
        assert_close(got, want, f"step {t}")
    compare_dumps(cache.dump_kv(0, pos0=n0 - 3), {key: val[n0 - 3:] for key, val in ref.dump(0).items()})
    cache.close()


@pytest.mark.parametrize("env", [{"BONSAI_KV_GENERIC": "1"}, {}])
def test_planar3_kernel_variants(bk, oracle, monkeypatch, env):
    """The 3-bit cache goes through the same tensor-core kernel (indices widened to nibbles in
    registers) from 2048 positions on."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    ctx = bk.Context(0)
    for lens in ([17], [143, 144, 145], [1000], [2047], [2048], [2049], [2063, 2064, 2065], [5000], [40000, 3, 2500]):
        got, want = run_both(bk, ctx, oracle, "planar3", MODE_PLANAR, 3, True, lens, seed=sum(lens) + 3)
        assert_close(got, want, f"{env} {lens}")
    ctx.close()


def test_planar3_tensor_core_path_other_group_sizes(bk, gpu_ctx, oracle):
    rng = np.random.default_rng(79)
    n = 2500
    for n_head, n_kv in ((4, 4), (8, 4), (8, 2), (16, 2)):
        k = rng.standard_normal((n, n_kv, HD)).astype(np.float32)
        v = rng.standard_normal((n, n_kv, HD)).astype(np.float32)
        q = rng.standard_normal((n_head, HD)).astype(np.float32)
        cache = bk.AttnCache(gpu_ctx, bk.parse_mode("planar3"), n_layers=1, n_ctx=n, n_head=n_head, n_kv=n_kv)
        cache.append(0, k, v)
        ref = oracle.cache(MODE_PLANAR, 3, True, n_head=n_head, n_kv=n_kv)
        for p in range(n):
            ref.append(0, k[p], v[p], p)
        want = ref.attend(0, q, n - 1, n, threads=8)
        got = cache.attend(0, q)[0]
        assert_close(got, want, f"{n_head}/{n_kv}")
        cache.close()


def test_fused_step_on_long_planar3_cache(bk, gpu_ctx, oracle):
    rng = np.random.default_rng(44)
    n0, steps = 2600, 12
    k, v = synth_kv(rng, n0 + steps)
    q = rng.standard_normal((steps, NH, HD)).astype(np.float32)
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode("planar3"), n_layers=1, n_ctx=n0 + steps)
    ref = oracle.cache(MODE_PLANAR, 3, True)
    cache.append(0, k[:n0], v[:n0])
    for p in range(n0):
        ref.append(0, k[p], v[p], p)
    for t in range(steps):
        launches = gpu_ctx.launch_count
        got = bk.full_attention_step(cache, 0, q[t], k[n0 + t], v[n0 + t], n0 + t)
        assert gpu_ctx.launch_count - launches == 1
        want = ref.step(0, q[t], k[n0 + t], v[n0 + t], n0 + t, threads=8)
        assert_close(got, want, f"step {t}")
    compare_dumps(cache.dump_kv(0, pos0=n0 - 3), {key: val[n0 - 3:] for key, val in ref.dump(0).items()})
    cache.close()


@pytest.mark.parametrize("env", [{"BONSAI_KV_GENERIC": "1"}, {}])
def test_f16_kernel_variants(bk, oracle, monkeypatch, env):
    """The f16 cache has the same two decode kernels behind one entry point (tensor cores from 2048
    positions on).  Lengths hit ragged tiles, single chunks, many chunks and a mixed batch."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    ctx = bk.Context(0)
    for lens in ([17], [127], [128], [129], [143, 144, 145], [1000], [2047], [2048], [2049], [2063, 2064, 2065], [5000], [40000, 3, 2500]):
        got, want = run_both(bk, ctx, oracle, "f16", MODE_F16, 0, False, lens, seed=sum(lens))
        assert_close(got, want, f"{env} {lens}")
    ctx.close()


def test_f16_tensor_core_path_other_group_sizes(bk, gpu_ctx, oracle):
    rng = np.random.default_rng(78)
    n = 2500
    for n_head, n_kv in ((4, 4), (8, 4), (8, 2), (16, 2)):
        k = rng.standard_normal((n, n_kv, HD)).astype(np.float32)
        v = rng.standard_normal((n, n_kv, HD)).astype(np.float32)
        q = rng.standard_normal((n_head, HD)).astype(np.float32)
        cache = bk.AttnCache(gpu_ctx, bk.parse_mode("f16"), n_layers=1, n_ctx=n, n_head=n_head, n_kv=n_kv)
        cache.append(0, k, v)
        ref = oracle.cache(MODE_F16, 0, False, n_head=n_head, n_kv=n_kv)
        for p in range(n):
            ref.append(0, k[p], v[p], p)
        want = ref.attend(0, q, n - 1, n, threads=8)
        got = cache.attend(0, q)[0]
        assert_close(got, want, f"{n_head}/{n_kv}")
        cache.close()


def test_f16_rows_past_the_end_do_not_leak_in(bk, gpu_ctx, oracle):
    """The tensor-core kernel copies whole 16-position tiles; rows past n_pos may hold anything,
    including f16 infinities (1e30 stored as f16), and must not reach the result."""
    rng = np.random.default_rng(5)
    n, extra = 2500 + 7, 9
    k, v = synth_kv(rng, n + extra)
    k[n:] = np.float32(1e30)
    v[n:] = np.float32(-1e30)
    q = rng.standard_normal((NH, HD)).astype(np.float32)
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode("f16"), n_layers=1, n_ctx=n + extra)
    cache.append(0, k, v)
    ref = oracle.cache(MODE_F16, 0, False)
    for p in range(n):
        ref.append(0, k[p], v[p], p)
    want = ref.attend(0, q, n - 1, n, threads=8)
    got = cache.attend(0, q[None], n_pos=[n], q_pos=[n - 1])[0]
    assert np.all(np.isfinite(got))
    assert_close(got, want)
    cache.close()


def test_fused_step_on_long_f16_cache(bk, gpu_ctx, oracle):
    """On a long f16 cache the attention step is one launch too; stored rows stay bit-exact."""
    rng = np.random.default_rng(43)
    n0, steps = 2600, 12
    k, v = synth_kv(rng, n0 + steps)
    q = rng.standard_normal((steps, NH, HD)).astype(np.float32)
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode("f16"), n_layers=1, n_ctx=n0 + steps)
    ref = oracle.cache(MODE_F16, 0, False)
    cache.append(0, k[:n0], v[:n0])
    for p in range(n0):
        ref.append(0, k[p], v[p], p)
    for t in range(steps):
        launches = gpu_ctx.launch_count
        got = bk.full_attention_step(cache, 0, q[t], k[n0 + t], v[n0 + t], n0 + t)
        assert gpu_ctx.launch_count - launches == 1
        want = ref.step(0, q[t], k[n0 + t], v[n0 + t], n0 + t, threads=8)
        assert_close(got, want, f"step {t}")
    compare_dumps(cache.dump_kv(0, pos0=n0 - 3), {key: val[n0 - 3:] for key, val in ref.dump(0).items()})
    cache.close()


ROW_KERNEL_MODES = [("f32", MODE_F32, 0, False), ("planar4k", MODE_PLANAR, 4, False), ("planar3k", MODE_PLANAR, 3, False),
                    ("planar2", MODE_PLANAR, 2, True)]   # (planar2: the 4-bit kernel with 2-bit rows widened to nibbles)


@pytest.mark.parametrize("tag,mode,bits,vq", ROW_KERNEL_MODES)
@pytest.mark.parametrize("env", [{"BONSAI_KV_GENERIC": "1"}, {}])
def test_f32_and_k_only_kernel_variants(bk, oracle, monkeypatch, env, tag, mode, bits, vq):
    """f32 caches and K-only 4/3-bit caches have the same two decode kernels behind one entry point (the
    tensor-core row kernel from 2048 positions on).  Lengths hit ragged tiles, single chunks, many chunks
    and a mixed batch."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    ctx = bk.Context(0)
    for lens in ([127], [128], [129], [143, 144, 145], [1000], [2047], [2048], [2049], [2063, 2064, 2065], [5000], [21000, 3, 2500]):
        got, want = run_both(bk, ctx, oracle, tag, mode, bits, vq, lens, seed=sum(lens) + bits)
        assert_close(got, want, f"{tag} {env} {lens}")
    ctx.close()


@pytest.mark.parametrize("tag,mode,bits,vq", ROW_KERNEL_MODES)
def test_f32_and_k_only_tensor_core_path_other_group_sizes(bk, gpu_ctx, oracle, tag, mode, bits, vq):
    rng = np.random.default_rng(79 + bits)
    n = 2500
    for n_head, n_kv in ((4, 4), (8, 4), (8, 2), (16, 2)):
        k = rng.standard_normal((n, n_kv, HD)).astype(np.float32)
        v = rng.standard_normal((n, n_kv, HD)).astype(np.float32)
        q = rng.standard_normal((n_head, HD)).astype(np.float32)
        cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_ctx=n, n_head=n_head, n_kv=n_kv)
        cache.append(0, k, v)
        ref = oracle.cache(mode, bits, vq, n_head=n_head, n_kv=n_kv)
        for p in range(n):
            ref.append(0, k[p], v[p], p)
        want = ref.attend(0, q, n - 1, n, threads=8)
        got = cache.attend(0, q)[0]
        assert_close(got, want, f"{tag} {n_head}/{n_kv}")
        cache.close()


@pytest.mark.parametrize("tag,mode,bits,vq", ROW_KERNEL_MODES)
def test_f32_rows_past_the_end_do_not_leak_in(bk, gpu_ctx, oracle, tag, mode, bits, vq):
    """The row kernel copies whole 16-position tiles; rows past n_pos may hold anything, including
    infinities and NaNs in f32 rows, and must not reach the result."""
    rng = np.random.default_rng(6 + bits)
    n, extra = 2500 + 7, 9
    k, v = synth_kv(rng, n + extra)
    k[n:] = np.float32(np.inf)
    v[n:] = np.float32(np.nan)
    q = rng.standard_normal((NH, HD)).astype(np.float32)
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_ctx=n + extra)
    cache.append(0, k, v)
    ref = oracle.cache(mode, bits, vq)
    for p in range(n):
        ref.append(0, k[p], v[p], p)
    want = ref.attend(0, q, n - 1, n, threads=8)
    got = cache.attend(0, q[None], n_pos=[n], q_pos=[n - 1])[0]
    assert np.all(np.isfinite(got))
    assert_close(got, want)
    cache.close()


@pytest.mark.parametrize("n0", [2600, 131])
@pytest.mark.parametrize("tag,mode,bits,vq", ROW_KERNEL_MODES)
def test_fused_step_on_long_f32_and_k_only_caches(bk, gpu_ctx, oracle, tag, mode, bits, vq, n0):
    """On f32, K-only and 2-bit caches (from 128 rows on) the attention step is one launch too; stored rows stay
    bit-exact."""
    rng = np.random.default_rng(44 + bits)
    steps = 12
    k, v = synth_kv(rng, n0 + steps)
    q = rng.standard_normal((steps, NH, HD)).astype(np.float32)
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_ctx=n0 + steps)
    ref = oracle.cache(mode, bits, vq)
    cache.append(0, k[:n0], v[:n0])
    for p in range(n0):
        ref.append(0, k[p], v[p], p)
    for t in range(steps):
        launches = gpu_ctx.launch_count
        got = bk.full_attention_step(cache, 0, q[t], k[n0 + t], v[n0 + t], n0 + t)
        assert gpu_ctx.launch_count - launches == 1
        want = ref.step(0, q[t], k[n0 + t], v[n0 + t], n0 + t, threads=8)
        assert_close(got, want, f"{tag} step {t}")
    compare_dumps(cache.dump_kv(0, pos0=n0 - 3), {key: val[n0 - 3:] for key, val in ref.dump(0).items()})
    cache.close()


@pytest.mark.parametrize("tag,bits", [("planar4", 4), ("planar3", 3), ("planar2", 2)])
def test_short_context_planar_tensor_core_path_is_precise(bk, gpu_ctx, oracle, tag, bits):
    """Below 2048 rows nothing averages the f16 table's rounding out, so the 4-, 3- and 2-bit kernel carries the
    remainders there: with x20 outlier channels and a peaked softmax the result stays within 1e-4 of the f32 CPU
    path (absolute and relative) at every length, ragged tiles included."""
    worst = 0.0
    for seed, n in enumerate((128, 129, 200, 517, 1000, 1531, 2047)):
        rng = np.random.default_rng(300 + 17 * seed + bits)
        k, v = synth_kv(rng, n)
        q = (rng.standard_normal((NH, HD)) * 3).astype(np.float32)
        cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_ctx=n)
        cache.append(0, k, v)
        ref = oracle.cache(MODE_PLANAR, bits, True)
        for p in range(n):
            ref.append(0, k[p], v[p], p)
        want = ref.attend(0, q, n - 1, n, threads=8)
        launches = gpu_ctx.launch_count
        got = cache.attend(0, q)[0]
        assert gpu_ctx.launch_count - launches == 1
        err = float(np.max(np.abs(got - want)))
        worst = max(worst, err, err / float(np.max(np.abs(want))))
        cache.close()
    assert worst <= 1e-4, worst


def test_f32_tensor_core_path_precision(bk, gpu_ctx, oracle):
    """The f32 row kernel splits every stored float into f16 hi + lo: with x20 outlier channels and a peaked
    softmax its result still agrees with the f32 CPU path to 2e-5 (the bar of the path is 1e-3)."""
    rng = np.random.default_rng(91)
    n = 3000
    k, v = synth_kv(rng, n)
    q = (rng.standard_normal((NH, HD)) * 3).astype(np.float32)
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode("f32"), n_layers=1, n_ctx=n)
    cache.append(0, k, v)
    ref = oracle.cache(MODE_F32, 0, False)
    for p in range(n):
        ref.append(0, k[p], v[p], p)
    want = ref.attend(0, q, n - 1, n, threads=8)
    got = cache.attend(0, q)[0]
    err = float(np.max(np.abs(got - want))) / float(np.max(np.abs(want)))
    assert err <= 2e-5, err
    cache.close()


@pytest.mark.parametrize("bits", range(1, 9))
def test_nearest_centroid_search_equals_the_reference_scan(bk, gpu_ctx, oracle, bits):
    """The kernels find the nearest centroid by binary search plus one neighbour check; the
    reference scans all levels.  Both must pick the same index everywhere, in particular at the
    centroids themselves, at the midpoints between neighbours and one ulp to either side.
    Vectors are built so that their rotated unit coordinates land on those values."""
    pq, opq = bk.PlanarQuant(HD, bits, gpu_ctx), oracle.pq(HD, bits)
    cb = oracle.codebook(HD, bits).astype(np.float32)
    mids = ((cb[:-1].astype(np.float64) + cb[1:]) / 2).astype(np.float32)
    pts = np.concatenate([cb, mids, np.nextafter(mids, np.float32(1)), np.nextafter(mids, np.float32(-1)),
                          np.nextafter(cb, np.float32(1)), np.nextafter(cb, np.float32(-1)),
                          np.array([0.0, -0.0, 0.3, -0.3, 0.9, -0.9], np.float32)])
    rng = np.random.default_rng(bits)
    rows = []
    for _ in range(24):
        target = rng.choice(pts, HD).astype(np.float32)              # wanted rotated unit coordinates
        x = opq.rotate_inv(target)[:HD]                               # vector whose rotation is about that
        rows.append(x / max(np.linalg.norm(x), 1e-30))                # unit norm: quantize() scales by ~1
    x = np.stack(rows).astype(np.float32)
    packed, norms = pq.quantize(x)
    for r in range(x.shape[0]):
        p_ref, n_ref = opq.quantize(x[r])
        assert np.array_equal(packed[r], p_ref), (bits, r)
        assert bits_of(norms[r]) == bits_of(n_ref)


# ---------------------------------------------------------------------------
# the layer form of the step: q|gate split, per-head RMSNorm, sigmoid gate
# ---------------------------------------------------------------------------

def test_rms_norm_rows_bits(bk, gpu_ctx, oracle, layer_golden):
    """bk_rms_norm_rows against the golden vectors and the oracle, bit for bit; the reference's
    two error cases (src/kernels.rs:810-811)."""
    g = layer_golden
    y = bk.rms_norm_rows(g["rms_small_x"], g["rms_small_w"], 4, 1e-6, ctx=gpu_ctx)
    assert np.array_equal(bits_of(y), g["rms_small_out"])
    y = bk.rms_norm_rows(g["rms_rows_x"].view(np.float32), g["rms_rows_w"].view(np.float32), HD, 1e-6, ctx=gpu_ctx)
    assert np.array_equal(bits_of(y), g["rms_rows_out"])
    rng = np.random.default_rng(3)
    for row_len, n_rows in ((256, 28), (128, 48), (1, 5), (1024, 3), (77, 9)):
        x = (rng.standard_normal(n_rows * row_len) * 3).astype(np.float32)
        w = rng.standard_normal(row_len).astype(np.float32)
        got = bk.rms_norm_rows(x, w, row_len, 1e-6, ctx=gpu_ctx)
        assert np.array_equal(bits_of(got), bits_of(oracle.rms_norm_rows(x, w, row_len, 1e-6))), row_len
    with pytest.raises(bk.BonsaiKvError):
        bk.rms_norm_rows(g["rms_small_x"], g["rms_small_w"], 3, 1e-6, ctx=gpu_ctx)
    with pytest.raises(bk.BonsaiKvError):
        bk.rms_norm_rows(g["rms_small_x"], g["rms_small_w"][:2], 4, 1e-6, ctx=gpu_ctx)


@pytest.mark.parametrize("tag", ["planar4", "f16"])
def test_layer_step_golden(bk, gpu_ctx, layer_golden, tag):
    """Three layer steps from an empty cache against the committed vectors."""
    g = {k[len(f"layer_{tag}_"):]: v for k, v in layer_golden.items() if k.startswith(f"layer_{tag}_")}
    f = lambda a: a.view(np.float32)
    n = g["out"].shape[0]
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_ctx=16)
    for pos in range(n):
        out = bk.full_attention_layer_core(cache, 0, f(g["qfull"])[pos], f(g["kraw"])[pos], f(g["vraw"])[pos],
                                           f(g["qw"]), f(g["kw"]), 1e-6, pos)
        assert_close(out.ravel(), f(g["out"])[pos], f"{tag} step {pos}")
    d = cache.dump_kv(0)
    if tag == "planar4":
        assert np.array_equal(d["kq"].reshape(n * 4, -1), g["k"]) and np.array_equal(d["vq"].reshape(n * 4, -1), g["v"])
        assert np.array_equal(bits_of(d["kn"].ravel()), g["kn"]) and np.array_equal(bits_of(d["vn"].ravel()), g["vn"])
    else:
        assert np.array_equal(d["k16"].reshape(n * 4, -1), g["k"]) and np.array_equal(d["v16"].reshape(n * 4, -1), g["v"])
    cache.close()


@pytest.mark.parametrize("tag,mode,bits,vq,n0", [("planar4", MODE_PLANAR, 4, True, 2600), ("f16", MODE_F16, 0, False, 2600),
                                                 ("planar4", MODE_PLANAR, 4, True, 300), ("f32", MODE_F32, 0, False, 500),
                                                 ("planar3", MODE_PLANAR, 3, True, 2600), ("planar4k", MODE_PLANAR, 4, False, 700),
                                                 ("planar4k", MODE_PLANAR, 4, False, 2600), ("f32", MODE_F32, 0, False, 2600),
                                                 ("planar4k", MODE_PLANAR, 4, False, 2331), ("planar3k", MODE_PLANAR, 3, False, 2600),
                                                 ("planar2", MODE_PLANAR, 2, True, 2600)])
def test_layer_step_on_a_filled_cache(bk, gpu_ctx, oracle, tag, mode, bits, vq, n0):
    """Layer steps after a prefill, on caches that take the tensor-core path (one launch per
    step) and on ones that do not: gated outputs within the bar, stored rows bit-exact."""
    rng = np.random.default_rng(n0 + bits)
    steps = 6
    k, v = synth_kv(rng, n0)
    qfull = (rng.standard_normal((steps, NH, 2 * HD)) * 2).astype(np.float32)
    kraw = (rng.standard_normal((steps, NKV, HD)) * 3).astype(np.float32)
    vraw = rng.standard_normal((steps, NKV, HD)).astype(np.float32)
    qw = (1 + 0.3 * rng.standard_normal(HD)).astype(np.float32)
    kw = (1 + 0.3 * rng.standard_normal(HD)).astype(np.float32)
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_ctx=n0 + steps)
    ref = oracle.cache(mode, bits, vq)
    cache.append(0, k, v)
    for p in range(n0):
        ref.append(0, k[p], v[p], p)
    # from 128 rows on these caches take a tensor-core kernel with the append fused in
    one_launch = n0 >= 128 and tag in ("planar4", "planar3", "planar2", "f16", "f32", "planar4k", "planar3k")
    for t in range(steps):
        launches = gpu_ctx.launch_count
        got = bk.full_attention_layer_core(cache, 0, qfull[t], kraw[t], vraw[t], qw, kw, 1e-6, n0 + t)
        assert (gpu_ctx.launch_count - launches == 1) == one_launch
        want = ref.layer_step(0, qfull[t], kraw[t], vraw[t], qw, kw, 1e-6, n0 + t, threads=8)
        assert_close(got, want, f"{tag} step {t}")
    compare_dumps(cache.dump_kv(0, pos0=n0 - 2), {key: val[n0 - 2:] for key, val in ref.dump(0).items()})
    with pytest.raises(bk.BonsaiKvError):  # not the next row
        bk.full_attention_layer_core(cache, 0, qfull[0], kraw[0], vraw[0], qw, kw, 1e-6, n0)
    cache.close()


# ---------------------------------------------------------------------------
# prompt-cache snapshots
# ---------------------------------------------------------------------------

def expected_snapshot(ref_dumps, mode_kind, bits, vq, n_kv, layout):
    """The snapshot bytes built in numpy from the oracle's stores: header, n_pos per layer, then
    per layer K and V in the reference's CPU layout (src/forward.rs:40-46) or, for quantized
    sides, its device rows (shaders/kv_store_q.comp:119-123: packed words then the norm word)."""
    n_layers = len(ref_dumps)
    hdr = np.array([0x53564B42, 1, layout, mode_kind, bits, int(vq), n_layers, n_kv, HD, 0, 0, 0], np.uint32)
    out = [hdr.tobytes(), np.array([d["n"] for d in ref_dumps], np.uint32).tobytes()]
    for d in ref_dumps:
        if d["n"] == 0:
            continue
        for rows, norms in ((d["k_rows"], d["k_norms"]), (d["v_rows"], d["v_norms"])):
            flat = np.ascontiguousarray(rows).reshape(d["n"] * n_kv, -1)
            if norms is None:
                out.append(flat.tobytes())
            elif layout == 0:
                out += [flat.tobytes(), np.ascontiguousarray(norms, np.float32).tobytes()]
            else:
                nb = np.ascontiguousarray(norms, np.float32).reshape(-1, 1).view(np.uint8)
                out.append(np.concatenate([flat.view(np.uint8), nb], axis=1).tobytes())
    return b"".join(out)


@pytest.mark.parametrize("tag,mode,bits,vq", [MODES[0], MODES[1], MODES[2], MODES[3], MODES[4]])
def test_snapshot_bytes_and_restore(bk, gpu_ctx, oracle, tag, mode, bits, vq):
    rng = np.random.default_rng(bits + 60)
    lens = [37, 0, 5]  # per layer
    kind = {MODE_F32: 0, MODE_F16: 1, MODE_PLANAR: 2}[mode]
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=3, n_ctx=64)
    ref = oracle.cache(mode, bits, vq, n_layer=3)
    for il, n in enumerate(lens):
        if n:
            k, v = synth_kv(rng, n)
            cache.append(il, k, v)
            for p in range(n):
                ref.append(il, k[p], v[p], p)
    dumps = []
    for il, n in enumerate(lens):
        d = ref.dump(il)
        if mode == MODE_PLANAR:
            e = dict(n=n, k_rows=d["kq"], k_norms=d["kn"], v_rows=d["vq"] if vq else d["v"], v_norms=d["vn"] if vq else None)
        elif mode == MODE_F16:
            e = dict(n=n, k_rows=d["k16"], k_norms=None, v_rows=d["v16"], v_norms=None)
        else:
            e = dict(n=n, k_rows=d["k"], k_norms=None, v_rows=d["v"], v_norms=None)
        dumps.append(e)
    blobs = {}
    for layout in (0, 1):
        blobs[layout] = cache.snapshot(layout=layout)
        assert blobs[layout] == expected_snapshot(dumps, kind, bits if mode == MODE_PLANAR else 0,
                                                  vq if mode == MODE_PLANAR else False, NKV, layout), (tag, layout)
    # restore into a cache with another context size and several sequences; attend on both
    q = rng.standard_normal((NH, HD)).astype(np.float32)
    want = cache.attend(0, q)[0]
    for layout in (0, 1):
        other = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=3, n_seqs=2, n_ctx=40)
        other.restore(blobs[layout], seq=1)
        assert [other.n_pos(il, 1) for il in range(3)] == lens and other.n_pos(0, 0) == 0
        got = other.attend(0, q[None], seq_ids=[1])[0]
        assert np.array_equal(bits_of(got), bits_of(want))
        compare_dumps(other.dump_kv(0, seq=1), cache.dump_kv(0))
        other.close()
    # refusals: other mode, too small a context, truncated or foreign bytes
    wrong = bk.AttnCache(gpu_ctx, bk.parse_mode("planar5" if tag != "planar5" else "f32"), n_layers=3, n_ctx=64)
    with pytest.raises(bk.BonsaiKvError):
        wrong.restore(blobs[0])
    wrong.close()
    small = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=3, n_ctx=16)
    with pytest.raises(bk.BonsaiKvError):
        small.restore(blobs[0])
    with pytest.raises(bk.BonsaiKvError):
        small.restore(blobs[0][:100])
    with pytest.raises(bk.BonsaiKvError):
        small.restore(b"\0" * 256)
    small.close()
    cache.close()


# ---------------------------------------------------------------------------
# batched (prefill) attention
# ---------------------------------------------------------------------------

def prefill_both(bk, gpu_ctx, oracle, tag, mode, bits, vq, n0, n_tok, seed, n_head=NH, n_kv=NKV, outliers=True):
    """n0 cached tokens, then a block of n_tok prompt tokens: the batched call against the oracle
    attending token by token (src/forward.rs:247-375 with q_pos = pos, n_pos = pos + 1)."""
    rng = np.random.default_rng(seed)
    n = n0 + n_tok
    k = rng.standard_normal((n, n_kv, HD)).astype(np.float32)
    v = rng.standard_normal((n, n_kv, HD)).astype(np.float32)
    if outliers:
        ch = rng.choice(HD, size=3, replace=False)
        k[:, :, ch] *= np.float32(20.0)
        v[:, :, ch] *= np.float32(20.0)
    q = rng.standard_normal((n_tok, n_head, HD)).astype(np.float32)
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_ctx=n, n_head=n_head, n_kv=n_kv)
    cache.append(0, k, v)
    ref = oracle.cache(mode, bits, vq, n_head=n_head, n_kv=n_kv)
    for p in range(n):
        ref.append(0, k[p], v[p], p)
    got = cache.prefill_attend(0, q, n0)
    want = np.stack([ref.attend(0, q[i], n0 + i, n0 + i + 1, threads=8) for i in range(n_tok)])
    cache.close()
    return got, want


@pytest.mark.parametrize("tag,mode,bits,vq", [MODES[2], MODES[3], MODES[1], MODES[8], MODES[0], ("planar2", MODE_PLANAR, 2, True),
                                              MODES[4], ("planar3k", MODE_PLANAR, 3, False)])
@pytest.mark.parametrize("n0,n_tok", [(0, 45), (300, 50), (3000, 100), (37, 3), (0, 1)])
def test_prefill_attention_equals_token_by_token(bk, gpu_ctx, oracle, tag, mode, bits, vq, n0, n_tok):
    """planar4 / planar3 / f16 take the batched tensor-core kernel (from 4 tokens on), the other
    modes the decode kernels with one entry per token; every token must meet the decode bar."""
    got, want = prefill_both(bk, gpu_ctx, oracle, tag, mode, bits, vq, n0, n_tok, seed=n0 + n_tok + bits)
    for i in range(n_tok):
        assert_close(got[i], want[i], f"{tag} n0={n0} token {i}")


@pytest.mark.parametrize("tag,mode,bits,vq", [MODES[2], MODES[3], MODES[1]])
def test_prefill_mma_sync_variant_and_empty_chunks(bk, oracle, monkeypatch, tag, mode, bits, vq):
    """The batched kernel exists twice: on tcgen05 with tensor-memory accumulators (default) and
    on mma.sync (BONSAI_KV_PREFILL=mma, read when the context is created).  A 700-token prompt
    from the empty cache gives two context chunks, of which the second is empty for the early
    query blocks; both kernels must handle it."""
    for env in ("mma", None):
        if env:
            monkeypatch.setenv("BONSAI_KV_PREFILL", env)
        else:
            monkeypatch.delenv("BONSAI_KV_PREFILL", raising=False)
        ctx = bk.Context(0)
        for n0, n_tok in ((0, 700), (300, 50), (3000, 100)):
            got, want = prefill_both(bk, ctx, oracle, tag, mode, bits, vq, n0, n_tok, seed=n0 + 7)
            for i in range(n_tok):
                assert_close(got[i], want[i], f"{env} {tag} n0={n0} token {i}")
        ctx.close()


def test_prefill_other_group_sizes_and_long_context(bk, gpu_ctx, oracle):
    for n_head, n_kv in ((4, 4), (8, 4), (8, 2)):
        got, want = prefill_both(bk, gpu_ctx, oracle, "planar4", MODE_PLANAR, 4, True, 500, 70, seed=n_head, n_head=n_head, n_kv=n_kv)
        assert_close(got, want, f"{n_head}/{n_kv}")
    got, want = prefill_both(bk, gpu_ctx, oracle, "planar4", MODE_PLANAR, 4, True, 20000, 30, seed=5)
    assert_close(got, want, "long")


def test_prefill_step_appends_then_attends(bk, gpu_ctx, oracle):
    """bk_prefill_step from the empty cache in blocks: rows bit-exact, outputs within the bar,
    and refusals for tokens that are not in the cache."""
    rng = np.random.default_rng(12)
    n, blk = 130, 50
    k, v = synth_kv(rng, n)
    q = rng.standard_normal((n, NH, HD)).astype(np.float32)
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode("planar4"), n_layers=1, n_ctx=n)
    ref = oracle.cache(MODE_PLANAR, 4, True)
    dq, dk, dv = gpu_ctx.to_device(q), gpu_ctx.to_device(k), gpu_ctx.to_device(v)
    do = gpu_ctx.alloc(n * NH * HD * 4)
    with pytest.raises(bk.BonsaiKvError):
        cache.prefill_attend(0, q[:5], 0)  # nothing appended yet
    for p0 in range(0, n, blk):
        m = min(blk, n - p0)
        cache.prefill_step_device(0, dq.offset(p0 * NH * HD * 4), dk.offset(p0 * NKV * HD * 4), dv.offset(p0 * NKV * HD * 4),
                                  do.offset(p0 * NH * HD * 4), p0, m)
    got = do.download((n, NH, HD), np.float32)
    for p in range(n):
        want = ref.step(0, q[p], k[p], v[p], p, threads=8)
        assert_close(got[p], want, f"token {p}")
    compare_dumps(cache.dump_kv(0), ref.dump(0))
    with pytest.raises(bk.BonsaiKvError):
        cache.prefill_step_device(0, dq.ptr, dk.ptr, dv.ptr, do.ptr, 5, 3)  # not the next row
    for b in (dq, dk, dv, do):
        b.free()
    cache.close()


def test_batched_step_one_launch_and_mixed_lengths(bk, gpu_ctx, oracle):
    """bk_attn_step_batch: a batch of long planar4 sequences is one launch per step (the decode
    kernel stores the new rows); a batch with a short sequence goes through append + decode.
    Rows bit-exact and outputs within the bar either way."""
    rng = np.random.default_rng(21)
    for lens, one_launch in (([4100, 6000, 9000], True), ([4100, 40, 6000], False)):
        n_seqs, steps = len(lens), 3
        cache = bk.AttnCache(gpu_ctx, bk.parse_mode("planar4"), n_layers=1, n_seqs=n_seqs, n_ctx=max(lens) + steps)
        refs = []
        for s, n in enumerate(lens):
            k, v = synth_kv(rng, n)
            cache.append(0, k, v, seq=s)
            ref = oracle.cache(MODE_PLANAR, 4, True)
            for p in range(n):
                ref.append(0, k[p], v[p], p)
            refs.append(ref)
        for t in range(steps):
            q = rng.standard_normal((n_seqs, NH, HD)).astype(np.float32)
            k = rng.standard_normal((n_seqs, NKV, HD)).astype(np.float32)
            v = rng.standard_normal((n_seqs, NKV, HD)).astype(np.float32)
            dq, dk, dv = gpu_ctx.to_device(q), gpu_ctx.to_device(k), gpu_ctx.to_device(v)
            do = gpu_ctx.alloc(n_seqs * NH * HD * 4)
            launches = gpu_ctx.launch_count
            cache.step_batch_device(0, dq.ptr, dk.ptr, dv.ptr, do.ptr, n_seqs)
            assert (gpu_ctx.launch_count - launches == 1) == one_launch
            got = do.download((n_seqs, NH, HD), np.float32)
            for s in range(n_seqs):
                want = refs[s].step(0, q[s], k[s], v[s], lens[s] + t, threads=8)
                assert_close(got[s], want, f"{lens} seq {s} step {t}")
            for b in (dq, dk, dv, do):
                b.free()
        for s in range(n_seqs):
            compare_dumps(cache.dump_kv(0, seq=s, pos0=lens[s] - 1), {key: val[lens[s] - 1:] for key, val in refs[s].dump(0).items()})
        cache.close()
