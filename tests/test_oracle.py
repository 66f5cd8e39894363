"""CPU tests of the oracle (oracle/bonsai_oracle.c).

Two groups: (1) the reference's own unit tests for this path, re-run against
the oracle (each test names the reference test it mirrors); (2) bit-for-bit
agreement with tests/golden/kvpath_golden.npz, which was produced by an
independent Python restatement (tests/golden/gen_golden.py).
"""
import numpy as np
import pytest

from oracle_lib import MODE_F16, MODE_F32, MODE_PLANAR

HD = 256


def bits_of(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def rng_list(oracle, seed, n):
    return oracle.rand_floats(seed, n)


# ---------------------------------------------------------------------------
# (1) the reference's unit tests
# ---------------------------------------------------------------------------

def test_centroids_are_sorted_symmetric_and_sized(oracle):
    """src/kvquant.rs:592-612"""
    for bits in (3, 4):
        c = oracle.codebook(HD, bits)
        assert len(c) == 1 << bits
        assert np.all(np.diff(c) > 0)
        n = len(c)
        for i in range(n // 2):
            assert abs(c[i] + c[n - 1 - i]) < 1e-6
        assert c[-1] < 4.0 / 16.0


def test_lloyd_max_beats_uniform(oracle):
    """src/kvquant.rs:615-628"""
    sigma2 = np.float32(1.0) / np.float32(HD)
    d3 = oracle.lib.or_expected_distortion(HD, 3)
    d4 = oracle.lib.or_expected_distortion(HD, 4)
    assert d3 < sigma2 and d4 < d3


def test_givens_is_orthogonal(oracle):
    """src/kvquant.rs:631-642"""
    p = oracle.pq(HD, 4)
    x = rng_list(oracle, 7, HD)
    back = p.rotate_inv(p.rotate(x))
    assert np.max(np.abs(back[:HD] - x)) < 1e-5


def test_quantize_roundtrip_error_is_small(oracle):
    """src/kvquant.rs:645-667: 64 vectors from one generator stream, worst rel-L2 < 0.12"""
    p = oracle.pq(HD, 4)
    stream = rng_list(oracle, 11, 64 * HD).reshape(64, HD)
    worst = 0.0
    for x in stream:
        packed, norm = p.quantize(x)
        y = p.dequantize(packed, norm)
        err = np.sqrt(np.sum((x - y) ** 2, dtype=np.float32))
        xn = np.sqrt(np.sum(x * x, dtype=np.float32))
        worst = max(worst, err / max(xn, 1e-9))
    assert worst < 0.12


def test_kv_mode_parsing(oracle):
    """src/kvquant.rs:670-720"""
    P = oracle.parse_mode
    assert P("") == (MODE_F32, 0, False)
    assert P("f32") == (MODE_F32, 0, False)
    for s in ("f16", "fp16", "half"):
        assert P(s) == (MODE_F16, 0, False)
    assert P("planar4") == (MODE_PLANAR, 4, True)
    assert P("planar4k") == (MODE_PLANAR, 4, False)
    assert P("iso3") == (MODE_PLANAR, 3, True)
    assert P("iso8k") == (MODE_PLANAR, 8, False)
    for s in ("planar9", "planar0", "garbage", "planark", "planar", "iso", "planar4kk", "planar-1", "k"):
        assert P(s) == (MODE_F32, 0, False), s
    assert P("planar+4") == (MODE_PLANAR, 4, True)  # Rust's u32 parser accepts a leading '+'
    assert P("planar04") == (MODE_PLANAR, 4, True)


def test_dot_rotated_matches_dequantized_dot(oracle):
    """src/kvquant.rs:723-738"""
    p = oracle.pq(HD, 4)
    stream = rng_list(oracle, 23, 2 * HD)
    k, q = stream[:HD], stream[HD:]
    packed, norm = p.quantize(k)
    khat = p.dequantize(packed, norm)
    a = p.dot_rotated(p.rotate(q), packed, norm)
    b = np.float32(0)
    for x, y in zip(q, khat):
        b = np.float32(b + np.float32(x * y))
    assert abs(a - b) < 1e-4


@pytest.mark.parametrize("bits", [3, 4])
def test_bit_packing_roundtrips_both_widths(oracle, bits):
    """src/kvquant.rs:763-776"""
    n = 256
    r = rng_list(oracle, 5 + bits, n)
    idx = ((np.abs(r) * np.float32(1000.0)).astype(np.uint32) % (1 << bits)).astype(np.uint8)
    packed = np.zeros(oracle.lib.or_packed_bytes(n, bits), np.uint8)
    oracle.lib.or_pack_bits(idx, n, bits, packed)
    back = np.zeros(n, np.uint8)
    oracle.lib.or_unpack_bits(packed, bits, n, back)
    assert np.array_equal(idx, back)


@pytest.mark.parametrize("bits", range(1, 9))
def test_row_packing_roundtrips_every_width_and_fits_row(oracle, bits):
    """src/kvquant.rs:779-794, plus: for n = 256 pack_idx equals the LE bitstream"""
    n = 256
    r = rng_list(oracle, 17 + bits, n)
    idx = ((np.abs(r) * np.float32(1000.0)).astype(np.uint32) % (1 << bits)).astype(np.uint8)
    nbytes = oracle.lib.or_packed_bytes(n, bits)
    assert nbytes == 32 * bits
    packed = np.zeros(nbytes, np.uint8)
    oracle.lib.or_pack_idx(idx, n, bits, packed)
    back = np.zeros(n, np.uint8)
    oracle.lib.or_unpack_idx(packed, n, bits, back)
    assert np.array_equal(idx, back)
    stream = np.zeros(nbytes, np.uint8)
    oracle.lib.or_pack_bits(idx, n, bits, stream)
    assert np.array_equal(packed, stream)


def test_groups3_matches_reference_3bit_layout(oracle):
    """src/kvquant.rs:797-813"""
    n = 256
    r = rng_list(oracle, 23, n)
    idx = ((np.abs(r) * np.float32(800.0)).astype(np.uint32) % 8).astype(np.uint8)
    packed = np.zeros(oracle.lib.or_packed_bytes(n, 3), np.uint8)
    oracle.lib.or_pack_idx(idx, n, 3, packed)
    for g in range(n // 8):
        v = int(packed[3 * g]) | int(packed[3 * g + 1]) << 8 | int(packed[3 * g + 2]) << 16
        for k in range(8):
            assert (v >> (3 * k)) & 7 == idx[g * 8 + k]


def test_half_conversions(oracle):
    """src/gguf.rs:951-965"""
    h2f = oracle.lib.or_half_to_f32
    assert h2f(0x3C00) == 1.0 and h2f(0xC000) == -2.0 and h2f(0x0000) == 0.0 and h2f(0x3800) == 0.5
    assert np.float32(h2f(0x0001)) == np.float32(5.9604645e-8)
    assert abs(h2f(0x03FF) - 6.097555e-5) < 1e-10
    assert np.isposinf(h2f(0x7C00)) and np.isnan(h2f(0x7E00))


def test_f32_to_half_roundtrips_and_rounds(oracle):
    """src/gguf.rs:968-984"""
    f2h, h2f = oracle.lib.or_f32_to_half, oracle.lib.or_half_to_f32
    assert f2h(1.0) == 0x3C00 and f2h(-2.0) == 0xC000 and f2h(0.5) == 0x3800 and f2h(0.0) == 0
    assert f2h(float("inf")) == 0x7C00 and f2h(float("-inf")) == 0xFC00
    s = 0x12345678
    M = (1 << 64) - 1
    for _ in range(2000):
        s ^= (s << 13) & M
        s ^= s >> 7
        s ^= (s << 17) & M
        v = np.float32(np.float32(np.float32(s >> 40) / np.float32(1 << 24)) * np.float32(20.0)) - np.float32(10.0)
        back = h2f(f2h(float(v)))
        assert abs(back - v) <= max(abs(v), 1e-3) * 1e-3


def test_softmax_rows_are_normalized_and_mask_safe(oracle):
    """src/kernels.rs:841-853"""
    x = np.array([1.0, 2.0, 3.0, -np.inf, 0.0, 0.0, 0.0, 0.0], np.float32)
    y = oracle.softmax_rows(x, 4)
    assert abs(y[:4].sum() - 1.0) < 1e-6 and y[3] == 0.0
    assert abs(y[4:].sum() - 1.0) < 1e-6 and np.all(np.abs(y[4:] - 0.25) < 1e-6)
    with pytest.raises(ValueError):
        oracle.softmax_rows(x, 3)


def test_cache_grows_per_token_and_indexes(oracle):
    """src/forward.rs:767-784 (mini geometry: 2 kv heads x 16 dims, layer 3 of 4)"""
    c = oracle.cache(MODE_F32, n_layer=4, n_head=4, n_kv=2, hd=16, n_rot=8,
                     sections=np.array([2, 1, 1, 0], np.int32), freq_base=1e4)
    assert c.n_pos(3) == 0
    krow = np.arange(32, dtype=np.float32)
    vrow = -np.arange(32, dtype=np.float32)
    c.append(3, krow, vrow, 0)  # position 0: the rope is the identity there
    c.append(3, krow, vrow, 0)
    assert c.n_pos(3) == 2 and c.n_pos(0) == 0
    d = c.dump(3)
    k, v = d["k"].ravel(), d["v"].ravel()
    assert k[0] == 0.0 and k[31] == 31.0 and k[32] == 0.0 and v[32 + 16] == -16.0


def test_check_attn_recipe(oracle):
    """src/bin/bonsai-vk.rs:315-372: 24 heads, 4 kv, hd 256, n_pos 37, tol 1e-4, against the
    recipe's own plain-f32 softmax (here in numpy float64 as the neutral reference)."""
    nh, nkv, hd, n_pos = 24, 4, 256, 37
    q = rng_list(oracle, 0x1010, nh * hd).reshape(nh, hd)
    kc = rng_list(oracle, 0x2020, n_pos * nkv * hd).reshape(n_pos, nkv, hd)
    vc = rng_list(oracle, 0x3030, n_pos * nkv * hd).reshape(n_pos, nkv, hd)
    c = oracle.cache(MODE_F32, n_rot=0 + 64)
    # position 0 for every token: rope is the identity, so the cache holds kc as given
    for p in range(n_pos):
        c.append(0, kc[p], vc[p], 0)
    got = c.attend(0, q, 0, n_pos)
    for h in range(nh):
        kv = h // 6
        s = (kc[:, kv, :].astype(np.float64) @ q[h].astype(np.float64)) / 16.0
        p = np.exp(s - s.max())
        p /= p.sum()
        want = p @ vc[:, kv, :].astype(np.float64)
        assert np.max(np.abs(got[h] - want)) < 1e-4


def test_planar_bits_outside_range_rejected(oracle):
    """src/kvquant.rs:337 asserts bits in 1..=8"""
    for b in (0, 9):
        with pytest.raises(AssertionError):
            oracle.pq(HD, b)


def test_threads_do_not_change_results(oracle):
    c = oracle.cache(MODE_PLANAR, 4, True)
    for p in range(9):
        c.append(0, rng_list(oracle, 100 + p, 1024), rng_list(oracle, 200 + p, 1024), p)
    q = rng_list(oracle, 300, 24 * 256)
    a = c.attend(0, q, 8, 9, threads=1)
    b = c.attend(0, q, 8, 9, threads=4)
    assert np.array_equal(bits_of(a), bits_of(b))


# ---------------------------------------------------------------------------
# (2) the independent Python restatement's fixture
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("bits", range(1, 9))
def test_golden_codebook(oracle, golden, bits):
    assert np.array_equal(bits_of(oracle.codebook(HD, bits)), golden[f"codebook_b{bits}"])
    assert oracle.lloyd_iters(1.0 / 16.0, bits) == int(golden[f"codebook_iters_b{bits}"][0])


def test_codebook_iteration_cap_is_part_of_the_format(oracle):
    its = [oracle.lloyd_iters(1.0 / 16.0, b) for b in range(1, 9)]
    assert its[3:] == [300] * 5 and all(i < 300 for i in its[:3])


def test_golden_givens_and_splitmix(oracle, golden):
    import ctypes as C
    assert np.array_equal(bits_of(oracle.givens(HD)), golden["givens"])
    st = C.c_uint64(42)
    assert oracle.lib.or_splitmix64(C.byref(st)) == int(golden["splitmix_first"][0]) == 0xBDD732262FEB6E95


def test_golden_rand_floats(oracle, golden):
    assert np.array_equal(bits_of(oracle.rand_floats(0x1010, 64)), golden["rand_0x1010"])


def test_golden_f16(oracle, golden):
    vin = golden["f16_in"].view(np.float32)
    got = np.array([oracle.lib.or_f32_to_half(float(v)) for v in vin], np.uint16)
    assert np.array_equal(got, golden["f16_out"])
    back = np.array([oracle.lib.or_half_to_f32(int(h)) for h in golden["half_in"]], np.float32)
    assert np.array_equal(bits_of(back), golden["half_out"])


def test_golden_rope(oracle, golden):
    head = golden["rope_in"].view(np.float32)
    for pos, want in zip(golden["rope_pos"], golden["rope_out"]):
        got = np.concatenate([oracle.rope(head[h * HD:(h + 1) * HD], *[int(p) for p in pos]) for h in range(2)])
        assert np.array_equal(bits_of(got), want), pos


@pytest.mark.parametrize("bits", range(1, 9))
def test_golden_quantize(oracle, golden, bits):
    p = oracle.pq(HD, bits)
    x = golden["quant_in"].view(np.float32)
    for r in range(x.shape[0]):
        packed, norm = p.quantize(x[r])
        assert np.array_equal(packed, golden[f"quant_bytes_b{bits}"][r]), (bits, r)
        assert bits_of(norm)[()] == golden[f"quant_norm_b{bits}"][r]


def test_golden_softmax(oracle, golden):
    assert np.array_equal(bits_of(oracle.softmax_rows(golden["softmax_in"], 4)), golden["softmax_out"])


@pytest.mark.parametrize("tag,mode,bits,vq", [("f32", MODE_F32, 0, False), ("f16", MODE_F16, 0, False),
                                              ("planar4", MODE_PLANAR, 4, True),
                                              ("planar3", MODE_PLANAR, 3, True),
                                              ("planar4k", MODE_PLANAR, 4, False)])
def test_golden_attention_steps(oracle, golden, tag, mode, bits, vq):
    """Three decode steps from an empty cache: outputs and every stored byte are bit-equal."""
    c = oracle.cache(mode, bits, vq)
    seed = 0xA000
    want = golden[f"attn_{tag}_out"]
    for pos in range(want.shape[0]):
        q = oracle.rand_floats(seed + 3 * pos, 24 * HD)
        k = oracle.rand_floats(seed + 3 * pos + 1, 4 * HD)
        v = oracle.rand_floats(seed + 3 * pos + 2, 4 * HD)
        out = c.step(0, q, k, v, pos)
        assert np.array_equal(bits_of(out.ravel()), want[pos]), (tag, pos)
    d = c.dump(0)
    n = want.shape[0]
    gk, gv = golden[f"attn_{tag}_k"], golden[f"attn_{tag}_v"]
    if mode == MODE_PLANAR:
        assert np.array_equal(d["kq"].reshape(n * 4, -1), gk)
        assert np.array_equal(bits_of(d["kn"].ravel()), golden[f"attn_{tag}_kn"])
        if vq:
            assert np.array_equal(d["vq"].reshape(n * 4, -1), gv)
            assert np.array_equal(bits_of(d["vn"].ravel()), golden[f"attn_{tag}_vn"])
        else:
            assert np.array_equal(bits_of(d["v"].reshape(n * 4, -1)), bits_of(gv))
    elif mode == MODE_F16:
        assert np.array_equal(d["k16"].reshape(n * 4, -1), gk) and np.array_equal(d["v16"].reshape(n * 4, -1), gv)
    else:
        assert np.array_equal(bits_of(d["k"].reshape(n * 4, -1)), bits_of(gk))
        assert np.array_equal(bits_of(d["v"].reshape(n * 4, -1)), bits_of(gv))


# ---------------------------------------------------------------------------
# the layer form of the step: q|gate split, per-head RMSNorm, sigmoid gate
# ---------------------------------------------------------------------------

def test_rms_norm_rows_matches_single_row_math(oracle):
    """src/kernels.rs:790-811"""
    x = np.array([1.0, 2.0, 3.0, 4.0, 0.5, -0.5, 2.0, -3.0], np.float32)
    w = np.array([0.5, 1.0, 1.5, 2.0], np.float32)
    eps = np.float32(1e-6)
    y = oracle.rms_norm_rows(x, w, 4, eps)
    for row in range(2):
        src = x[4 * row:4 * row + 4]
        ss = np.float32(0)
        for v in src:
            ss = np.float32(ss + v * v)
        scale = np.float32(1.0) / np.sqrt(np.float32(ss / np.float32(4.0) + eps))
        for i in range(4):
            assert abs(y[4 * row + i] - src[i] * scale * w[i]) < 1e-6
    with pytest.raises(ValueError):
        oracle.rms_norm_rows(x, w, 3, eps)
    with pytest.raises(ValueError):
        oracle.rms_norm_rows(x, w[:2], 4, eps)


def test_sigmoid_hits_expected_points(oracle):
    """src/kernels.rs:834-835"""
    assert abs(oracle.sigmoid(0.0) - 0.5) < 1e-7
    assert oracle.sigmoid(-1000.0) == 0.0


def test_golden_rms_norm_and_sigmoid(oracle, layer_golden):
    g = layer_golden
    y = oracle.rms_norm_rows(g["rms_small_x"], g["rms_small_w"], 4, 1e-6)
    assert np.array_equal(bits_of(y), g["rms_small_out"])
    y = oracle.rms_norm_rows(g["rms_rows_x"].view(np.float32), g["rms_rows_w"].view(np.float32), HD, 1e-6)
    assert np.array_equal(bits_of(y), g["rms_rows_out"])
    got = np.array([oracle.sigmoid(float(v)) for v in g["sigmoid_in"]], np.float32)
    assert np.array_equal(bits_of(got), g["sigmoid_out"])


@pytest.mark.parametrize("tag,mode,bits,vq", [("planar4", MODE_PLANAR, 4, True), ("f16", MODE_F16, 0, False)])
def test_golden_layer_steps(oracle, layer_golden, tag, mode, bits, vq):
    """Three layer steps from an empty cache: gated outputs and stored bytes are bit-equal."""
    g = {k[len(f"layer_{tag}_"):]: v for k, v in layer_golden.items() if k.startswith(f"layer_{tag}_")}
    f = lambda a: a.view(np.float32)
    c = oracle.cache(mode, bits, vq)
    n = g["out"].shape[0]
    for pos in range(n):
        out = c.layer_step(0, f(g["qfull"])[pos], f(g["kraw"])[pos], f(g["vraw"])[pos], f(g["qw"]), f(g["kw"]), 1e-6, pos)
        assert np.array_equal(bits_of(out.ravel()), g["out"][pos]), (tag, pos)
    d = c.dump(0)
    if mode == MODE_PLANAR:
        assert np.array_equal(d["kq"].reshape(n * 4, -1), g["k"]) and np.array_equal(d["vq"].reshape(n * 4, -1), g["v"])
        assert np.array_equal(bits_of(d["kn"].ravel()), g["kn"]) and np.array_equal(bits_of(d["vn"].ravel()), g["vn"])
    else:
        assert np.array_equal(d["k16"].reshape(n * 4, -1), g["k"]) and np.array_equal(d["v16"].reshape(n * 4, -1), g["v"])
