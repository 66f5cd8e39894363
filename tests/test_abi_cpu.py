"""CPU-side checks of the C ABI: the library loads, exports every declared symbol, and its
host-side pieces (mode parser, environment readers, set-up tables) agree with the oracle.
No compute entry point is called here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from oracle_lib import MODE_F16, MODE_F32, MODE_PLANAR

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "bonsai_kv.h")).read()
    return sorted(set(re.findall(r"BK_API[^;(]*?\b(bk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(bk):
    lib = C.CDLL(bk.library_path())
    names = declared_symbols()
    assert len(names) >= 50
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/bonsai_kv.h but not exported"


def test_ctypes_table_covers_the_header(bk):
    assert sorted(bk._abi.SIGNATURES) == declared_symbols()


def test_version_and_status_strings(bk):
    lib = bk._abi.load()
    assert b"sm_100a" in lib.bk_version()
    assert lib.bk_status_string(0) == b"ok" and lib.bk_status_string(4).startswith(b"position")


def test_parse_mode_matches_reference_table(bk, oracle):
    """src/kvquant.rs:670-720 through the ABI, cross-checked with the oracle on more strings."""
    kinds = {MODE_F32: "f32", MODE_F16: "f16", MODE_PLANAR: "planar"}
    cases = ["", "f32", "f16", "fp16", "half", "planar4", "planar4k", "iso3", "iso8k", "planar9", "planar0",
             "garbage", "planark", "planar", "iso", "isok", "planar1", "planar8", "iso1k", "planar+4",
             "planar04", "planar4kk", "PLANAR4", "planar 4", "planar4 ", "k", "f16k", "planar-1", "iso99999999999"]
    for s in cases:
        kind, bits, vq = oracle.parse_mode(s)
        m = bk.parse_mode(s)
        assert (m.kind, m.bits, m.v_quant) == (kinds[kind], bits, vq), s
    assert bk.parse_mode("planar4") == bk.Planar(4, True)
    assert bk.parse_mode("iso8k") == bk.Planar(8, False)


def test_quantizers_follow_the_mode(bk):
    """src/kvquant.rs:711-719 (construction only; no GPU call)."""
    class FakeCtx:  # quantizers_for only stores the context
        pass
    k, v = bk.quantizers_for(bk.parse_mode("planar4"), 256, FakeCtx())
    assert k is not None and v is not None
    k, v = bk.quantizers_for(bk.parse_mode("planar4k"), 256, FakeCtx())
    assert k is not None and v is None
    assert bk.quantizers_for(bk.parse_mode("f16"), 256, FakeCtx()) == (None, None)
    assert bk.quantizers_for(bk.parse_mode("f32"), 256, FakeCtx()) == (None, None)
    with pytest.raises(AssertionError):
        bk.PlanarQuant(256, 9, FakeCtx())
    assert bk.PlanarQuant(256, 3, FakeCtx()).packed_len() == 96


def test_env_readers(bk, monkeypatch):
    """BONSAI_KV (src/kvquant.rs:546-550) and BONSAI_CTX (src/gdev.rs:39-48)."""
    monkeypatch.delenv("BONSAI_KV", raising=False)
    monkeypatch.delenv("BONSAI_CTX", raising=False)
    assert bk.mode_from_env() == bk.F32 and bk.n_ctx_env() == 2048
    monkeypatch.setenv("BONSAI_KV", "planar3k")
    assert bk.mode_from_env() == bk.Planar(3, False)
    for val, want in [("16", 16), ("262144", 262144), ("15", 2048), ("262145", 2048), ("abc", 2048), ("4096", 4096)]:
        monkeypatch.setenv("BONSAI_CTX", val)
        assert bk.n_ctx_env() == want, val


@pytest.mark.parametrize("bits", range(1, 9))
def test_setup_tables_equal_the_oracle(bk, oracle, bits):
    """The library's own host set-up code (not the oracle) builds the codebook and the
    Givens table; both must equal the oracle's bit for bit."""
    assert np.array_equal(bk.codebook(256, bits).view(np.uint32), oracle.codebook(256, bits).view(np.uint32))
    assert np.array_equal(bk.givens_table(256).view(np.uint32), oracle.givens(256).view(np.uint32))
    assert bk.packed_bytes(256, bits) == 32 * bits == bk._abi.load().bk_kvq_packed_len(256, bits)


@pytest.mark.parametrize("bits", [1, 2, 3, 4])
def test_threshold_cells_give_the_reference_scan(bk, oracle, bits):
    """The bulk append finds the nearest centroid with one table read and one comparison.  The table is built
    on the host; here it is checked against the reference's scan (src/kvquant.rs:357-370: ascending, strict
    '<', f32 differences) on the values where the two could part: centroids, exact midpoints, the decision
    thresholds themselves, cell edges, each with their neighbouring floats, and a dense random sample."""
    lib = bk._abi.load()
    cells = np.zeros((512, 2), np.uint32)
    assert lib.bk_kvq_threshold_cells(bits, cells.ctypes.data) == 0
    count, thr = cells[:, 0].astype(np.int64), cells[:, 1].copy().view(np.float32)
    book = oracle.codebook(256, bits).astype(np.float32)
    n = 1 << bits
    assert count[0] == 0 and count[-1] + np.isfinite(thr[-1]) <= n - 1 and np.all(np.diff(count) >= 0)
    assert int(np.isfinite(thr).sum()) == n - 1            # every threshold sits in a cell of its own

    def neighbours(x, k=3):
        out = [np.float32(x)]
        lo = hi = np.float32(x)
        for _ in range(k):
            lo, hi = np.nextafter(lo, np.float32(-np.inf)), np.nextafter(hi, np.float32(np.inf))
            out += [lo, hi]
        return out
    probes = []
    for c in book:
        probes += neighbours(c)
    for a, b in zip(book[:-1], book[1:]):
        probes += neighbours(np.float32(0.5) * (a + b)) + neighbours(np.float32((np.float64(a) + np.float64(b)) / 2))
    for t in thr[np.isfinite(thr)]:
        probes += neighbours(t, 5)
    for k in range(0, 513):
        probes += neighbours(np.float32(k) / np.float32(1024) - np.float32(0.25))
    probes += [np.float32(x) for x in (-3.9, -1.0, -0.26, -0.25, 0.0, -0.0, 0.25, 0.26, 1.0, 3.9)]
    rng = np.random.default_rng(bits)
    v = np.concatenate([np.array(probes, np.float32), (rng.standard_normal(200000) / 16).astype(np.float32),
                        rng.uniform(-0.3, 0.3, 200000).astype(np.float32)])
    want = np.argmin(np.abs(v[:, None] - book[None, :]), axis=1)       # f32 differences; first minimum = lowest index
    cell = np.clip(np.floor((v + np.float32(0.25)) * np.float32(1024)).astype(np.int64), 0, 511)
    got = count[cell] + (v >= thr[cell])
    bad = np.flatnonzero(got != want)
    assert bad.size == 0, (v[bad[:5]], got[bad[:5]], want[bad[:5]])


def test_default_config_is_qwen35(bk):
    cfg = bk._abi.CacheConfig()
    bk._abi.load().bk_default_config(C.byref(cfg))
    assert (cfg.n_layers, cfg.n_head, cfg.n_kv, cfg.hd, cfg.n_rot) == (16, 24, 4, 256, 64)
    assert list(cfg.sections) == [11, 11, 10, 0] and cfg.freq_base == np.float32(1e7)


def test_null_arguments_are_rejected_without_a_device(bk):
    lib = bk._abi.load()
    assert lib.bk_synchronize(None) == bk._abi.BK_ERR_INVALID
    assert lib.bk_cache_n_pos(None, 0, 0) == -1
    assert lib.bk_kvq_packed_len(256, 0) == 0 and lib.bk_kvq_packed_len(256, 9) == 0
    assert lib.bk_parse_mode(None, None) == bk._abi.BK_ERR_INVALID
    assert lib.bk_ctx_create(0, None) == bk._abi.BK_ERR_INVALID
    assert lib.bk_lse_merge(None, 1, 1, 256, None, None) == bk._abi.BK_ERR_INVALID


def test_no_cpu_fallback(bk):
    """Without a GPU the context cannot be created and says why; nothing computes on the CPU."""
    import shutil
    if shutil.which("nvidia-smi"):
        pytest.skip("a GPU is present")
    with pytest.raises(bk.BonsaiKvError) as e:
        bk.Context(0)
    assert e.value.status in (bk._abi.BK_ERR_CUDA, bk._abi.BK_ERR_INVALID)
