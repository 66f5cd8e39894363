"""bk_decode_attn_noalloc against bk_decode_attn.

The no-alloc entry point exists for hosts that may not allocate once they are serving (all of
HBM already belongs to the caches; a later cudaMalloc would synchronise the device or fail on a
fragmented heap) or that call from a thread where the CUDA allocator must not be entered.  It
keeps its split-K scratch in a fixed array inside the library.  This file checks, through the C
ABI, that it returns what the ordinary entry point returns AND what the CPU oracle computes, on two
calls in a row (the second call finds the array as the first left it), and that it rejects requests
beyond its stated limits.  It is named to be collected last and runs on its own as well as after the other tests.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

NH, NKV, HD = 24, 4, 256
ABS_TOL = REL_TOL = 1e-3  # the bar the other GPU parity tests use


def _decode(cache, fn, q_dev, out_dev, n_seqs):
    cache.ctx.check(fn(cache.h, 0, n_seqs, None, None, None, q_dev.ptr, out_dev.ptr))
    return out_dev.download((n_seqs, NH, HD), np.float32)


@pytest.mark.parametrize("tag", ["planar4", "f16"])
def test_noalloc_matches_regular_entry_point_twice(bk, gpu_ctx, oracle, tag):
    from oracle_lib import MODE_F16, MODE_PLANAR
    rng = np.random.default_rng(5)
    lens = [5000, 300, 0, 2048]           # both kernels, many chunks, an empty sequence
    cache = bk.AttnCache(gpu_ctx, bk.parse_mode(tag), n_layers=1, n_seqs=len(lens), n_ctx=max(lens))
    refs = []
    for s, n in enumerate(lens):
        ref = oracle.cache(MODE_PLANAR, 4, True) if tag == "planar4" else oracle.cache(MODE_F16)
        refs.append(ref)
        if n:
            k = rng.standard_normal((n, NKV, HD)).astype(np.float32)
            v = rng.standard_normal((n, NKV, HD)).astype(np.float32)
            k[:, :, [3, 77, 190]] *= np.float32(20.0)
            v[:, :, [3, 77, 190]] *= np.float32(20.0)
            cache.append(0, k, v, seq=s)
            for p in range(n):
                ref.append(0, k[p], v[p], p)
    lib = gpu_ctx.lib
    out_a, out_b = gpu_ctx.alloc(len(lens) * NH * HD * 4), gpu_ctx.alloc(len(lens) * NH * HD * 4)
    for call in range(2):                 # two calls in a row through the new entry point
        q = rng.standard_normal((len(lens), NH, HD)).astype(np.float32)
        q_dev = gpu_ctx.to_device(q)
        want = _decode(cache, lib.bk_decode_attn, q_dev, out_a, len(lens))
        got = _decode(cache, lib.bk_decode_attn_noalloc, q_dev, out_b, len(lens))
        err = np.max(np.abs(got.astype(np.float64) - want))
        assert err <= ABS_TOL and err / max(np.max(np.abs(want)), 1e-30) <= REL_TOL, (tag, call, err)
        assert np.all(got[2] == 0.0)
        for s, n in enumerate(lens):          # third column: the CPU oracle
            if n:
                cpu = refs[s].attend(0, q[s], n - 1, n, threads=8).astype(np.float64)
                e2 = np.max(np.abs(got[s] - cpu))
                assert e2 <= ABS_TOL and e2 / max(np.max(np.abs(cpu)), 1e-30) <= REL_TOL, (tag, call, s, e2)
        q_dev.free()
    cache.close()


def test_noalloc_rejects_sizes_beyond_its_scratch(bk, gpu_ctx):
    cache = bk.AttnCache(gpu_ctx, bk.F32, n_layers=1, n_seqs=1, n_ctx=8)
    lib = gpu_ctx.lib
    buf = gpu_ctx.alloc(65 * NH * HD * 4)
    ids = (C.c_int32 * 65)(*([0] * 65))
    st = lib.bk_decode_attn_noalloc(cache.h, 0, 65, ids, None, None, buf.ptr, buf.ptr)
    assert st == bk._abi.BK_ERR_INVALID and b"64 sequences" in lib.bk_last_error(gpu_ctx.h)
    assert lib.bk_decode_attn_noalloc(cache.h, 3, 1, None, None, None, buf.ptr, buf.ptr) == bk._abi.BK_ERR_INVALID
    assert lib.bk_decode_attn_noalloc(cache.h, 0, 1, None, None, None, None, buf.ptr) == bk._abi.BK_ERR_INVALID
    cache.close()
