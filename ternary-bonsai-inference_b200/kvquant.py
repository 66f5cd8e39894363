"""Host-side mirror of the reference's `src/kvquant.rs` over the C ABI.

Same names and argument meaning as the reference (`KvMode`, `parse_mode`,
`mode_from_env`, `quantizers_for`, `codebook`, `givens_table`, `PlanarQuant`),
so the parity tests read like the reference's own unit tests.  Every numeric
method runs on the GPU through libbonsai_kv.so; nothing here computes on the CPU
except the one-time tables the reference also builds on the CPU.
"""
import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _abi
from .device import Context

DEFAULT_HD = 256  # src/kvquant.rs:26


@dataclass(frozen=True)
class KvMode:
    """src/kvquant.rs:486-507.  kind is 'f32', 'f16' or 'planar'."""
    kind: str = "f32"
    bits: int = 0
    v_quant: bool = False

    def bytes_per_coord(self):
        return {"f32": 4.0, "f16": 2.0}.get(self.kind, self.bits / 8.0)

    def is_f32(self):
        return self.kind == "f32"

    def to_struct(self):
        k = {"f32": _abi.BK_MODE_F32, "f16": _abi.BK_MODE_F16, "planar": _abi.BK_MODE_PLANAR}[self.kind]
        return _abi.KvModeStruct(k, self.bits, int(self.v_quant))

    @staticmethod
    def from_struct(s):
        kind = {_abi.BK_MODE_F32: "f32", _abi.BK_MODE_F16: "f16", _abi.BK_MODE_PLANAR: "planar"}[s.kind]
        return KvMode(kind, int(s.bits), bool(s.v_quant))


F32 = KvMode("f32")
F16 = KvMode("f16")


def Planar(bits, v_quant=True):
    return KvMode("planar", bits, v_quant)


def parse_mode(s):
    """src/kvquant.rs:515-543: unknown values (and widths outside 1..8) are f32."""
    out = _abi.KvModeStruct()
    _abi.check(_abi.load().bk_parse_mode(s.encode(), C.byref(out)))
    return KvMode.from_struct(out)


def mode_from_env():
    """src/kvquant.rs:546-550: BONSAI_KV, f32 when unset."""
    out = _abi.KvModeStruct()
    _abi.check(_abi.load().bk_mode_from_env(C.byref(out)))
    return KvMode.from_struct(out)


def packed_bytes(n, bits):
    """src/kvquant.rs:184-186"""
    return (n * bits + 7) // 8


def codebook(d, bits):
    """src/kvquant.rs:103-114"""
    out = np.zeros(1 << bits, dtype=np.float32)
    _abi.check(_abi.load().bk_kvq_codebook(d, bits, out.ctypes.data))
    return out


def givens_table(d):
    """src/kvquant.rs:131-145: (cos, sin) per pair, shape [ceil(d/2), 2]."""
    out = np.zeros(((d + 1) // 2, 2), dtype=np.float32)
    _abi.check(_abi.load().bk_kvq_givens(d, out.ctypes.data))
    return out


_default_ctx = None


def default_context():
    global _default_ctx
    if _default_ctx is None:
        _default_ctx = Context(0)
    return _default_ctx


class PlanarQuant:
    """src/kvquant.rs:325-478.  Methods take one vector or a batch [n, hd]."""

    def __init__(self, hd, bits, ctx=None):
        assert 1 <= bits <= 8, "bits must be 1..8"  # src/kvquant.rs:337
        self.hd, self.bits = hd, bits
        self.n_groups = (hd + 1) // 2
        self.hd_padded = self.n_groups * 2
        self.ctx = ctx or default_context()

    def packed_len(self):
        return int(_abi.load().bk_kvq_packed_len(self.hd, self.bits))

    def centroids(self):
        return codebook(self.hd, self.bits)

    def _batch(self, x, width, dtype):
        a = np.ascontiguousarray(x, dtype=dtype)
        single = a.ndim == 1
        a = a.reshape(-1, width)
        return a, single

    def quantize(self, x):
        """-> (packed uint8 [.., packed_len], norm float32 [..])"""
        a, single = self._batch(x, self.hd, np.float32)
        n = a.shape[0]
        packed = np.zeros((n, self.packed_len()), np.uint8)
        norms = np.zeros(n, np.float32)
        c = self.ctx
        c.check(c.lib.bk_kvq_quantize(c.h, self.hd, self.bits, n, a.ctypes.data, packed.ctypes.data, norms.ctypes.data))
        return (packed[0], norms[0]) if single else (packed, norms)

    def dequantize(self, packed, norm):
        p, single = self._batch(packed, self.packed_len(), np.uint8)
        nrm = np.ascontiguousarray(norm, np.float32).reshape(-1)
        out = np.zeros((p.shape[0], self.hd), np.float32)
        c = self.ctx
        c.check(c.lib.bk_kvq_dequantize(c.h, self.hd, self.bits, p.shape[0], p.ctypes.data, nrm.ctypes.data, out.ctypes.data))
        return out[0] if single else out

    def _rot(self, x, inverse):
        a, single = self._batch(x, self.hd, np.float32)
        out = np.zeros_like(a)
        c = self.ctx
        c.check(c.lib.bk_kvq_rotate(c.h, self.hd, a.shape[0], inverse, a.ctypes.data, out.ctypes.data))
        return out[0] if single else out

    def rotate(self, x):
        return self._rot(x, 0)

    def rotate_inv(self, x):
        return self._rot(x, 1)

    def dot_rotated(self, q_rot, packed, norm):
        q, single = self._batch(q_rot, self.hd, np.float32)
        p, _ = self._batch(packed, self.packed_len(), np.uint8)
        nrm = np.ascontiguousarray(norm, np.float32).reshape(-1)
        out = np.zeros(q.shape[0], np.float32)
        c = self.ctx
        c.check(c.lib.bk_kvq_dot_rotated(c.h, self.hd, self.bits, q.shape[0], q.ctypes.data, p.ctypes.data,
                                         nrm.ctypes.data, out.ctypes.data))
        return out[0] if single else out


def quantizers_for(mode, hd, ctx=None):
    """src/kvquant.rs:554-567: (K quantizer, V quantizer), None where that side is not quantized."""
    if mode.kind == "planar":
        k = PlanarQuant(hd, mode.bits, ctx)
        return k, (PlanarQuant(hd, mode.bits, ctx) if mode.v_quant else None)
    return None, None


def rope_imrope(heads, p_t, p_h, p_w, p_e, n_dims=64, sections=(11, 11, 10, 0), freq_base=1e7, ctx=None):
    """src/rope.rs:9-70 on one head vector or a batch [n, hd]; returns the rotated copy."""
    c = ctx or default_context()
    a = np.ascontiguousarray(heads, np.float32).copy()
    flat = a.reshape(-1, a.shape[-1])
    sec = (C.c_int32 * 4)(*sections)
    c.check(c.lib.bk_rope_imrope(c.h, flat.shape[0], flat.shape[1], flat.ctypes.data, p_t, p_h, p_w, p_e,
                                 n_dims, sec, freq_base))
    return a


def f32_to_half(x, ctx=None):
    """src/gguf.rs:914-944, element-wise."""
    c = ctx or default_context()
    a = np.ascontiguousarray(x, np.float32)
    out = np.zeros(a.shape, np.uint16)
    c.check(c.lib.bk_f32_to_half(c.h, a.size, a.ctypes.data, out.ctypes.data))
    return out


def half_to_f32(h, ctx=None):
    """src/gguf.rs:881-911, element-wise."""
    c = ctx or default_context()
    a = np.ascontiguousarray(h, np.uint16)
    out = np.zeros(a.shape, np.float32)
    c.check(c.lib.bk_half_to_f32(c.h, a.size, a.ctypes.data, out.ctypes.data))
    return out
