"""ctypes binding of oracle/libbonsai_oracle.so (the CPU checker).

Only tests, the smoke check and the benchmark's CPU baseline may import this.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
MODE_F32, MODE_F16, MODE_PLANAR = 0, 1, 2

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


def build_oracle():
    so = os.path.join(ORACLE_DIR, "libbonsai_oracle.so")
    src = os.path.join(ORACLE_DIR, "bonsai_oracle.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", ORACLE_DIR, "-s"])
    return so


def load_oracle():
    lib = C.CDLL(build_oracle())
    sz, u, i, f, d, vp = C.c_size_t, C.c_uint, C.c_int, C.c_float, C.c_double, C.c_void_p
    sigs = {
        "or_solve_lloyd_max": (i, [d, u, _f32p]),
        "or_codebook": (None, [sz, u, _f32p]),
        "or_expected_distortion": (f, [sz, u]),
        "or_splitmix64": (C.c_uint64, [C.POINTER(C.c_uint64)]),
        "or_givens_table": (None, [sz, _f32p]),
        "or_packed_bytes": (sz, [sz, u]),
        "or_pack_bits": (None, [_u8p, sz, u, _u8p]),
        "or_unpack_bits": (None, [_u8p, u, sz, _u8p]),
        "or_pack_idx": (None, [_u8p, sz, u, _u8p]),
        "or_unpack_idx": (None, [_u8p, sz, u, _u8p]),
        "or_pq_new": (vp, [sz, u]),
        "or_pq_free": (None, [vp]),
        "or_pq_packed_len": (sz, [vp]),
        "or_pq_rotate": (None, [vp, _f32p, sz, _f32p]),
        "or_pq_rotate_inv": (None, [vp, _f32p, sz, _f32p]),
        "or_pq_quantize": (None, [vp, _f32p, _u8p, C.POINTER(f)]),
        "or_pq_dequantize": (None, [vp, _u8p, f, _f32p]),
        "or_pq_dot_rotated": (f, [vp, _f32p, _u8p, f]),
        "or_parse_mode": (None, [C.c_char_p, C.POINTER(i), C.POINTER(i), C.POINTER(i)]),
        "or_rope_imrope": (None, [_f32p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, sz, _i32p, f]),
        "or_half_to_f32": (f, [C.c_uint16]),
        "or_f32_to_half": (C.c_uint16, [f]),
        "or_softmax_rows": (i, [_f32p, sz, sz, _f32p]),
        "or_cache_new": (vp, [sz, sz, sz, sz, sz, _i32p, f, i, i, i]),
        "or_cache_free": (None, [vp]),
        "or_cache_reset": (None, [vp]),
        "or_cache_n_pos": (sz, [vp, sz]),
        "or_append_token": (None, [vp, sz, _f32p, _f32p, sz]),
        "or_attend": (i, [vp, sz, _f32p, sz, sz, _f32p, i]),
        "or_attn_step": (i, [vp, sz, _f32p, _f32p, _f32p, sz, _f32p, i]),
        "or_rms_norm_rows": (i, [_f32p, sz, _f32p, sz, sz, C.c_float, _f32p]),
        "or_sigmoid": (C.c_float, [C.c_float]),
        "or_attn_layer_step": (i, [vp, sz, _f32p, _f32p, _f32p, _f32p, _f32p, C.c_float, sz, _f32p, i]),
        "or_rand_floats": (None, [C.c_uint64, sz, _f32p]),
        "or_pq2_row_bytes": (sz, [sz]),
        "or_pq2_decode_row": (None, [_u8p, sz, _f32p]),
        "or_pq2_dot_row": (i, [_u8p, sz, sz, sz, _f32p, _f32p]),
        "or_pq2_matmul": (i, [_u8p, sz, sz, sz, sz, _f32p, sz, _f32p]),
        "or_max_threads": (i, []),
    }
    for name in ("or_cache_k", "or_cache_v", "or_cache_k16", "or_cache_v16", "or_cache_kq",
                 "or_cache_vq", "or_cache_kn", "or_cache_vn"):
        sigs[name] = (vp, [vp, sz])
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return Oracle(lib)


SECTIONS = np.array([11, 11, 10, 0], dtype=np.int32)


class OracleCache:
    """The reference's AttnCache + attention step (src/forward.rs:30-140, 247-375) on the CPU."""

    def __init__(self, lib, mode, bits=0, v_quant=False, n_layer=1, n_head=24, n_kv=4, hd=256,
                 n_rot=64, sections=SECTIONS, freq_base=1e7):
        self.lib, self.mode, self.bits, self.v_quant = lib, mode, bits, bool(v_quant)
        self.n_head, self.n_kv, self.hd = n_head, n_kv, hd
        self.h = lib.or_cache_new(n_layer, n_head, n_kv, hd, n_rot,
                                  np.ascontiguousarray(sections, dtype=np.int32), freq_base,
                                  mode, bits, int(v_quant))

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.or_cache_free(self.h)
            self.h = None

    def n_pos(self, il=0):
        return self.lib.or_cache_n_pos(self.h, il)

    def reset(self):
        self.lib.or_cache_reset(self.h)

    def append(self, il, k, v, pos):
        self.lib.or_append_token(self.h, il, np.ascontiguousarray(k, np.float32).ravel(),
                                 np.ascontiguousarray(v, np.float32).ravel(), pos)

    def attend(self, il, q, q_pos, n_pos, threads=1):
        out = np.zeros(self.n_head * self.hd, dtype=np.float32)
        rc = self.lib.or_attend(self.h, il, np.ascontiguousarray(q, np.float32).ravel(), q_pos, n_pos,
                                out, threads)
        if rc != 0:
            raise ValueError(f"or_attend rc={rc}")
        return out.reshape(self.n_head, self.hd)

    def step(self, il, q, k, v, pos, threads=1):
        out = np.zeros(self.n_head * self.hd, dtype=np.float32)
        rc = self.lib.or_attn_step(self.h, il, np.ascontiguousarray(q, np.float32).ravel(),
                                   np.ascontiguousarray(k, np.float32).ravel(),
                                   np.ascontiguousarray(v, np.float32).ravel(), pos, out, threads)
        if rc != 0:
            raise ValueError(f"or_attn_step rc={rc}")
        return out.reshape(self.n_head, self.hd)

    def layer_step(self, il, qfull, kraw, vraw, q_norm_w, k_norm_w, eps, pos, threads=1):
        """src/forward.rs:237-382 without the matvecs."""
        out = np.zeros(self.n_head * self.hd, dtype=np.float32)
        f = lambda a: np.ascontiguousarray(a, np.float32).ravel()
        rc = self.lib.or_attn_layer_step(self.h, il, f(qfull), f(kraw), f(vraw), f(q_norm_w), f(k_norm_w), eps, pos,
                                         out, threads)
        if rc != 0:
            raise ValueError(f"or_attn_layer_step rc={rc}")
        return out.reshape(self.n_head, self.hd)

    def _view(self, fn, il, count, dtype):
        ptr = fn(self.h, il)
        if not ptr or count == 0:
            return np.zeros(0, dtype=dtype)
        buf = (C.c_char * (count * np.dtype(dtype).itemsize)).from_address(ptr)
        return np.frombuffer(buf, dtype=dtype).copy()

    def dump(self, il=0):
        """Stores of one layer as the reference lays them out ([token][kv_head][...])."""
        n, nkv, hd = self.n_pos(il), self.n_kv, self.hd
        L = self.lib
        if self.mode == MODE_PLANAR:
            plen = 32 * self.bits * hd // 256
            d = {"kq": self._view(L.or_cache_kq, il, n * nkv * plen, np.uint8).reshape(n, nkv, plen),
                 "kn": self._view(L.or_cache_kn, il, n * nkv, np.float32).reshape(n, nkv)}
            if self.v_quant:
                d["vq"] = self._view(L.or_cache_vq, il, n * nkv * plen, np.uint8).reshape(n, nkv, plen)
                d["vn"] = self._view(L.or_cache_vn, il, n * nkv, np.float32).reshape(n, nkv)
            else:
                d["v"] = self._view(L.or_cache_v, il, n * nkv * hd, np.float32).reshape(n, nkv, hd)
            return d
        if self.mode == MODE_F16:
            return {"k16": self._view(L.or_cache_k16, il, n * nkv * hd, np.uint16).reshape(n, nkv, hd),
                    "v16": self._view(L.or_cache_v16, il, n * nkv * hd, np.uint16).reshape(n, nkv, hd)}
        return {"k": self._view(L.or_cache_k, il, n * nkv * hd, np.float32).reshape(n, nkv, hd),
                "v": self._view(L.or_cache_v, il, n * nkv * hd, np.float32).reshape(n, nkv, hd)}


class Oracle:
    def __init__(self, lib):
        self.lib = lib

    def codebook(self, d, bits):
        out = np.zeros(1 << bits, dtype=np.float32)
        self.lib.or_codebook(d, bits, out)
        return out

    def lloyd_iters(self, sigma, bits):
        out = np.zeros(1 << bits, dtype=np.float32)
        return self.lib.or_solve_lloyd_max(sigma, bits, out)

    def givens(self, d):
        out = np.zeros(((d + 1) // 2) * 2, dtype=np.float32)
        self.lib.or_givens_table(d, out)
        return out.reshape(-1, 2)

    def rand_floats(self, seed, n):
        out = np.zeros(n, dtype=np.float32)
        self.lib.or_rand_floats(seed, n, out)
        return out

    def parse_mode(self, s):
        m, b, v = C.c_int(), C.c_int(), C.c_int()
        self.lib.or_parse_mode(s.encode(), C.byref(m), C.byref(b), C.byref(v))
        return m.value, b.value, bool(v.value)

    def rope(self, head, p_t, p_h, p_w, p_e, n_dims=64, sections=SECTIONS, freq_base=1e7):
        h = np.ascontiguousarray(head, dtype=np.float32).copy()
        self.lib.or_rope_imrope(h, p_t, p_h, p_w, p_e, n_dims, np.ascontiguousarray(sections, np.int32), freq_base)
        return h

    def softmax_rows(self, x, row_len):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.zeros_like(x)
        rc = self.lib.or_softmax_rows(x, x.size, row_len, out)
        if rc != 0:
            raise ValueError("softmax_rows: length not divisible by row_len")
        return out

    def rms_norm_rows(self, x, w, row_len, eps):
        x = np.ascontiguousarray(x, dtype=np.float32).ravel()
        w = np.ascontiguousarray(w, dtype=np.float32).ravel()
        out = np.zeros_like(x)
        rc = self.lib.or_rms_norm_rows(x, x.size, w, w.size, row_len, eps, out)
        if rc != 0:
            raise ValueError("rms_norm_rows: bad weight length or ragged x")
        return out

    def sigmoid(self, x):
        return float(self.lib.or_sigmoid(x))

    # ---- PQ2_0 ternary rows (src/kernels.rs:204-420) ----
    def pq2_row_bytes(self, ne0):
        return int(self.lib.or_pq2_row_bytes(ne0))

    def pq2_decode_row(self, raw, ne0):
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        out = np.zeros(ne0, np.float32)
        self.lib.or_pq2_decode_row(raw, ne0, out)
        return out

    def pq2_dot_row(self, payload, ne0, row, x):
        payload = np.ascontiguousarray(payload, dtype=np.uint8)
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.size != ne0:
            raise ValueError("dot_pq2_0_row: x length")
        out = np.zeros(1, np.float32)
        if self.lib.or_pq2_dot_row(payload, payload.size, ne0, row, x, out) != 0:
            raise ValueError("dot_pq2_0_row: row outside the payload")
        return float(out[0])

    def pq2_matmul(self, payload, ne0, base_row, n_rows, x, n_tok=1):
        payload = np.ascontiguousarray(payload, dtype=np.uint8)
        x = np.ascontiguousarray(x, dtype=np.float32).ravel()
        if x.size != n_tok * ne0:
            raise ValueError("pq2_matmul_n: x length")
        y = np.zeros(n_tok * n_rows, np.float32)
        if self.lib.or_pq2_matmul(payload, payload.size, ne0, base_row, n_rows, x, n_tok, y) != 0:
            raise ValueError("pq2_matmul_n: row range exceeds payload")
        return y.reshape(n_tok, n_rows)

    def pq(self, hd, bits):
        return OraclePQ(self.lib, hd, bits)

    def cache(self, mode, bits=0, v_quant=False, **kw):
        return OracleCache(self.lib, mode, bits, v_quant, **kw)


class OraclePQ:
    """PlanarQuant of src/kvquant.rs:325-478."""

    def __init__(self, lib, hd, bits):
        self.lib, self.hd, self.bits = lib, hd, bits
        self.h = lib.or_pq_new(hd, bits)
        if not self.h:
            raise AssertionError("bits must be 1..8")
        self.hd_padded = ((hd + 1) // 2) * 2

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.or_pq_free(self.h)
            self.h = None

    def packed_len(self):
        return self.lib.or_pq_packed_len(self.h)

    def rotate(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(self.hd_padded, np.float32)
        self.lib.or_pq_rotate(self.h, x, x.size, out)
        return out

    def rotate_inv(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(self.hd_padded, np.float32)
        self.lib.or_pq_rotate_inv(self.h, x, x.size, out)
        return out

    def quantize(self, x):
        packed = np.zeros(self.packed_len(), np.uint8)
        norm = C.c_float()
        self.lib.or_pq_quantize(self.h, np.ascontiguousarray(x, np.float32), packed, C.byref(norm))
        return packed, np.float32(norm.value)

    def dequantize(self, packed, norm):
        out = np.zeros(self.hd, np.float32)
        self.lib.or_pq_dequantize(self.h, np.ascontiguousarray(packed, np.uint8), float(norm), out)
        return out

    def dot_rotated(self, q_rot, packed, norm):
        return np.float32(self.lib.or_pq_dot_rotated(self.h, np.ascontiguousarray(q_rot, np.float32),
                                                     np.ascontiguousarray(packed, np.uint8), float(norm)))
