"""Host-side mirror of the reference's attention step and its caches.

`AttnCache` keeps the shape of `src/forward.rs:30-140` (per-layer stores that
grow by one `[kv_head][head_dim]` block per token, `n_pos`, the append variants)
and of the device cache allocation in `src/gdev.rs:329-469` (everything for
`n_ctx` positions up front, mode from BONSAI_KV, context from BONSAI_CTX), with
an added sequence axis for batched decoding.  `full_attention_step` is the part
of `full_attention_layer` between the q/k RMSNorm and the sigmoid gate
(`src/forward.rs:247-375`).
"""
import ctypes as C

import numpy as np

from . import _abi
from .device import Context
from .kvquant import KvMode, mode_from_env


def n_ctx_env():
    """src/gdev.rs:39-48: BONSAI_CTX in 16..=262144, default 2048."""
    return int(_abi.load().bk_n_ctx_from_env())


def _i32_array(values):
    if values is None:
        return None
    a = np.ascontiguousarray(values, dtype=np.int32)
    return a.ctypes.data_as(C.POINTER(C.c_int32)), a


class AttnCache:
    """Device KV cache of the full-attention layers (K roped, V raw)."""

    def __init__(self, ctx=None, mode=None, n_layers=16, n_seqs=1, n_ctx=None, n_head=24, n_kv=4, hd=256,
                 n_rot=64, sections=(11, 11, 10, 0), freq_base=1e7, rope_positions=0):
        self.ctx = ctx or Context(0)
        self.mode = mode if mode is not None else mode_from_env()
        cfg = _abi.CacheConfig()
        self.ctx.lib.bk_default_config(C.byref(cfg))
        cfg.n_layers, cfg.n_seqs = n_layers, n_seqs
        cfg.n_ctx = n_ctx if n_ctx is not None else n_ctx_env()
        cfg.n_head, cfg.n_kv, cfg.hd, cfg.n_rot = n_head, n_kv, hd, n_rot
        cfg.sections = (C.c_int32 * 4)(*sections)
        cfg.freq_base = freq_base
        cfg.rope_positions = rope_positions
        cfg.mode = self.mode.to_struct()
        self.cfg = cfg
        self.n_layers, self.n_seqs, self.n_ctx = n_layers, n_seqs, cfg.n_ctx
        self.n_head, self.n_kv, self.hd = n_head, n_kv, hd
        self.n_kv_elems = n_kv * hd
        h = C.c_void_p()
        self.ctx.check(self.ctx.lib.bk_cache_create(self.ctx.h, C.byref(cfg), C.byref(h)))
        self.h = h

    def close(self):
        if getattr(self, "h", None) and self.ctx.h:
            self.ctx.lib.bk_cache_destroy(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- bookkeeping ------------------------------------------------------------
    def n_pos(self, il, seq=0):
        """src/forward.rs:78-86"""
        return int(self.ctx.lib.bk_cache_n_pos(self.h, il, seq))

    def set_n_pos(self, il, seq, n):
        self.ctx.check(self.ctx.lib.bk_cache_set_n_pos(self.h, il, seq, n))

    def reset(self, seq=-1):
        """Decoder::reset, src/forward.rs:640-656"""
        self.ctx.check(self.ctx.lib.bk_cache_reset(self.h, seq))

    def kv_quantized(self):
        """src/gdev.rs:550-552"""
        return self.mode.kind != "f32"

    def device_bytes(self):
        return int(self.ctx.lib.bk_cache_device_bytes(self.h))

    def row_bytes(self, is_v=False):
        return int(self.ctx.lib.bk_cache_row_bytes(self.h, int(is_v)))

    # -- append -----------------------------------------------------------------
    def append(self, il, krow, vrow, pos=None, seq=0):
        """src/forward.rs:259-285: rope K at `pos` (default: the next row), store K and V by
        mode.  krow/vrow: host arrays of n_tokens * n_kv_elems floats."""
        k = np.ascontiguousarray(krow, np.float32).reshape(-1, self.n_kv_elems)
        v = np.ascontiguousarray(vrow, np.float32).reshape(-1, self.n_kv_elems)
        assert k.shape == v.shape
        if pos is None:
            pos = self.n_pos(il, seq)
        self.ctx.check(self.ctx.lib.bk_append_host(self.h, il, seq, pos, k.shape[0], k.ctypes.data, v.ctypes.data))

    def append_device(self, il, k_ptr, v_ptr, n_tokens=1, pos=None, seq=0):
        if pos is None:
            pos = self.n_pos(il, seq)
        self.ctx.check(self.ctx.lib.bk_append(self.h, il, seq, pos, n_tokens, k_ptr, v_ptr))

    def append_batch_device(self, il, k_ptr, v_ptr, n_seqs, seq_ids=None, rope_pos=None):
        sp, _s = _i32_array(seq_ids) or (None, None)
        rp, _r = _i32_array(rope_pos) or (None, None)
        self.ctx.check(self.ctx.lib.bk_append_batch(self.h, il, n_seqs, sp, rp, k_ptr, v_ptr))

    # -- attention ----------------------------------------------------------------
    def decode_device(self, il, q_ptr, out_ptr, n_seqs=1, seq_ids=None, n_pos=None, q_pos=None, partial=False):
        sp, _s = _i32_array(seq_ids) or (None, None)
        np_, _n = _i32_array(n_pos) or (None, None)
        qp, _q = _i32_array(q_pos) or (None, None)
        fn = self.ctx.lib.bk_decode_attn_partial if partial else self.ctx.lib.bk_decode_attn
        self.ctx.check(fn(self.h, il, n_seqs, sp, np_, qp, q_ptr, out_ptr))

    def attend(self, il, q, n_seqs=1, seq_ids=None, n_pos=None, q_pos=None, partial=False):
        """Decode attention for host q [n_seqs, n_head, hd]; returns host out."""
        qa = np.ascontiguousarray(q, np.float32).reshape(n_seqs, self.n_head, self.hd)
        width = self.hd + 2 if partial else self.hd
        dq = self.ctx.to_device(qa)
        do = self.ctx.alloc(n_seqs * self.n_head * width * 4)
        self.decode_device(il, dq.ptr, do.ptr, n_seqs, seq_ids, n_pos, q_pos, partial)
        out = do.download((n_seqs, self.n_head, width), np.float32)
        dq.free()
        do.free()
        return out

    def step(self, il, q, k, v, pos, seq=0):
        """The attention step with the reference's shape: host q/k/v in, host out [n_head, hd]."""
        qa = np.ascontiguousarray(q, np.float32).ravel()
        ka = np.ascontiguousarray(k, np.float32).ravel()
        va = np.ascontiguousarray(v, np.float32).ravel()
        assert qa.size == self.n_head * self.hd and ka.size == self.n_kv_elems and va.size == self.n_kv_elems
        out = np.zeros((self.n_head, self.hd), np.float32)
        self.ctx.check(self.ctx.lib.bk_attn_step_host(self.h, il, seq, pos, qa.ctypes.data, ka.ctypes.data,
                                                      va.ctypes.data, out.ctypes.data))
        return out

    def step_batch_device(self, il, q_ptr, k_ptr, v_ptr, out_ptr, n_seqs, seq_ids=None):
        """One new token for each of n_seqs independent sequences: append + attend (asynchronous)."""
        sp, _s = _i32_array(seq_ids) or (None, None)
        self.ctx.check(self.ctx.lib.bk_attn_step_batch(self.h, il, n_seqs, sp, q_ptr, k_ptr, v_ptr, out_ptr))

    def prefill_attend(self, il, q, pos0, seq=0):
        """Causal attention of a block of prompt tokens already in the cache: host q [n, n_head, hd],
        token i at position pos0 + i; returns [n, n_head, hd]."""
        qa = np.ascontiguousarray(q, np.float32).reshape(-1, self.n_head, self.hd)
        n = qa.shape[0]
        dq = self.ctx.to_device(qa)
        do = self.ctx.alloc(max(n, 1) * self.n_head * self.hd * 4)
        self.ctx.check(self.ctx.lib.bk_prefill_attn(self.h, il, seq, pos0, n, dq.ptr, do.ptr))
        out = do.download((n, self.n_head, self.hd), np.float32)
        dq.free()
        do.free()
        return out

    def prefill_step_device(self, il, q_ptr, k_ptr, v_ptr, out_ptr, pos0, n_tokens, seq=0):
        """Append a block of tokens and attend causally, device pointers (asynchronous)."""
        self.ctx.check(self.ctx.lib.bk_prefill_step(self.h, il, seq, pos0, n_tokens, q_ptr, k_ptr, v_ptr, out_ptr))

    def snapshot(self, seq=0, layout=0):
        """All layers of one sequence as bytes (layout 0: the reference's CPU stores, 1: its device rows)."""
        n = self.ctx.lib.bk_cache_snapshot_bytes(self.h, seq)
        buf = np.zeros(max(n, 1), np.uint8)
        written = C.c_size_t(0)
        self.ctx.check(self.ctx.lib.bk_cache_snapshot_save(self.h, seq, layout, buf.ctypes.data, n, C.byref(written)))
        return buf[:written.value].tobytes()

    def restore(self, blob, seq=0):
        """Load a snapshot taken from a cache of the same mode and head geometry; sets n_pos."""
        buf = np.frombuffer(blob, np.uint8)
        self.ctx.check(self.ctx.lib.bk_cache_snapshot_load(self.h, seq, buf.ctypes.data, buf.size))

    def layer_step(self, il, qfull, kraw, vraw, q_norm_w, k_norm_w, eps, pos, seq=0):
        """The layer form of the step on host arrays: qfull [n_head, 2*hd] ([q | gate] per head),
        kraw/vraw [n_kv, hd], norm weights [hd]; returns attention * sigmoid(gate), [n_head, hd]."""
        qa = np.ascontiguousarray(qfull, np.float32).ravel()
        ka = np.ascontiguousarray(kraw, np.float32).ravel()
        va = np.ascontiguousarray(vraw, np.float32).ravel()
        qw = np.ascontiguousarray(q_norm_w, np.float32).ravel()
        kw = np.ascontiguousarray(k_norm_w, np.float32).ravel()
        assert qa.size == 2 * self.n_head * self.hd and ka.size == self.n_kv_elems and va.size == self.n_kv_elems
        assert qw.size == self.hd and kw.size == self.hd
        out = np.zeros((self.n_head, self.hd), np.float32)
        self.ctx.check(self.ctx.lib.bk_attn_layer_step_host(self.h, il, seq, pos, qa.ctypes.data, ka.ctypes.data,
                                                            va.ctypes.data, qw.ctypes.data, kw.ctypes.data,
                                                            float(eps), out.ctypes.data))
        return out

    def layer_step_device(self, il, qfull_ptr, kraw_ptr, vraw_ptr, q_norm_w_ptr, k_norm_w_ptr, eps, out_ptr, pos, seq=0):
        """The same on device pointers (asynchronous)."""
        self.ctx.check(self.ctx.lib.bk_attn_layer_step(self.h, il, seq, pos, qfull_ptr, kraw_ptr, vraw_ptr,
                                                       q_norm_w_ptr, k_norm_w_ptr, float(eps), out_ptr))

    def step_device(self, il, q_ptr, k_ptr, v_ptr, out_ptr, pos, seq=0):
        """The attention step on device pointers (asynchronous): append at `pos`, attend over pos+1."""
        self.ctx.check(self.ctx.lib.bk_attn_step(self.h, il, seq, pos, q_ptr, k_ptr, v_ptr, out_ptr))

    # -- dump_kv (src/gdev.rs:1433-1445) ---------------------------------------------
    def dump_kv(self, il, n_pos=None, seq=0, pos0=0):
        """Rows [pos0, pos0+n_pos) as the reference's CPU cache lays them out."""
        if n_pos is None:
            n_pos = self.n_pos(il, seq) - pos0
        n, nkv, hd = n_pos, self.n_kv, self.hd
        m = self.mode
        out = {}
        if m.kind == "planar":
            plen = 32 * m.bits
            out["kq"] = np.zeros((n, nkv, plen), np.uint8)
            out["kn"] = np.zeros((n, nkv), np.float32)
            if m.v_quant:
                out["vq"] = np.zeros((n, nkv, plen), np.uint8)
                out["vn"] = np.zeros((n, nkv), np.float32)
                args = (out["kq"], out["kn"], out["vq"], out["vn"])
            else:
                out["v"] = np.zeros((n, nkv, hd), np.float32)
                args = (out["kq"], out["kn"], out["v"], None)
        elif m.kind == "f16":
            out["k16"] = np.zeros((n, nkv, hd), np.uint16)
            out["v16"] = np.zeros((n, nkv, hd), np.uint16)
            args = (out["k16"], None, out["v16"], None)
        else:
            out["k"] = np.zeros((n, nkv, hd), np.float32)
            out["v"] = np.zeros((n, nkv, hd), np.float32)
            args = (out["k"], None, out["v"], None)
        ptrs = [a.ctypes.data if a is not None else None for a in args]
        self.ctx.check(self.ctx.lib.bk_cache_download(self.h, il, seq, pos0, n, *ptrs))
        return out

    def upload_kv(self, il, rows, seq=0, pos0=0):
        """Inverse of dump_kv (snapshot restore); `rows` is a dict as dump_kv returns."""
        m = self.mode
        if m.kind == "planar":
            args = (rows["kq"], rows["kn"], rows["vq"] if m.v_quant else rows["v"], rows["vn"] if m.v_quant else None)
        elif m.kind == "f16":
            args = (rows["k16"], None, rows["v16"], None)
        else:
            args = (rows["k"], None, rows["v"], None)
        arrs = [np.ascontiguousarray(a) if a is not None else None for a in args]
        n = arrs[0].shape[0]
        ptrs = [a.ctypes.data if a is not None else None for a in arrs]
        self.ctx.check(self.ctx.lib.bk_cache_upload(self.h, il, seq, pos0, n, *ptrs))


def full_attention_step(cache, il, q, k, v, pos, seq=0):
    """src/forward.rs:247-375: q [n_head*hd] and k [n_kv*hd] RMS-normed, v raw; returns the
    pre-gate attention output [n_head, hd]."""
    return cache.step(il, q, k, v, pos, seq)


def full_attention_layer_core(cache, il, qfull, kraw, vraw, q_norm_w, k_norm_w, eps, pos, seq=0):
    """src/forward.rs:237-382 without the matvecs: split [q | gate], per-head RMSNorm of q and k,
    both ropes, the cache append, GQA attention and the sigmoid gate.  Returns the input of the
    output projection, [n_head, hd]."""
    return cache.layer_step(il, qfull, kraw, vraw, q_norm_w, k_norm_w, eps, pos, seq)


def rms_norm_rows(x, w, row_len, eps, ctx=None):
    """src/kernels.rs:97-122; raises like the reference on a bad weight length or a ragged x."""
    from .kvquant import default_context
    c = ctx or default_context()
    xa = np.ascontiguousarray(x, np.float32).ravel()
    wa = np.ascontiguousarray(w, np.float32).ravel()
    if wa.size != row_len:
        raise _abi.BonsaiKvError(_abi.BK_ERR_INVALID, f"rms_norm_rows: weight len {wa.size} != row_len {row_len}")
    if xa.size % row_len != 0:
        raise _abi.BonsaiKvError(_abi.BK_ERR_INVALID, f"rms_norm_rows: x len {xa.size} not divisible by row_len {row_len}")
    out = np.zeros_like(xa)
    c.check(c.lib.bk_rms_norm_rows(c.h, xa.size // row_len, row_len, xa.ctypes.data, wa.ctypes.data, float(eps),
                                   out.ctypes.data))
    return out


def attn_step(ctx, q, kcache, vcache, n_pos, nheads, kvheads, hd):
    """Gpu::attn_step, src/vk.rs:1671-1752: one-shot f32 attention over host caches."""
    q = np.ascontiguousarray(q, np.float32)
    kc = np.ascontiguousarray(kcache, np.float32)
    vc = np.ascontiguousarray(vcache, np.float32)
    kv_stride = kvheads * hd
    if q.size != nheads * hd or kc.size != n_pos * kv_stride or vc.size != n_pos * kv_stride or hd > 256:
        raise _abi.BonsaiKvError(_abi.BK_ERR_INVALID,
                                 f"attn_step: q {q.size} ({nheads}x{hd}), k/v {kc.size} ({n_pos} pos x {kv_stride})")
    out = np.zeros((nheads, hd), np.float32)
    ctx.check(ctx.lib.bk_attn_oneshot_host(ctx.h, q.ctypes.data, kc.ctypes.data, vc.ctypes.data, n_pos, nheads,
                                           kvheads, hd, out.ctypes.data))
    return out
