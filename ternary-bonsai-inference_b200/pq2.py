"""PQ2_0 ternary weight rows on the device: the matvec either side of the attention path.

Mirrors src/kernels.rs:204-420 (`pq2_row_bytes`, `pq2_matvec_range`, `pq2_matmul_n`): a tensor
is its GGUF payload, rows back to back, each row ceil(ne0 / 128) blocks of 34 bytes (f16 scale +
128 two-bit codes, weight = (code - 1) * scale).  The payload is uploaded once and stays in
device memory; every product streams it once per group of four activations.
"""
import ctypes as C

import numpy as np

from . import _abi

QK = 128
BLOCK_BYTES = 34


def pq2_row_bytes(ne0):
    """src/kernels.rs:208-211."""
    return -(-int(ne0) // QK) * BLOCK_BYTES


def pack_pq2(codes, scales):
    """Rows of two-bit codes [n_rows, ne0] (0..3) and f16 block scales [n_rows, ceil(ne0 / 128)]
    -> payload bytes in the row format above (codes past ne0 in the last block are zero)."""
    codes = np.ascontiguousarray(codes, np.uint8)
    n_rows, ne0 = codes.shape
    nb = -(-ne0 // QK)
    sc = np.ascontiguousarray(scales, np.float16).reshape(n_rows, nb)
    padded = np.zeros((n_rows, nb * QK), np.uint8)
    padded[:, :ne0] = codes & 3
    quad = padded.reshape(n_rows, nb, QK // 4, 4)
    qs = (quad[..., 0] | (quad[..., 1] << 2) | (quad[..., 2] << 4) | (quad[..., 3] << 6)).astype(np.uint8)
    out = np.zeros((n_rows, nb, BLOCK_BYTES), np.uint8)
    out[..., :2] = sc.view(np.uint8).reshape(n_rows, nb, 2)
    out[..., 2:] = qs
    return out.reshape(-1)


class _Seg(C.Structure):
    _fields_ = [("payload_dev", C.c_void_p), ("payload_bytes", C.c_size_t), ("base_row", C.c_int64), ("n_rows", C.c_int64),
                ("y_dev", C.c_void_p)]


def pq2_matvec_multi_device(ctx, tensors, x_ptr, y_ptrs, n_tok=1):
    """Up to four tensors with the same ne0 against one x in one launch (the q, k and v projections
    of a layer); y_ptrs[i] receives [n_tok, tensors[i].n_rows].  Asynchronous, device pointers."""
    segs = (_Seg * len(tensors))()
    for sg, t, yp in zip(segs, tensors, y_ptrs):
        sg.payload_dev, sg.payload_bytes, sg.base_row, sg.n_rows, sg.y_dev = t.buf.ptr, t.payload_bytes, 0, t.n_rows, yp
    ctx.check(ctx.lib.bk_pq2_matvec_multi(ctx.h, len(tensors), C.cast(segs, C.c_void_p), tensors[0].ne0, x_ptr, n_tok))


class Pq2Tensor:
    """A PQ2_0 tensor resident in device memory."""

    def __init__(self, ctx, payload, ne0):
        self.ctx = ctx
        self.ne0 = int(ne0)
        pl = np.ascontiguousarray(payload, np.uint8).ravel()
        self.payload_bytes = int(pl.size)
        self.row_bytes = pq2_row_bytes(ne0)
        self.n_rows = self.payload_bytes // self.row_bytes
        self.buf = ctx.to_device(pl if pl.size else np.zeros(1, np.uint8))

    def free(self):
        if self.buf is not None:
            self.buf.free()
            self.buf = None

    def matmul_n(self, x, n_tok, base_row=0, n_rows=None):
        """pq2_matmul_n (src/kernels.rs:340-420): host x [n_tok, ne0] -> y [n_tok, n_rows]."""
        n_rows = self.n_rows - base_row if n_rows is None else n_rows
        xa = np.ascontiguousarray(x, np.float32).ravel()
        if xa.size != n_tok * self.ne0:
            raise _abi.BonsaiKvError(_abi.BK_ERR_INVALID, f"pq2_matmul_n: x length {xa.size} != n_tok {n_tok} * ne0 {self.ne0}")
        y = np.zeros((n_tok, n_rows), np.float32)
        self.ctx.check(self.ctx.lib.bk_pq2_matvec_host(self.ctx.h, self.buf.ptr, self.payload_bytes, self.ne0, base_row, n_rows,
                                                       xa.ctypes.data, n_tok, y.ctypes.data))
        return y

    def matvec(self, x, base_row=0, n_rows=None):
        """pq2_matvec_range (src/kernels.rs:274-330): host x [ne0] -> y [n_rows]."""
        xa = np.ascontiguousarray(x, np.float32).ravel()
        if xa.size != self.ne0:
            raise _abi.BonsaiKvError(_abi.BK_ERR_INVALID, f"pq2_matvec_range: x length {xa.size} != ne0 {self.ne0}")
        return self.matmul_n(xa, 1, base_row, n_rows)[0]

    def matvec_device(self, x_ptr, y_ptr, n_tok=1, base_row=0, n_rows=None):
        """Device pointers, asynchronous on the context's stream."""
        n_rows = self.n_rows - base_row if n_rows is None else n_rows
        self.ctx.check(self.ctx.lib.bk_pq2_matvec(self.ctx.h, self.buf.ptr, self.payload_bytes, self.ne0, base_row, n_rows,
                                                  x_ptr, n_tok, y_ptr))
