"""Context and device-buffer helpers over the C ABI (no torch, no CUDA binding needed)."""
import ctypes as C

import numpy as np

from . import _abi


class Context:
    """One CUDA stream on one device; not thread-safe, like the reference's single decode thread."""

    def __init__(self, device=0):
        self.lib = _abi.load()
        h = C.c_void_p()
        _abi.check(self.lib.bk_ctx_create(device, C.byref(h)))
        self.h = h
        self.device = device

    def close(self):
        if getattr(self, "h", None):
            self.lib.bk_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, status):
        _abi.check(status, self.h)

    def synchronize(self):
        self.check(self.lib.bk_synchronize(self.h))

    @property
    def stream(self):
        return self.lib.bk_ctx_stream(self.h)

    @property
    def launch_count(self):
        return int(self.lib.bk_ctx_launch_count(self.h))

    # -- memory -------------------------------------------------------------
    def alloc(self, nbytes):
        return DeviceBuffer(self, int(nbytes))

    def to_device(self, array):
        a = np.ascontiguousarray(array)
        buf = self.alloc(max(a.nbytes, 1))
        buf.upload(a)
        return buf

    def pinned(self, shape, dtype):
        return PinnedArray(self, shape, dtype)

    # -- timing ---------------------------------------------------------------
    def event(self):
        return Event(self)


class DeviceBuffer:
    def __init__(self, ctx, nbytes):
        self.ctx, self.nbytes = ctx, nbytes
        p = C.c_void_p()
        ctx.check(ctx.lib.bk_dev_alloc(ctx.h, nbytes, C.byref(p)))
        self.ptr = p.value

    def free(self):
        if getattr(self, "ptr", None) and self.ctx.h:
            self.ctx.lib.bk_dev_free(self.ctx.h, self.ptr)
        self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def offset(self, nbytes):
        return self.ptr + int(nbytes)

    def upload(self, array, sync=True):
        a = np.ascontiguousarray(array)
        assert a.nbytes <= self.nbytes
        self.ctx.check(self.ctx.lib.bk_memcpy_h2d(self.ctx.h, self.ptr, a.ctypes.data, a.nbytes))
        if sync:
            self.ctx.synchronize()

    def download(self, shape, dtype):
        out = np.empty(shape, dtype=dtype)
        assert out.nbytes <= self.nbytes
        self.ctx.check(self.ctx.lib.bk_memcpy_d2h(self.ctx.h, out.ctypes.data, self.ptr, out.nbytes))
        self.ctx.synchronize()
        return out

    def zero(self):
        self.ctx.check(self.ctx.lib.bk_memset_dev(self.ctx.h, self.ptr, 0, self.nbytes))


class PinnedArray:
    """A numpy view over page-locked host memory (for asynchronous copies)."""

    def __init__(self, ctx, shape, dtype):
        self.ctx = ctx
        dt = np.dtype(dtype)
        n = int(np.prod(shape)) * dt.itemsize
        p = C.c_void_p()
        ctx.check(ctx.lib.bk_host_alloc_pinned(ctx.h, max(n, 1), C.byref(p)))
        self.ptr = p.value
        buf = (C.c_char * max(n, 1)).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=dt, count=int(np.prod(shape))).reshape(shape)
        self.nbytes = n

    def free(self):
        if getattr(self, "ptr", None) and self.ctx.h:
            self.array = None
            self.ctx.lib.bk_host_free_pinned(self.ctx.h, self.ptr)
        self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Event:
    def __init__(self, ctx):
        self.ctx = ctx
        p = C.c_void_p()
        ctx.check(ctx.lib.bk_event_create(ctx.h, C.byref(p)))
        self.h = p

    def record(self):
        self.ctx.check(self.ctx.lib.bk_event_record(self.ctx.h, self.h))

    def elapsed_ms(self, stop):
        ms = C.c_float()
        self.ctx.check(self.ctx.lib.bk_event_elapsed_ms(self.ctx.h, self.h, stop.h, C.byref(ms)))
        return ms.value

    def __del__(self):
        try:
            if getattr(self, "h", None):
                self.ctx.lib.bk_event_destroy(self.h)
                self.h = None
        except Exception:
            pass
