"""ctypes declarations for every entry point of include/bonsai_kv.h.

The shared library is required: there is no Python or CPU fallback.  If
libbonsai_kv.so is missing the import fails with instructions to build it.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libbonsai_kv.so")

BK_OK, BK_ERR_INVALID, BK_ERR_CUDA, BK_ERR_OOM, BK_ERR_RANGE, BK_ERR_UNSUPPORTED = range(6)
BK_MODE_F32, BK_MODE_F16, BK_MODE_PLANAR = 0, 1, 2


class KvModeStruct(C.Structure):
    _fields_ = [("kind", C.c_int32), ("bits", C.c_int32), ("v_quant", C.c_int32)]


class CacheConfig(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("n_seqs", C.c_int32), ("n_ctx", C.c_int32),
                ("n_head", C.c_int32), ("n_kv", C.c_int32), ("hd", C.c_int32), ("n_rot", C.c_int32),
                ("sections", C.c_int32 * 4), ("freq_base", C.c_float), ("rope_positions", C.c_int32),
                ("mode", KvModeStruct)]


_vp, _i32, _i64, _sz, _f = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t, C.c_float
_pi32 = C.POINTER(C.c_int32)
_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); the order follows include/bonsai_kv.h
SIGNATURES = {
    "bk_version": (C.c_char_p, []),
    "bk_status_string": (C.c_char_p, [C.c_int]),
    "bk_ctx_create": (C.c_int, [C.c_int, _pp]),
    "bk_ctx_destroy": (None, [_vp]),
    "bk_last_error": (C.c_char_p, [_vp]),
    "bk_synchronize": (C.c_int, [_vp]),
    "bk_ctx_stream": (_vp, [_vp]),
    "bk_ctx_device": (C.c_int, [_vp]),
    "bk_parse_mode": (C.c_int, [C.c_char_p, C.POINTER(KvModeStruct)]),
    "bk_mode_from_env": (C.c_int, [C.POINTER(KvModeStruct)]),
    "bk_n_ctx_from_env": (_i32, []),
    "bk_default_config": (None, [C.POINTER(CacheConfig)]),
    "bk_cache_create": (C.c_int, [_vp, C.POINTER(CacheConfig), _pp]),
    "bk_cache_destroy": (None, [_vp]),
    "bk_cache_reset": (C.c_int, [_vp, _i32]),
    "bk_cache_n_pos": (_i32, [_vp, _i32, _i32]),
    "bk_cache_set_n_pos": (C.c_int, [_vp, _i32, _i32, _i32]),
    "bk_cache_get_config": (C.c_int, [_vp, C.POINTER(CacheConfig)]),
    "bk_cache_row_bytes": (_i32, [_vp, _i32]),
    "bk_cache_device_bytes": (_sz, [_vp]),
    "bk_cache_download": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "bk_cache_upload": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "bk_append": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _vp, _vp]),
    "bk_append_host": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _vp, _vp]),
    "bk_append_batch": (C.c_int, [_vp, _i32, _i32, _pi32, _pi32, _vp, _vp]),
    "bk_decode_attn": (C.c_int, [_vp, _i32, _i32, _pi32, _pi32, _pi32, _vp, _vp]),
    "bk_decode_attn_partial": (C.c_int, [_vp, _i32, _i32, _pi32, _pi32, _pi32, _vp, _vp]),
    "bk_decode_attn_noalloc": (C.c_int, [_vp, _i32, _i32, _pi32, _pi32, _pi32, _vp, _vp]),
    "bk_lse_merge": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp]),
    "bk_mailbox_create": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _pp, _vp]),
    "bk_mailbox_open_peers": (C.c_int, [_vp, _vp]),
    "bk_mailbox_destroy": (None, [_vp]),
    "bk_exchange_merge": (C.c_int, [_vp, _i32, _vp, _vp, C.c_uint32]),
    "bk_decode_attn_split": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, C.c_uint32]),
    "bk_attn_step": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "bk_attn_step_host": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "bk_cache_snapshot_bytes": (_sz, [_vp, _i32]),
    "bk_cache_snapshot_save": (C.c_int, [_vp, _i32, _i32, _vp, _sz, _vp]),
    "bk_cache_snapshot_load": (C.c_int, [_vp, _i32, _vp, _sz]),
    "bk_attn_step_batch": (C.c_int, [_vp, _i32, _i32, _pi32, _vp, _vp, _vp, _vp]),
    "bk_prefill_attn": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _vp, _vp]),
    "bk_prefill_step": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "bk_attn_step_split": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, C.c_uint32]),
    "bk_attn_layer_step": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _f, _vp]),
    "bk_attn_layer_step_host": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _f, _vp]),
    "bk_rms_norm_rows": (C.c_int, [_vp, _i32, _i32, _vp, _vp, _f, _vp]),
    "bk_pq2_row_bytes": (_sz, [_i64]),
    "bk_pq2_matvec": (C.c_int, [_vp, _vp, _sz, _i64, _i64, _i64, _vp, _i32, _vp]),
    "bk_pq2_matvec_multi": (C.c_int, [_vp, _i32, _vp, _i64, _vp, _i32]),
    "bk_pq2_matvec_host": (C.c_int, [_vp, _vp, _sz, _i64, _i64, _i64, _vp, _i32, _vp]),
    "bk_attn_oneshot_host": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "bk_kvq_packed_len": (_sz, [_i32, _i32]),
    "bk_kvq_codebook": (C.c_int, [_i32, _i32, _vp]),
    "bk_kvq_givens": (C.c_int, [_i32, _vp]),
    "bk_kvq_threshold_cells": (C.c_int, [_i32, _vp]),
    "bk_kvq_quantize": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp, _vp]),
    "bk_kvq_dequantize": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp, _vp]),
    "bk_kvq_rotate": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp]),
    "bk_kvq_dot_rotated": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "bk_rope_imrope": (C.c_int, [_vp, _i32, _i32, _vp, _i64, _i64, _i64, _i64, _i32, _pi32, _f]),
    "bk_f32_to_half": (C.c_int, [_vp, _sz, _vp, _vp]),
    "bk_half_to_f32": (C.c_int, [_vp, _sz, _vp, _vp]),
    "bk_dev_alloc": (C.c_int, [_vp, _sz, _pp]),
    "bk_dev_free": (C.c_int, [_vp, _vp]),
    "bk_host_alloc_pinned": (C.c_int, [_vp, _sz, _pp]),
    "bk_host_free_pinned": (C.c_int, [_vp, _vp]),
    "bk_memcpy_h2d": (C.c_int, [_vp, _vp, _vp, _sz]),
    "bk_memcpy_d2h": (C.c_int, [_vp, _vp, _vp, _sz]),
    "bk_memset_dev": (C.c_int, [_vp, _vp, C.c_int, _sz]),
    "bk_event_create": (C.c_int, [_vp, _pp]),
    "bk_event_destroy": (None, [_vp]),
    "bk_event_record": (C.c_int, [_vp, _vp]),
    "bk_event_elapsed_ms": (C.c_int, [_vp, _vp, _vp, C.POINTER(C.c_float)]),
    "bk_ctx_launch_count": (C.c_uint64, [_vp]),
}

_lib = None


def load():
    """Load libbonsai_kv.so and attach the signatures (once)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python {os.path.join(HERE, 'build.py')}` "
            "(needs nvcc; there is no CPU fallback for this path)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


class BonsaiKvError(RuntimeError):
    """A bk_status other than BK_OK; `.status` holds the code (Result::Err in the reference)."""

    def __init__(self, status, text):
        super().__init__(text)
        self.status = status


def check(status, ctx_handle=None):
    if status == BK_OK:
        return
    lib = load()
    text = lib.bk_last_error(ctx_handle) or b""
    name = lib.bk_status_string(status).decode()
    raise BonsaiKvError(status, f"{name}: {text.decode(errors='replace')}")
