"""B200-native KV-cache path of herlangga72/ternary-bonsai-inference.

The package is a thin host-side mirror of the reference's interfaces for this
path (`kvquant`, the `AttnCache` / attention step of `forward`) over the C ABI of
libbonsai_kv.so (include/bonsai_kv.h).  The directory name contains '-', so
import it with importlib:

    import importlib
    bk = importlib.import_module("ternary-bonsai-inference_b200")
"""
from . import _abi
from ._abi import BonsaiKvError
from .device import Context, DeviceBuffer, Event, PinnedArray
from .forward import (AttnCache, attn_step, full_attention_layer_core, full_attention_step, n_ctx_env,
                      rms_norm_rows)
from .kvquant import (DEFAULT_HD, F16, F32, KvMode, Planar, PlanarQuant, codebook, f32_to_half,
                      givens_table, half_to_f32, mode_from_env, packed_bytes, parse_mode,
                      quantizers_for, rope_imrope)
from .pq2 import Pq2Tensor, pack_pq2, pq2_matvec_multi_device, pq2_row_bytes

__all__ = ["AttnCache", "BonsaiKvError", "Context", "DEFAULT_HD", "DeviceBuffer", "Event", "F16", "F32",
           "KvMode", "PinnedArray", "Planar", "PlanarQuant", "Pq2Tensor", "pack_pq2", "pq2_matvec_multi_device", "pq2_row_bytes", "attn_step", "codebook", "f32_to_half",
           "full_attention_layer_core", "full_attention_step", "givens_table", "half_to_f32", "mode_from_env", "n_ctx_env", "rms_norm_rows",
           "packed_bytes", "parse_mode", "quantizers_for", "rope_imrope"]


def library_path():
    return _abi.LIB_PATH
