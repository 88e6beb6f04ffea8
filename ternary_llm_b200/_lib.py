"""ctypes binding of libtllm_b200.so (the C ABI in include/tllm_b200.h).

There is no fallback: if the shared library is missing or a call fails, an
exception is raised.
"""
from __future__ import annotations

import ctypes
import os

PKG = os.path.dirname(os.path.abspath(__file__))
# TLLM_B200_LIB names another build of the library to load (the diagnostic one, see build.py)
LIB_PATH = os.environ.get("TLLM_B200_LIB") or os.path.join(PKG, "libtllm_b200.so")

_vp = ctypes.c_void_p
_int = ctypes.c_int

# name -> (restype, argtypes); must list every symbol the headers under include/ declare
SIGNATURES = {
    "tllm_b200_status_string": (ctypes.c_char_p, [_int]),
    "tllm_b200_last_error": (ctypes.c_char_p, []),
    "tllm_b200_version": (_int, []),
    "tllm_b200_gemv": (_int, [_vp] * 5 + [_int] * 3 + [_vp]),
    "tllm_b200_gemv_batched": (_int, [_vp] * 5 + [_int] * 4 + [_vp]),
    "tllm_b200_gemv_int8": (_int, [_vp] * 4 + [ctypes.c_float, _vp] + [_int] * 3 + [_vp]),
    "tllm_b200_quantize_absmax_int8": (_int, [_vp] * 3 + [_int, _vp]),
    "tllm_b200_gemm": (_int, [_vp] * 5 + [_int] * 4 + [_vp]),
    "tllm_b200_packed_bytes": (ctypes.c_size_t, [_int, _int]),
    "tllm_b200_weight_prepare": (_int, [_vp] * 3 + [_int] * 3 + [_vp, ctypes.c_size_t, _vp]),
    "tllm_b200_weight_unpack": (_int, [_vp] + [_int] * 3 + [_vp] * 4),
    "tllm_b200_weight_register": (_int, [_vp, _vp, _int, _int]),
    "tllm_b200_weight_unregister": (_int, [_vp]),
    "tllm_b200_gemv_packed": (_int, [_vp] * 3 + [_int] * 3 + [_vp]),
    "tllm_b200_gemv_int8_packed": (_int, [_vp, _vp, ctypes.c_float, _vp, _int, _int, _vp]),
    "tllm_b200_check_device_errors": (_int, [_vp]),
    "tllm_b200_gemm_packed": (_int, [_vp] * 3 + [_int] * 3 + [_vp]),
    "tllm_b200_gemv_packed_noalloc": (_int, [_vp] * 3 + [_int] * 2 + [_vp]),
    "tllm_b200_gemv_packed_noalloc_status": (_int, [_vp]),
    "tllm_b200_gemv_packed_allreduce": (_int, [_vp] * 3 + [_int] * 4 + [_vp] * 2 + [_int, _vp]),
    "tllm_b200_allreduce_trace": (_int, [_vp, _int]),
    "tllm_b200_gemv_packed_multi": (_int, [_int, _vp, _vp, _vp, _int, _vp, _vp]),
    "tllm_b200_gemv_packed_multi_norm": (_int, [_int, _vp, _vp, _vp, _int, _vp, _vp, _vp, _vp, ctypes.c_float, _vp]),
    # include/tllm_b200_layer.h
    "tllm_b200_rmsnorm": (_int, [_vp] * 5 + [_int, _int, ctypes.c_float, _vp]),
    "tllm_b200_rope": (_int, [_vp, _vp] + [_int] * 6 + [ctypes.c_float, _vp]),
    "tllm_b200_copy_to_kv_cache": (_int, [_vp] * 4 + [_int] * 6 + [_vp]),
    "tllm_b200_rope_append": (_int, [_vp] * 5 + [_int] * 6 + [ctypes.c_float, _int, _vp]),
    "tllm_b200_attention": (_int, [_vp] * 4 + [_int] * 7 + [_vp]),
    "tllm_b200_attention_decode": (_int, [_vp] * 6 + [_int] * 4 + [ctypes.c_float, _int, _vp]),
    "tllm_b200_silu_mul": (_int, [_vp] * 3 + [_int, _vp]),
    "tllm_b200_add": (_int, [_vp] * 3 + [_int, _vp]),
    "tllm_b200_embedding_lookup": (_int, [_vp] * 3 + [_int, _int, _vp]),
    "tllm_b200_fp16_gemv": (_int, [_vp] * 3 + [_int, _int, _vp]),
    "tllm_b200_fp16_gemm": (_int, [_vp] * 3 + [_int] * 3 + [_vp]),
    "tllm_b200_gemv_int8_packed_multi": (_int, [_int, _vp, _vp, _vp, _int, _vp, _vp, _vp]),
    "tllm_b200_decoder_create": (_int, [_vp, _int, _vp]),
    "tllm_b200_decoder_create_batched": (_int, [_vp, _int, _int, _vp]),
    "tllm_b200_decoder_destroy": (None, [_vp]),
    "tllm_b200_decoder_forward_seq": (_int, [_vp, _int, _vp, _int, _int, _vp, _vp]),
    "tllm_b200_decoder_forward_batch": (_int, [_vp, _vp, _int, _int, _vp, _vp]),
    "tllm_b200_decoder_reset": (_int, [_vp, _vp]),
    "tllm_b200_decoder_forward": (_int, [_vp, _vp, _int, _int, _vp, _vp]),
    "tllm_b200_decoder_generate": (_int, [_vp, _int, _int, _int, _vp, _vp]),
}


class TernaryWeightDesc(ctypes.Structure):
    """tllm_b200_ternary_weight (include/tllm_b200_layer.h)."""
    _fields_ = [("nonzero_masks", _vp), ("sign_masks", _vp), ("scales", _vp),
                ("out_features", _int), ("in_features", _int)]


class LayerWeightsDesc(ctypes.Structure):
    """tllm_b200_layer_weights."""
    _fields_ = [(n, TernaryWeightDesc) for n in
                ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")] + \
               [("attn_norm_weight", _vp), ("ffn_norm_weight", _vp)]


class ModelDesc(ctypes.Structure):
    """tllm_b200_model_desc."""
    _fields_ = [(n, _int) for n in ("vocab_size", "hidden_dim", "intermediate_dim", "n_layers", "n_heads",
                                    "n_kv_heads", "max_seq_len", "head_dim", "group_size")] + \
               [("rope_theta", ctypes.c_float), ("rms_norm_eps", ctypes.c_float),
                ("embedding_table", _vp), ("final_norm_weight", _vp), ("lm_head_weight", _vp),
                ("lm_head_ternary", TernaryWeightDesc), ("layers", ctypes.POINTER(LayerWeightsDesc))]


class TllmError(RuntimeError):
    def __init__(self, status: int, text: str, detail: str):
        super().__init__(f"tllm_b200 status {status} ({text}): {detail}")
        self.status = status


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m ternary_llm_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != 0:
        h = lib()
        raise TllmError(status, h.tllm_b200_status_string(status).decode(),
                        h.tllm_b200_last_error().decode())
