"""ternary_llm_b200: B200-native ternary weight contraction (decode GEMV, prefill
GEMM) behind the operator interface of jastaq/ternary-llm.

The compute lives in libtllm_b200.so (hand-written sm_100a CUDA behind the C ABI
of include/tllm_b200.h and include/tllm_b200_layer.h); this package is the thin host
side: ops (the contraction), layer_ops (the operators either side of it inside a
decoder layer) and Decoder (the reference's Transformer on both).
"""
from . import pack  # noqa: F401
from ._lib import LIB_PATH, TllmError, lib  # noqa: F401
from .ops import (GROUP_SIZE, MAX_BATCH, FusedAllReduce, PreparedWeight, ternary_gemv_packed_allreduce, check_device_errors, packed_bytes, quantize_absmax_int8,  # noqa: F401
                  ternary_gemm, ternary_gemm_packed, ternary_gemv, ternary_gemv_batched, ternary_gemv_int8,
                  ternary_gemv_int8_packed, ternary_gemv_packed, ternary_gemv_packed_multi,
                  ternary_gemv_packed_multi_norm, prepare_group)

from . import layer_ops  # noqa: F401,E402
from .decoder import Decoder  # noqa: F401,E402

__all__ = ["layer_ops", "Decoder", "prepare_group", "pack", "lib", "TllmError", "LIB_PATH", "GROUP_SIZE", "MAX_BATCH", "ternary_gemv",
           "ternary_gemv_batched", "ternary_gemv_int8", "quantize_absmax_int8", "ternary_gemm",
           "PreparedWeight", "FusedAllReduce", "ternary_gemv_packed_allreduce", "ternary_gemm_packed", "check_device_errors", "packed_bytes", "ternary_gemv_packed", "ternary_gemv_int8_packed", "ternary_gemv_packed_multi", "ternary_gemv_packed_multi_norm"]
