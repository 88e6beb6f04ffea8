"""ctypes bindings for the checker libraries (TEST INFRASTRUCTURE ONLY).

  liboracle_cpu.so   oracle/cpu_reference.c, this repository's C restatement of
                     the reference's scalar matvec
  _ref/libref.so     the reference project's own sources compiled unmodified
                     (oracle/Makefile target `ref`); optional

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import
this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# Where a checkout of the reference project is looked for (optional; only build steps use
# it): the directory named by TLLM_REFERENCE_DIR, else a directory `reference` beside this
# repository's own directory.
REF_DIR = os.environ.get("TLLM_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
_PORT = os.path.join(_HERE, "liboracle_cpu.so")
_REF = os.path.join(_HERE, "_ref", "libref.so")

_u32p = ctypes.POINTER(ctypes.c_uint32)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_f32p = ctypes.POINTER(ctypes.c_float)
_i8p = ctypes.POINTER(ctypes.c_int8)


def build(ref_dir: str | None = REF_DIR) -> None:
    """Compile the C restatement, and the reference's own sources when they are
    present on this machine."""
    subprocess.check_call(["make", "-s", "-C", _HERE])
    if ref_dir and os.path.isdir(ref_dir):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", f"REF={ref_dir}"])
        pkg_lib = os.path.join(os.path.dirname(_HERE), "ternary_llm_b200", "libtllm_b200.so")
        if os.path.exists(pkg_lib):      # drop-in checks link against the built library
            subprocess.check_call(["make", "-s", "-C", _HERE, "dropin", f"REF={ref_dir}"])


DROPIN_TEST = os.path.join(_HERE, "_ref", "test_gemv_dropin")
ENGINE_LINK = os.path.join(_HERE, "_ref", "engine_link")


_port = None
_ref = None


def port():
    global _port
    if _port is None:
        if not os.path.exists(_PORT):
            build(None)
        lib = ctypes.CDLL(_PORT)
        lib.oracle_matvec_f32.argtypes = [_u32p, _u32p, _f32p, _f32p, _f32p] + [ctypes.c_int] * 3
        lib.oracle_matvec_f32_mt.argtypes = [_u32p, _u32p, _f32p, _f32p, _f32p] + [ctypes.c_int] * 4
        lib.oracle_matvec_f16.argtypes = [_u32p, _u32p, _u16p, _u16p, _f32p] + [ctypes.c_int] * 5
        lib.oracle_matvec_i8.argtypes = [_u32p, _u32p, _u16p, _i8p, ctypes.c_float, _f32p] + [ctypes.c_int] * 4
        lib.oracle_num_threads.restype = ctypes.c_int
        _port = lib
    return _port


def have_ref() -> bool:
    return os.path.exists(_REF)


def ref():
    """The reference's compiled sources; raises if oracle/_ref was not built."""
    global _ref
    if _ref is None:
        lib = ctypes.CDLL(_REF)
        lib.ref_cpu_reference.argtypes = [_u32p, _u32p, _f32p, _f32p, _f32p] + [ctypes.c_int] * 3
        vp = ctypes.c_void_p
        lib.ref_ternary_gemv.argtypes = [vp] * 5 + [ctypes.c_int] * 3 + [vp]
        lib.ref_ternary_gemv_int8.argtypes = [vp] * 4 + [ctypes.c_float, vp] + [ctypes.c_int] * 3 + [vp]
        lib.ref_quantize_absmax_int8.argtypes = [vp] * 3 + [ctypes.c_int, vp]
        lib.ref_ternary_gemm.argtypes = [vp] * 5 + [ctypes.c_int] * 4 + [vp]
        i, f = ctypes.c_int, ctypes.c_float
        lib.ref_rmsnorm_forward.argtypes = [vp] * 5 + [i, i, f, vp]
        lib.ref_rope_forward.argtypes = [vp, vp] + [i] * 6 + [f, vp]
        lib.ref_attention_forward.argtypes = [vp] * 4 + [i] * 7 + [vp]
        lib.ref_silu_mul_forward.argtypes = [vp] * 3 + [i, vp]
        lib.ref_add_forward.argtypes = [vp] * 3 + [i, vp]
        lib.ref_embedding_lookup.argtypes = [vp] * 3 + [i, i, vp]
        lib.ref_copy_to_kv_cache.argtypes = [vp] * 4 + [i] * 6 + [vp]
        lib.ref_fp16_gemv.argtypes = [vp] * 3 + [i, i, vp]
        lib.ref_fp16_gemm.argtypes = [vp] * 3 + [i] * 3 + [vp]
        _ref = lib
    return _ref


def _p(a, t):
    return a.ctypes.data_as(t)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def matvec_f32(nz, sg, scales_f32, x_f32, group_size=128, threads=1, use_ref=False):
    """Scalar float32 matvec on float scales/inputs (the reference signature).
    use_ref=True calls the reference's compiled cpu_reference itself."""
    nz, sg = _c(nz, np.uint32), _c(sg, np.uint32)
    s, x = _c(scales_f32, np.float32), _c(x_f32, np.float32)
    rows, cols = nz.shape[0], nz.shape[1] * 32
    y = np.empty(rows, np.float32)
    if use_ref:
        if threads == 1:
            ref().ref_cpu_reference(_p(nz, _u32p), _p(sg, _u32p), _p(s, _f32p), _p(x, _f32p),
                                    _p(y, _f32p), rows, cols, group_size)
        else:
            _ref_threaded(nz, sg, s, x, y, rows, cols, group_size, threads)
    elif threads == 1:
        port().oracle_matvec_f32(_p(nz, _u32p), _p(sg, _u32p), _p(s, _f32p), _p(x, _f32p),
                                 _p(y, _f32p), rows, cols, group_size)
    else:
        port().oracle_matvec_f32_mt(_p(nz, _u32p), _p(sg, _u32p), _p(s, _f32p), _p(x, _f32p),
                                    _p(y, _f32p), rows, cols, group_size, threads)
    return y


def _ref_threaded(nz, sg, s, x, y, rows, cols, gs, threads):
    """Rows are independent, so the reference's single-threaded function is run
    on disjoint row ranges from several host threads (ctypes drops the GIL)."""
    from concurrent.futures import ThreadPoolExecutor
    if threads <= 0:
        threads = os.cpu_count() or 1
    fn = ref().ref_cpu_reference
    mpr, gpr = cols // 32, cols // gs
    step = (rows + threads - 1) // threads

    def run(r0):
        n = min(step, rows - r0)
        if n <= 0:
            return
        fn(ctypes.cast(nz.ctypes.data + r0 * mpr * 4, _u32p),
           ctypes.cast(sg.ctypes.data + r0 * mpr * 4, _u32p),
           ctypes.cast(s.ctypes.data + r0 * gpr * 4, _f32p), _p(x, _f32p),
           ctypes.cast(y.ctypes.data + r0 * 4, _f32p), n, cols, gs)

    with ThreadPoolExecutor(threads) as ex:
        list(ex.map(run, range(0, rows, step)))


def matvec_f16(nz, sg, scales_f16, x_f16, group_size=128, threads=0):
    """float16 scales and activations, x [K] or [B,K]; float32 result."""
    nz, sg = _c(nz, np.uint32), _c(sg, np.uint32)
    s = _c(scales_f16, np.float16).view(np.uint16)
    x = _c(x_f16, np.float16)
    single = x.ndim == 1
    x2 = np.atleast_2d(x).view(np.uint16)
    rows, cols = nz.shape[0], nz.shape[1] * 32
    y = np.empty((x2.shape[0], rows), np.float32)
    port().oracle_matvec_f16(_p(nz, _u32p), _p(sg, _u32p), _p(s, _u16p), _p(x2, _u16p),
                             _p(y, _f32p), x2.shape[0], rows, cols, group_size, threads)
    return y[0] if single else y


def matvec_i8(nz, sg, scales_f16, x_i8, input_scale, group_size=128, threads=0):
    nz, sg = _c(nz, np.uint32), _c(sg, np.uint32)
    s = _c(scales_f16, np.float16).view(np.uint16)
    x = _c(x_i8, np.int8)
    rows, cols = nz.shape[0], nz.shape[1] * 32
    y = np.empty(rows, np.float32)
    port().oracle_matvec_i8(_p(nz, _u32p), _p(sg, _u32p), _p(s, _u16p), _p(x, _i8p),
                            float(input_scale), _p(y, _f32p), rows, cols, group_size, threads)
    return y


def num_threads() -> int:
    return int(port().oracle_num_threads())
