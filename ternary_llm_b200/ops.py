"""Host-side mirror of the reference's operator interface for the contraction path.

The four functions carry the names and argument order of the reference's
include/kernels.cuh:11-40 (namespace ternary) and call the C ABI of
libtllm_b200.so with the tensors' device pointers on torch's current stream.
PyTorch is used only to own device memory and streams.  All tensors must be
CUDA tensors on the current device and contiguous; nothing here computes on the
CPU or falls back to torch ops.
"""
from __future__ import annotations

import torch

from . import _lib

GROUP_SIZE = 128
MAX_BATCH = 16


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _chk(t: torch.Tensor, dtype, name: str, numel: int | None = None) -> int:
    """Device pointer of `t` after the checks that keep a launch from touching memory it
    should not: CUDA tensor on the CURRENT device (the kernels run on the current device's
    stream), the stated dtype, contiguous, and at least `numel` elements when given."""
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (no CPU path exists)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    cur = torch.cuda.current_device()
    if t.device.index != cur:
        raise ValueError(f"{name} is on cuda:{t.device.index} but the current device is cuda:{cur}; "
                         f"make the tensor's device current (torch.cuda.device) before the call")
    if numel is not None and t.numel() < numel:
        raise ValueError(f"{name} holds {t.numel()} elements, the call needs {numel}")
    return t.data_ptr()


def _mask_dtype_ok(t: torch.Tensor) -> bool:
    return t.dtype in (torch.int32, torch.uint32)


def _dims(rows: int, cols: int, batch: int = 1) -> None:
    if rows < 1 or cols < GROUP_SIZE or cols % GROUP_SIZE or batch < 1:
        raise ValueError(f"rows={rows} cols={cols} batch={batch}: need rows, batch >= 1 and cols a positive multiple of 128")


def _weights(nonzero_masks, sign_masks, scales, rows: int | None = None, cols: int | None = None):
    for n, t in (("nonzero_masks", nonzero_masks), ("sign_masks", sign_masks)):
        if not _mask_dtype_ok(t):
            raise TypeError(f"{n} must be int32/uint32 words, got {t.dtype}")
    words = scl = None
    if rows is not None:
        _dims(rows, cols)
        words, scl = rows * (cols // 32), rows * (cols // GROUP_SIZE)
    return (_chk(nonzero_masks, nonzero_masks.dtype, "nonzero_masks", words),
            _chk(sign_masks, sign_masks.dtype, "sign_masks", words),
            _chk(scales, torch.float16, "scales", scl))


def ternary_gemv(nonzero_masks, sign_masks, scales, input, output, rows: int, cols: int,
                 group_size: int = GROUP_SIZE) -> None:
    """y = W x for one FP16 vector (reference include/kernels.cuh:11-14)."""
    nz, sg, sc = _weights(nonzero_masks, sign_masks, scales, rows, cols)
    _lib.check(_lib.lib().tllm_b200_gemv(nz, sg, sc, _chk(input, torch.float16, "input", cols),
                                         _chk(output, torch.float16, "output", rows),
                                         rows, cols, group_size, _stream()))


def ternary_gemv_batched(nonzero_masks, sign_masks, scales, input, output, batch: int, rows: int,
                         cols: int, group_size: int = GROUP_SIZE) -> None:
    """y[b] = W x[b] for 1..16 vectors in one pass over the weights."""
    nz, sg, sc = _weights(nonzero_masks, sign_masks, scales, rows, cols)
    _dims(rows, cols, batch)
    _lib.check(_lib.lib().tllm_b200_gemv_batched(nz, sg, sc, _chk(input, torch.float16, "input", batch * cols),
                                                 _chk(output, torch.float16, "output", batch * rows),
                                                 batch, rows, cols, group_size, _stream()))


def ternary_gemv_int8(nonzero_masks, sign_masks, weight_scales, input_int8, input_scale: float,
                      output, rows: int, cols: int, group_size: int = GROUP_SIZE) -> None:
    """INT8-activation GEMV (reference include/kernels.cuh:19-24)."""
    nz, sg, sc = _weights(nonzero_masks, sign_masks, weight_scales, rows, cols)
    _lib.check(_lib.lib().tllm_b200_gemv_int8(nz, sg, sc, _chk(input_int8, torch.int8, "input_int8", cols),
                                              float(input_scale), _chk(output, torch.float16, "output", rows),
                                              rows, cols, group_size, _stream()))


def quantize_absmax_int8(input, output, scale, n: int) -> None:
    """half[n] -> int8[n] + device float scale (reference include/kernels.cuh:30-32)."""
    if n < 1:
        raise ValueError(f"n={n} must be positive")
    _lib.check(_lib.lib().tllm_b200_quantize_absmax_int8(
        _chk(input, torch.float16, "input", n), _chk(output, torch.int8, "output", n),
        _chk(scale, torch.float32, "scale", 1), n, _stream()))


def ternary_gemm(A, nz_B, sign_B, scales_B, C, M: int, N: int, K: int,
                 group_size: int = GROUP_SIZE) -> None:
    """C[M,N] = A[M,K] . W^T (reference include/kernels.cuh:37-40)."""
    nz, sg, sc = _weights(nz_B, sign_B, scales_B, N, K)
    _dims(N, K, M)
    _lib.check(_lib.lib().tllm_b200_gemm(_chk(A, torch.float16, "A", M * K), nz, sg, sc,
                                         _chk(C, torch.float16, "C", M * N), M, N, K, group_size, _stream()))


# --------------------------------------------------------------------------
# Prepared weights (load-time repack for the streaming tensor-core GEMV)
# --------------------------------------------------------------------------
def packed_bytes(rows: int, cols: int) -> int:
    return int(_lib.lib().tllm_b200_packed_bytes(rows, cols))


class PreparedWeight:
    """One ternary matrix in the packed layout, made from the three reference
    arrays.  Keeps the source tensors alive and, with register=True, makes the
    reference-signature entry points (ternary_gemv ...) called with these source
    tensors use the packed copy, as the C++ engine integration does."""

    def __init__(self, nonzero_masks, sign_masks, scales, rows: int, cols: int, register: bool = True,
                 keep_source: bool = True, storage=None):
        """storage: a uint8 CUDA tensor (view) of packed_bytes(rows, cols) bytes to pack into
        instead of a fresh allocation -- see prepare_group."""
        nz, sg, sc = _weights(nonzero_masks, sign_masks, scales, rows, cols)
        self.rows, self.cols = rows, cols
        if register and not keep_source:
            raise ValueError("registered weights are keyed by the source tensor and must keep it")
        # the source tensors can be dropped when only the packed entry points are used
        self.nonzero_masks, self.sign_masks, self.scales = (
            (nonzero_masks, sign_masks, scales) if keep_source else (None, None, None))
        nbytes = packed_bytes(rows, cols)
        if nbytes == 0:
            raise ValueError(f"unsupported shape rows={rows} cols={cols}")
        if storage is None:
            storage = torch.empty(nbytes, dtype=torch.uint8, device=nonzero_masks.device)
        elif (storage.numel() != nbytes or storage.dtype != torch.uint8 or not storage.is_contiguous()
              or storage.device != nonzero_masks.device):
            raise ValueError(f"storage must be a contiguous uint8 tensor of {nbytes} bytes on {nonzero_masks.device}")
        self.packed = storage
        _lib.check(_lib.lib().tllm_b200_weight_prepare(nz, sg, sc, rows, cols, GROUP_SIZE,
                                                       self.packed.data_ptr(), nbytes, _stream()))
        self.registered = False
        if register:
            _lib.check(_lib.lib().tllm_b200_weight_register(nz, self.packed.data_ptr(), rows, cols))
            self.registered = True

    def unpack(self):
        """Back to (nonzero_masks, sign_masks, scales) in the reference layout."""
        dev = self.packed.device
        nz = torch.empty(self.rows, self.cols // 32, dtype=torch.int32, device=dev)
        sg = torch.empty_like(nz)
        sc = torch.empty(self.rows, self.cols // GROUP_SIZE, dtype=torch.float16, device=dev)
        _lib.check(_lib.lib().tllm_b200_weight_unpack(_chk(self.packed, torch.uint8, "packed weights"), self.rows,
                                                      self.cols, GROUP_SIZE,
                                                      nz.data_ptr(), sg.data_ptr(), sc.data_ptr(), _stream()))
        return nz, sg, sc

    def release(self):
        if self.registered:
            _lib.lib().tllm_b200_weight_unregister(self.nonzero_masks.data_ptr())
            self.registered = False

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


def prepare_group(weights, register: bool = False, keep_source: bool = False):
    """Packs several matrices that share their input vector (q, k, v; gate, up) back to back
    in one allocation.  weights: list of (nonzero_masks, sign_masks, scales, rows, cols).
    ternary_gemv_packed_multi on the returned list streams them as ONE matrix in a single
    launch (every row count but the last must be a multiple of 16 for that)."""
    sizes = [packed_bytes(r, c) for (_, _, _, r, c) in weights]
    buf = torch.empty(sum(sizes), dtype=torch.uint8, device=weights[0][0].device)
    out, off = [], 0
    for (nz, sg, sc, r, c), n in zip(weights, sizes):
        out.append(PreparedWeight(nz, sg, sc, r, c, register=register, keep_source=keep_source or register,
                                  storage=buf[off:off + n]))
        off += n
    return out


def ternary_gemv_packed(w: PreparedWeight, input, output, batch: int = 1) -> None:
    """y[b] = W x[b] on prepared weights, FP16 activations, 1..16 vectors."""
    _dims(w.rows, w.cols, batch)
    _lib.check(_lib.lib().tllm_b200_gemv_packed(_chk(w.packed, torch.uint8, "packed weights"),
                                                _chk(input, torch.float16, "input", batch * w.cols),
                                                _chk(output, torch.float16, "output", batch * w.rows), batch, w.rows, w.cols,
                                                _stream()))


def ternary_gemv_int8_packed(w: PreparedWeight, input_int8, input_scale: float, output) -> None:
    """INT8-activation GEMV on prepared weights."""
    _lib.check(_lib.lib().tllm_b200_gemv_int8_packed(_chk(w.packed, torch.uint8, "packed weights"),
                                                     _chk(input_int8, torch.int8, "input_int8", w.cols),
                                                     float(input_scale), _chk(output, torch.float16, "output", w.rows),
                                                     w.rows, w.cols, _stream()))


def ternary_gemv_packed_multi(weights, input, outputs) -> None:
    """y_i = W_i x for up to 4 prepared matrices sharing the vector x (q/k/v, gate/up)
    in one launch."""
    import ctypes
    n = len(weights)
    cols = weights[0].cols
    if any(w.cols != cols for w in weights) or len(outputs) != n:
        raise ValueError("fused matrices must share the column count and have one output each")
    packed = (ctypes.c_void_p * n)(*[_chk(w.packed, torch.uint8, "packed weights") for w in weights])
    ys = (ctypes.c_void_p * n)(*[_chk(y, torch.float16, "output", w.rows) for w, y in zip(weights, outputs)])
    rows = (ctypes.c_int * n)(*[w.rows for w in weights])
    _lib.check(_lib.lib().tllm_b200_gemv_packed_multi(n, packed, ys, rows, cols,
                                                      _chk(input, torch.float16, "input", cols), _stream()))


def ternary_gemv_packed_multi_norm(weights, a, b, norm_weight, res_out, eps: float, outputs) -> None:
    """y_i = W_i x with x = rmsnorm(a (+ b)) * norm_weight made inside the launch (b and res_out
    may be None; res_out receives a + b and must be a different tensor).  weights: matrices
    packed back to back (prepare_group), or a single prepared matrix in a list."""
    import ctypes
    n = len(weights)
    cols = weights[0].cols
    if any(w.cols != cols for w in weights) or len(outputs) != n:
        raise ValueError("fused matrices must share the column count and have one output each")
    if res_out is not None and (res_out.data_ptr() == a.data_ptr() or (b is not None and res_out.data_ptr() == b.data_ptr())):
        raise ValueError("res_out must not alias an input")
    packed = (ctypes.c_void_p * n)(*[_chk(w.packed, torch.uint8, "packed weights") for w in weights])
    ys = (ctypes.c_void_p * n)(*[_chk(y, torch.float16, "output", w.rows) for w, y in zip(weights, outputs)])
    rows = (ctypes.c_int * n)(*[w.rows for w in weights])
    _lib.check(_lib.lib().tllm_b200_gemv_packed_multi_norm(
        n, packed, ys, rows, cols, _chk(a, torch.float16, "a", cols),
        _chk(b, torch.float16, "b", cols) if b is not None else None,
        _chk(norm_weight, torch.float16, "norm_weight", cols),
        _chk(res_out, torch.float16, "res_out", cols) if res_out is not None else None, float(eps), _stream()))


AR_MAX_CTAS = 256


class FusedAllReduce:
    """Peer-memory buffers for tllm_b200_gemv_packed_allreduce, one per process group.

    Allocates one symmetric-memory tensor per rank (the receive slots),
    exchanges the mappings with torch's symmetric-memory rendezvous, and keeps the
    per-rank pointer tables.  PyTorch is used for the mapping only; the data path is the
    GEMV kernel's own peer stores."""

    def __init__(self, group, rows_max: int, device):
        import ctypes

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rows_max = rows_max
        recv_bytes = 2 * self.world * rows_max * 8          # {value, launch number} words, two parities
        self.buf = symm_mem.empty(recv_bytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group.group_name if hasattr(group, "group_name") else group)
        torch.cuda.synchronize()
        dist.barrier(group)
        ptrs = list(self.handle.buffer_ptrs)
        self.recv = (ctypes.c_void_p * self.world)(*ptrs)
        self.epoch = torch.zeros(AR_MAX_CTAS, dtype=torch.int32, device=device)
        self._trace = None

    def trace(self, records: int = 0):
        """records > 0: start recording the time stamps of this device's fused all-reduce
        launches (tllm_b200_allreduce_trace) into a buffer of that many records; 0: stop and
        return what was recorded as an int64 array [n, 8] (see the header for the fields)."""
        if records > 0:
            self._trace = torch.zeros(records, 8, dtype=torch.int64, device=self.epoch.device)
            _lib.check(_lib.lib().tllm_b200_allreduce_trace(self._trace.data_ptr(), records))
            return None
        _lib.check(_lib.lib().tllm_b200_allreduce_trace(None, 0))
        out, self._trace = self._trace, None
        torch.cuda.synchronize()
        return None if out is None else out.cpu().numpy()


def ternary_gemv_packed_allreduce(w: PreparedWeight, input, output, ar: FusedAllReduce) -> None:
    """Row-parallel y = sum over ranks of W_r x_r with the all-reduce fused into the kernel."""
    _lib.check(_lib.lib().tllm_b200_gemv_packed_allreduce(
        _chk(w.packed, torch.uint8, "packed weights"), _chk(input, torch.float16, "input", w.cols),
        _chk(output, torch.float16, "output", w.rows),
        w.rows, w.cols, ar.rank, ar.world, ar.recv, ar.epoch.data_ptr(), ar.rows_max, _stream()))


def ternary_gemm_packed(A, w: PreparedWeight, C, M: int) -> None:
    """C[M,N] = A[M,K] . W^T on prepared weights (tcgen05 kernel for M > 8)."""
    _dims(w.rows, w.cols, M)
    _lib.check(_lib.lib().tllm_b200_gemm_packed(_chk(A, torch.float16, "A", M * w.cols),
                                                _chk(w.packed, torch.uint8, "packed weights"),
                                                _chk(C, torch.float16, "C", M * w.rows), M, w.rows, w.cols, _stream()))


def check_device_errors() -> None:
    """Synchronises the current stream and raises if a kernel's bounded wait expired."""
    _lib.check(_lib.lib().tllm_b200_check_device_errors(_stream()))
