"""CPU checks of the host side: packer against the reference's fixtures, the
shared library's exported symbols against the header, argument validation that
needs no GPU."""
import ctypes
import os
import re

import numpy as np
import pytest

import ternary_llm_b200 as tl
from ternary_llm_b200 import _lib, pack

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name))
    cases = {}
    for key in z.files:
        case, field = key.split("/")
        cases.setdefault(case, {})[field] = z[key]
    return cases


def test_packer_matches_reference_fixtures(golden_dir):
    for name, c in _load(golden_dir, "packing.npz").items():
        t, s = pack.ternarize_tensor(c["w"], 128, 0.7)
        assert (t == c["ternary"]).all(), name
        assert (s.view(np.uint16) == c["scales"].view(np.uint16)).all(), name
        nz, sg = pack.pack_ternary_to_bitmasks(t)
        assert nz.dtype == np.uint32 and (nz == c["nz"]).all() and (sg == c["sign"]).all(), name
        assert (pack.unpack_bitmasks(nz, sg) == t).all(), name


def test_packer_known_words():
    t = np.zeros((2, 64), np.int8)
    t[0, 0], t[0, 1], t[0, 31] = 1, -1, 1
    nz, sg = pack.pack_ternary_to_bitmasks(t)
    assert nz[0, 0] == 0x80000003 and sg[0, 0] == 0x80000001


def test_packer_rejects_bad_shapes():
    with pytest.raises(ValueError):
        pack.pack_ternary_to_bitmasks(np.zeros((2, 33), np.int8))


def test_pad_to_multiple():
    assert pack.pad_to_multiple(np.ones((4, 50)), 32).shape == (4, 64)
    assert pack.pad_to_multiple(np.ones((4, 64)), 32).shape == (4, 64)


def test_random_weight_distribution():
    nz, sg, sc = pack.random_ternary_weight(128, 1024, seed=1)
    t = pack.unpack_bitmasks(nz, sg)
    assert 0.40 < (t == 0).mean() < 0.44
    assert (sg & ~nz == 0).all()
    assert sc.shape == (128, 8) and sc.dtype == np.float16


def test_library_exports_every_declared_symbol():
    headers = [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))
               if f.endswith(".h")]
    declared = set()
    for h in headers:
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        declared |= set(re.findall(r"\b(tllm_b200_\w+)\s*\(", text))
    assert declared, "no declarations found"
    handle = ctypes.CDLL(tl.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(handle, name), f"{name} declared in include/ but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes table and header disagree"


def test_status_strings_and_version():
    h = tl.lib()
    assert h.tllm_b200_version() >= 1000
    assert h.tllm_b200_status_string(0) == b"ok"
    for st in range(-10, 0):
        assert h.tllm_b200_status_string(st) not in (b"", b"unknown status")


def test_argument_errors_need_no_gpu():
    h = tl.lib()
    # null pointers and bad shapes are rejected before any CUDA call
    assert h.tllm_b200_gemv(None, None, None, None, None, 16, 128, 128, None) == -1
    buf = ctypes.create_string_buffer(4096 + 64)
    p = (ctypes.addressof(buf) + 63) & ~63
    assert h.tllm_b200_gemv(p, p, p, p, p, 16, 100, 128, None) == -3      # cols % 128
    assert h.tllm_b200_gemv(p, p, p, p, p, 16, 128, 64, None) == -4       # group size
    assert h.tllm_b200_gemv(p + 4, p, p, p, p, 16, 128, 128, None) == -2  # alignment
    assert h.tllm_b200_gemv_batched(p, p, p, p, p, 17, 16, 128, 128, None) == -5
    assert h.tllm_b200_gemm(p, p, p, p, p, 0, 16, 128, 128, None) == -3
    assert b"cols" in h.tllm_b200_last_error() or b"M=" in h.tllm_b200_last_error()


def test_layer_argument_errors_need_no_gpu():
    h = tl.lib()
    buf = ctypes.create_string_buffer(4096 + 64)
    p = (ctypes.addressof(buf) + 63) & ~63
    assert h.tllm_b200_rmsnorm(None, p, p, None, None, 1, 128, 1e-5, None) == -1
    assert h.tllm_b200_rmsnorm(p, p, p, None, None, 1, 0, 1e-5, None) == -3
    assert h.tllm_b200_rope(p, None, 1, 1, 4, 2, 64, 0, 10000.0, None) == -1
    assert h.tllm_b200_rope(p, p, 1, 1, 4, 2, 63, 0, 10000.0, None) == -3            # odd head_dim
    assert h.tllm_b200_attention(p, p, p, None, 1, 4, 2, 64, 1, 1, 8, None) == -1
    assert h.tllm_b200_attention(p, p, p, p, 1, 0, 2, 64, 1, 1, 8, None) == -3
    assert h.tllm_b200_silu_mul(p, p, p, -1, None) == -3
    assert h.tllm_b200_add(p + 2, p, p, 8, None) == -2
    assert h.tllm_b200_fp16_gemv(p, p, p, 4, 0, None) == -3
    assert h.tllm_b200_embedding_lookup(p, None, p, 1, 8, None) == -1
    assert h.tllm_b200_decoder_create(None, 0, None) == -1
    assert h.tllm_b200_decoder_reset(None, None) == -1
    assert h.tllm_b200_decoder_generate(None, 0, 0, 1, None, None) == -1
    tables = (ctypes.c_void_p * 1)(p)
    rows = (ctypes.c_int * 1)(16)
    assert h.tllm_b200_gemv_int8_packed_multi(5, tables, tables, rows, 128, p, p, None) == -5
    assert h.tllm_b200_gemv_int8_packed_multi(1, tables, tables, rows, 100, p, p, None) == -3
    # a model description with an unsupported group size is refused before anything is allocated
    d = _lib.ModelDesc()
    layers = (_lib.LayerWeightsDesc * 1)()
    d.layers, d.embedding_table, d.final_norm_weight = layers, p, p
    d.group_size, d.n_layers = 64, 1
    out = ctypes.c_void_p()
    assert h.tllm_b200_decoder_create(ctypes.byref(d), 0, ctypes.byref(out)) == -4


def test_ops_refuse_cpu_tensors():
    import torch
    a = torch.zeros(16, 4, dtype=torch.int32)
    s = torch.zeros(16, 1, dtype=torch.float16)
    x = torch.zeros(128, dtype=torch.float16)
    y = torch.zeros(16, dtype=torch.float16)
    with pytest.raises(ValueError):
        tl.ternary_gemv(a, a, s, x, y, 16, 128)


class _FakeCuda:
    """Stands in for a CUDA tensor in the wrappers' checks (no GPU on the build machine): the
    checks read only these attributes."""

    def __init__(self, numel, dtype, index=0, contiguous=True):
        import torch
        self._n, self.dtype, self.is_cuda = numel, dtype, True
        self.device = torch.device("cuda", index)
        self._c = contiguous

    def numel(self):
        return self._n

    def is_contiguous(self):
        return self._c

    def data_ptr(self):
        return 0x1000


def test_wrappers_refuse_short_tensors_and_foreign_devices(monkeypatch):
    """Nothing may be launched on a tensor that is too small for the stated shape or that lives
    on another GPU than the current one: the kernels trust rows/cols and run on the current
    device, so either mistake would make them touch memory that is not theirs."""
    import torch
    from ternary_llm_b200 import ops
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)

    class NoCall:
        def __getattr__(self, name):
            def fn(*a):
                raise AssertionError(f"{name} was called although an argument check should have failed")
            return fn
    monkeypatch.setattr(_lib, "lib", lambda: NoCall())
    n, k = 64, 256
    i32, f16, i8 = torch.int32, torch.float16, torch.int8
    good = lambda: (_FakeCuda(n * k // 32, i32), _FakeCuda(n * k // 32, i32), _FakeCuda(n * k // 128, f16))
    # short mask / scale / input / output arrays
    for bad in range(3):
        w = list(good())
        w[bad] = _FakeCuda(w[bad].numel() - 1, w[bad].dtype)
        with pytest.raises(ValueError, match="holds"):
            tl.ternary_gemv(*w, _FakeCuda(k, f16), _FakeCuda(n, f16), n, k)
    with pytest.raises(ValueError, match="holds"):
        tl.ternary_gemv(*good(), _FakeCuda(k - 1, f16), _FakeCuda(n, f16), n, k)
    with pytest.raises(ValueError, match="holds"):
        tl.ternary_gemv(*good(), _FakeCuda(k, f16), _FakeCuda(n - 1, f16), n, k)
    with pytest.raises(ValueError, match="holds"):
        tl.ternary_gemv_batched(*good(), _FakeCuda(3 * k, f16), _FakeCuda(4 * n, f16), 4, n, k)
    with pytest.raises(ValueError, match="holds"):
        tl.ternary_gemv_int8(*good(), _FakeCuda(k - 16, i8), 1.0, _FakeCuda(n, f16), n, k)
    with pytest.raises(ValueError, match="holds"):
        tl.ternary_gemm(_FakeCuda(2 * k, f16), *good(), _FakeCuda(3 * n, f16), 3, n, k)
    with pytest.raises(ValueError, match="holds"):
        tl.quantize_absmax_int8(_FakeCuda(k, f16), _FakeCuda(k, i8), _FakeCuda(0, torch.float32), k)
    # a tensor on another device than the current one
    with pytest.raises(ValueError, match="current device"):
        tl.ternary_gemv(*good(), _FakeCuda(k, f16, index=1), _FakeCuda(n, f16), n, k)
    with pytest.raises(ValueError, match="current device"):
        ops.PreparedWeight(_FakeCuda(n * k // 32, i32, index=1), _FakeCuda(n * k // 32, i32, index=1),
                           _FakeCuda(n * k // 128, f16, index=1), n, k)
    # shapes the kernels do not take
    with pytest.raises(ValueError, match="multiple of 128"):
        tl.ternary_gemv(*good(), _FakeCuda(k, f16), _FakeCuda(n, f16), n, 200)


def test_torch_synth_matches_numpy_packer():
    import torch
    from ternary_llm_b200 import synth
    w = torch.randn(40, 512, generator=torch.Generator().manual_seed(3)) * 0.02
    nz, sg, sc = synth.ternarize_pack(w)
    t, s = pack.ternarize_tensor(w.numpy(), 128, 0.7)
    n2, g2 = pack.pack_ternary_to_bitmasks(t)
    assert (nz.numpy().view(np.uint32) == n2).all() and (sg.numpy().view(np.uint32) == g2).all()
    assert (sc.numpy().reshape(-1).view(np.uint16) == s.view(np.uint16)).all()
