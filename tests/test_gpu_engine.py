"""The reference engine end to end on a tiny random-init model: its own ternary kernels
against this library behind the unchanged call sites (oracle/engine_main.cpp)."""
import os
import tempfile

import numpy as np
import pytest

from oracle import cpu
from tests import _engine_e2e as e2e
from ternary_llm_b200 import tllm_format as tf

pytestmark = pytest.mark.gpu
HAVE = all(os.path.exists(os.path.join(os.path.dirname(cpu.DROPIN_TEST), n)) for n in ("engine_ref", "engine_tllm"))


@pytest.mark.skipif(not HAVE, reason="engine binaries not built (needs the reference checkout)")
def test_engine_logits_agree_between_reference_kernels_and_this_library():
    cfg = tf.TllmConfig(**e2e.ARCHS["tiny"])
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "tiny.tllm")
        tf.write_tllm(path, tf.random_model(cfg, seed=7))
        # prefill only: the GEMM path (M = 48 tokens)
        res = e2e.run_engines(path, 48, 0, d)
        a, b = res["engine_ref"][1], res["engine_tllm"][1]
        assert np.isfinite(a).all() and np.isfinite(b).all()
        assert np.abs(a - b).max() <= 2e-2 * max(1.0, np.abs(a).max())
        # prefill + decode steps: GEMV (INT8 activation) path behind the same call sites
        res = e2e.run_engines(path, 16, 4, d)
        a, b = res["engine_ref"][1], res["engine_tllm"][1]
        assert np.isfinite(b).all()
        if res["engine_ref"][0]["last_token"] == res["engine_tllm"][0]["last_token"]:
            assert np.abs(a - b).max() <= 5e-2 * max(1.0, np.abs(a).max())
