"""The .tllm container: header bytes, section order and sizes, writer <-> reader round
trip, and (when the reference checkout is present) the reference's own offset checker."""
import os
import struct
import subprocess
import sys

import numpy as np
import pytest

from oracle.cpu import REF_DIR
from ternary_llm_b200 import tllm_format as tf

DIAGNOSE = os.path.join(REF_DIR, "tools", "diagnose_format.py")

CFG = tf.TllmConfig(vocab_size=320, hidden_dim=256, intermediate_dim=512, n_layers=2, n_heads=4,
                    n_kv_heads=2, head_dim=64, max_seq_len=128, rope_theta=500000.0, rms_norm_eps=1e-5)


def test_header_bytes_match_the_reference_struct():
    raw = CFG.pack_header()
    assert len(raw) == 256 and raw[60:] == b"\x00" * 196
    f = struct.unpack("<15I", raw[:60])
    assert f[0] == 0x544C4C4D and f[1] == 1 and f[2] == 0
    assert f[3:11] == (320, 256, 512, 2, 4, 2, 128, 64)
    assert struct.unpack("<f", struct.pack("<I", f[11]))[0] == 500000.0
    assert f[12] == 128 and f[14] == 0
    back = tf.TllmConfig.unpack_header(raw)
    assert back == CFG
    with pytest.raises(ValueError):
        tf.TllmConfig.unpack_header(b"\x00" * 256)


@pytest.mark.parametrize("ternary_head", [False, True])
def test_round_trip_and_sizes(tmp_path, ternary_head):
    cfg = tf.TllmConfig(**{**CFG.__dict__, "lm_head_ternary": ternary_head})
    m = tf.random_model(cfg, seed=3)
    m.tokenizer = b"not a real tokenizer"
    path = str(tmp_path / "m.tllm")
    tf.write_tllm(path, m)
    assert os.path.getsize(path) == tf.expected_size(cfg, len(m.tokenizer))
    r = tf.read_tllm(path)
    assert r.config == cfg and r.tokenizer == m.tokenizer
    assert np.array_equal(r.embedding, m.embedding) and np.array_equal(r.final_norm, m.final_norm)
    for a, b in zip(r.layers, m.layers):
        for name in tf.PROJ_NAMES:
            assert np.array_equal(a[name].nonzero_masks, b[name].nonzero_masks)
            assert np.array_equal(a[name].sign_masks, b[name].sign_masks)
            assert np.array_equal(a[name].scales.view(np.uint16), b[name].scales.view(np.uint16))
        assert np.array_equal(a["attn_norm"], b["attn_norm"])
    shapes = dict((n, (o, i)) for n, o, i in cfg.proj_shapes())
    assert r.layers[0]["q_proj"].shape == shapes["q_proj"] == (256, 256)
    assert r.layers[0]["k_proj"].shape == (128, 256) and r.layers[0]["down_proj"].shape == (256, 512)
    # the q_proj of layer 0 starts right after header + embedding (src/model.cpp:129-139)
    raw = open(path, "rb").read()
    off = 256 + 320 * 256 * 2
    assert raw[off:off + 16] == m.layers[0]["q_proj"].nonzero_masks.tobytes()[:16]


def test_truncated_file_is_rejected(tmp_path):
    m = tf.random_model(CFG, seed=1)
    path = str(tmp_path / "m.tllm")
    tf.write_tllm(path, m)
    data = open(path, "rb").read()
    open(path, "wb").write(data[:len(data) // 2])
    with pytest.raises(ValueError):
        tf.read_tllm(path)


@pytest.mark.skipif(not os.path.exists(DIAGNOSE),
                    reason="reference checkout not present")
def test_reference_offset_checker_accepts_the_file(tmp_path):
    m = tf.random_model(CFG, seed=2)
    m.tokenizer = b"x" * 100
    path = str(tmp_path / "m.tllm")
    tf.write_tllm(path, m)
    out = subprocess.run([sys.executable, DIAGNOSE, path],
                         capture_output=True, text=True, check=True).stdout
    assert "MISMATCH" not in out and "Looks valid" in out
    assert "Tokenizer size at expected position: 100 bytes" in out
