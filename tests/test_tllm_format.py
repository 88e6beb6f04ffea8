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


@pytest.mark.parametrize("world", [1, 2, 4])
def test_tensor_parallel_shards_reassemble_the_projection(world):
    """Column shards stacked and row shards summed give the unsharded oracle result; the
    shards' unpacked ternary values are the corresponding slices bit for bit."""
    from oracle import oracle
    cfg = tf.TllmConfig(**{**CFG.__dict__, "hidden_dim": 512, "intermediate_dim": 1024, "n_heads": 8, "n_layers": 1,
                           "vocab_size": 32})
    m = tf.random_model(cfg, seed=9)
    rng = np.random.default_rng(21)
    for name, rows, cols in cfg.proj_shapes():
        t = m.layers[0][name]
        x = rng.standard_normal(cols).astype(np.float16)
        full = oracle.ternary_matvec(t.nonzero_masks, t.sign_masks, t.scales, x, 128, np.float64)
        tern = oracle.unpack_bitmasks(t.nonzero_masks, t.sign_masks)
        parts = [tf.shard_ternary(t, name, r, world) for r in range(world)]
        c = np.ascontiguousarray
        if name in tf.TP_COLUMN:
            assert all(p.shape == (rows // world, cols) for p in parts)
            y = np.concatenate([oracle.ternary_matvec(c(p.nonzero_masks), c(p.sign_masks), c(p.scales), x, 128,
                                                      np.float64) for p in parts])
            assert np.array_equal(y, full)
            got = np.concatenate([oracle.unpack_bitmasks(c(p.nonzero_masks), c(p.sign_masks)) for p in parts], 0)
        else:
            assert name in tf.TP_ROW and all(p.shape == (rows, cols // world) for p in parts)
            kw = cols // world
            y = sum(oracle.ternary_matvec(c(p.nonzero_masks), c(p.sign_masks), c(p.scales), x[r * kw:(r + 1) * kw],
                                          128, np.float64) for r, p in enumerate(parts))
            bound = oracle.tolerance_bound(t.nonzero_masks, t.sign_masks, t.scales, x)
            assert (np.abs(y - full) <= 1e-9 * bound + 1e-12).all()
            got = np.concatenate([oracle.unpack_bitmasks(c(p.nonzero_masks), c(p.sign_masks)) for p in parts], 1)
        assert np.array_equal(got, tern)


def test_shards_that_do_not_divide_are_rejected():
    m = tf.random_model(CFG, seed=9)
    layer = m.layers[0]
    with pytest.raises(ValueError):
        tf.shard_ternary(layer["o_proj"], "o_proj", 0, 4)        # 256 columns: 64 per rank is no whole group
    with pytest.raises(ValueError):
        tf.shard_ternary(layer["k_proj"], "k_proj", 0, 3)
    with pytest.raises(ValueError):
        tf.shard_ternary(layer["q_proj"], "q_proj", 2, 2)
    with pytest.raises(ValueError):
        tf.shard_ternary(layer["q_proj"], "lm_head", 0, 2)
    assert tf.shard_ternary(layer["q_proj"], "q_proj", 0, 1) is layer["q_proj"]
