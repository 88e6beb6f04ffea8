"""The decoder (include/tllm_b200_layer.h: the reference's Transformer on this library's
kernels) against the numpy restatement of the reference forward pass on a small random
model, its graph-replayed greedy loop against step-by-step calls, and the reference
engine's own Transformer linked against this library for every operator."""
import os
import tempfile

import numpy as np
import pytest
import torch

import ternary_llm_b200 as tl
from oracle import cpu
from oracle import layer_oracle as LO
from tests import _engine_e2e as e2e
from ternary_llm_b200 import tllm_format as tf

pytestmark = pytest.mark.gpu


def cfg_small(**kw):
    base = dict(vocab_size=1024, hidden_dim=256, intermediate_dim=512, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=64,
                max_seq_len=320, rope_theta=10000.0, rms_norm_eps=1e-5)
    base.update(kw)
    return tf.TllmConfig(**base)


def toks(n, vocab, seed=0):
    return np.random.default_rng(seed).integers(0, vocab, n).astype(np.int32)


def close(a, b, rel):
    a, b = a.astype(np.float32), b.astype(np.float32)
    return np.abs(a - b).max() <= rel * max(1.0, np.abs(b).max())


@pytest.mark.parametrize("ternary_head", [False, True])
def test_prefill_and_decode_logits_against_the_oracle(ternary_head):
    cfg = cfg_small(lm_head_ternary=ternary_head)
    model = tf.random_model(cfg, seed=11)
    t = toks(12, cfg.vocab_size)
    for int8 in (False, True):
        dec = tl.Decoder(model, int8_decode=int8)
        ora = LO.Transformer(model, int8_decode=int8)
        got = dec.forward(torch.from_numpy(t[:9]).cuda(), 0).float().cpu().numpy()
        want = ora.forward(list(t[:9]), 0)
        assert close(got, want, 2e-2), "prefill"
        for i in range(9, 12):
            got = dec.forward(torch.from_numpy(t[i:i + 1]).cuda(), i).float().cpu().numpy()
            want = ora.forward([int(t[i])], i)
            assert np.isfinite(got).all()
            assert close(got, want, 4e-2), f"decode step {i} int8={int8}"
        dec.close()


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(8, 1, 128), (4, 4, 64), (16, 1, 32), (8, 2, 16)])
def test_fused_decode_attention_geometries(heads, kv_heads, head_dim):
    """Single-token steps (RoPE + append + attention in one launch) for grouped-query, multi-head and
    multi-query layouts, across the 128-position split boundary, against the oracle."""
    hidden = max(256, heads * head_dim)
    cfg = cfg_small(hidden_dim=hidden, intermediate_dim=512, n_layers=1, n_heads=heads, n_kv_heads=kv_heads,
                    head_dim=head_dim, max_seq_len=192, vocab_size=512)
    model = tf.random_model(cfg, seed=heads * 7 + head_dim)
    t = toks(140, cfg.vocab_size, seed=2)
    dec = tl.Decoder(model, int8_decode=True)
    ora = LO.Transformer(model, int8_decode=True)
    dec.forward(torch.from_numpy(t[:126]).cuda(), 0)
    ora.forward(list(t[:126]), 0)
    for i in range(126, 131):          # positions 126..130: one split, then two
        got = dec.forward(torch.from_numpy(t[i:i + 1]).cuda(), i).float().cpu().numpy()
        want = ora.forward([int(t[i])], i)
        assert np.isfinite(got).all()
        assert close(got, want, 4e-2), f"position {i}"
    tl.check_device_errors()
    dec.close()


@pytest.mark.parametrize("batch", [2, 5, 9])
def test_batched_lock_step_decode_matches_independent_sequences(batch):
    """B sequences with their own KV caches decoded in lock step (GEMV passes up to 6 sequences,
    the tcgen05 GEMM above) against the oracle run once per sequence (FP16 activations)."""
    cfg = cfg_small(max_seq_len=64)
    model = tf.random_model(cfg, seed=21)
    dec = tl.Decoder(model, int8_decode=True, max_batch=batch)
    oracles = [LO.Transformer(model, int8_decode=False) for _ in range(batch)]
    prompts = [toks(7, cfg.vocab_size, seed=100 + b) for b in range(batch)]
    for b in range(batch):
        got = dec.forward_seq(b, torch.from_numpy(prompts[b]).cuda(), 0).float().cpu().numpy()
        want = oracles[b].forward(list(prompts[b]), 0)
        assert close(got, want, 2e-2), f"prefill of sequence {b}"
    nxt = toks(batch, cfg.vocab_size, seed=7)
    for step in range(3):
        got = dec.forward_batch(torch.from_numpy(nxt).cuda(), 7 + step).float().cpu().numpy()
        assert got.shape == (batch, cfg.vocab_size) and np.isfinite(got).all()
        for b in range(batch):
            want = oracles[b].forward([int(nxt[b])], 7 + step)
            assert close(got[b], want, 4e-2), f"step {step} sequence {b}"
        nxt = got.argmax(axis=1).astype(np.int32)
    with pytest.raises(tl.TllmError):
        dec.forward_seq(batch, torch.from_numpy(prompts[0]).cuda(), 0)
    tl.check_device_errors()
    dec.close()


def test_generate_replays_the_same_steps_as_forward():
    cfg = cfg_small(n_layers=3, max_seq_len=320)
    model = tf.random_model(cfg, seed=3)
    dec = tl.Decoder(model, int8_decode=True)
    prompt = torch.from_numpy(toks(270, cfg.vocab_size, 1)).cuda()      # crosses a 256-position attention split
    logits = dec.forward(prompt, 0)
    first = int(logits.float().argmax().item())
    # reference loop: forward one token, argmax on the host
    want, tok, pos = [], first, prompt.numel()
    for _ in range(12):
        lg = dec.forward(torch.tensor([tok], dtype=torch.int32, device="cuda"), pos)
        tok = int(lg.float().argmax().item())
        want.append(tok)
        pos += 1
    dec.reset()
    dec.forward(prompt, 0)
    got, ms = dec.generate(first, prompt.numel(), 12)
    assert got == want
    assert ms > 0
    # a second call reuses the captured graph
    dec.reset()
    dec.forward(prompt, 0)
    got2, _ = dec.generate(first, prompt.numel(), 12)
    assert got2 == want
    tl.check_device_errors()
    dec.close()


def test_benchmark_shapes_properties():
    """At the benchmark's 1B layer shapes (hidden 2048, 32/8 heads of 64, intermediate 8192; 2 layers,
    a 4096-token vocabulary to keep it quick): the graph-replayed loop reproduces step-by-step
    forward calls token for token, a repeated step is idempotent, and reset + prefill restores
    the same logits bit for bit."""
    cfg = tf.TllmConfig(vocab_size=4096, hidden_dim=2048, intermediate_dim=8192, n_layers=2, n_heads=32, n_kv_heads=8,
                        head_dim=64, max_seq_len=512, rope_theta=500000.0, rms_norm_eps=1e-5)
    model = tf.random_model(cfg, seed=4)
    dec = tl.Decoder(model, int8_decode=True)
    prompt = torch.from_numpy(toks(300, cfg.vocab_size, 3)).cuda()
    l0 = dec.forward(prompt, 0).clone()
    first = int(l0.float().argmax().item())
    a = dec.forward(torch.tensor([first], dtype=torch.int32, device="cuda"), 300).clone()
    b = dec.forward(torch.tensor([first], dtype=torch.int32, device="cuda"), 300).clone()
    assert torch.equal(a, b), "a repeated step must rewrite the same cache slot and logits"
    want, tok, pos = [], first, 300
    for _ in range(10):
        tok = int(dec.forward(torch.tensor([tok], dtype=torch.int32, device="cuda"), pos).float().argmax().item())
        want.append(tok)
        pos += 1
    dec.reset()
    l1 = dec.forward(prompt, 0).clone()
    assert torch.equal(l0, l1), "reset + prefill must reproduce the logits"
    got, _ = dec.generate(first, 300, 10)
    assert got == want
    # up to the last cache position (four active attention splits), and not beyond it
    long_prompt = torch.from_numpy(toks(500, cfg.vocab_size, 5)).cuda()
    dec.reset()
    f2 = int(dec.forward(long_prompt, 0).float().argmax().item())
    got2, _ = dec.generate(f2, 500, 12)                       # positions 500..511
    want2, tok, pos = [], f2, 500
    dec.reset()
    dec.forward(long_prompt, 0)
    for _ in range(12):
        tok = int(dec.forward(torch.tensor([tok], dtype=torch.int32, device="cuda"), pos).float().argmax().item())
        want2.append(tok)
        pos += 1
    assert got2 == want2
    with pytest.raises(tl.TllmError):
        dec.generate(f2, 500, 13)
    # the FP16 single-token path stays close to the INT8 one on the same model
    dec.reset()
    dec.forward(prompt, 0)
    a = dec.forward(torch.tensor([first], dtype=torch.int32, device="cuda"), 300).clone()
    dec16 = tl.Decoder(model, int8_decode=False)
    dec16.forward(prompt, 0)
    c = dec16.forward(torch.tensor([first], dtype=torch.int32, device="cuda"), 300).float()
    assert (c - a.float()).abs().max().item() <= 0.15 * max(1.0, a.float().abs().max().item())
    tl.check_device_errors()
    dec.close()
    dec16.close()


def test_create_rejects_bad_models():
    cfg = cfg_small()
    model = tf.random_model(cfg, seed=1)
    model.layers[0]["q_proj"].sign_masks = model.layers[0]["q_proj"].sign_masks.copy()
    model.layers[0]["q_proj"].sign_masks[0, 0] |= ~model.layers[0]["q_proj"].nonzero_masks[0, 0]
    if (model.layers[0]["q_proj"].sign_masks[0, 0] & ~model.layers[0]["q_proj"].nonzero_masks[0, 0]) != 0:
        with pytest.raises(tl.TllmError) as e:
            tl.Decoder(model)
        assert e.value.status == -8


HAVE = all(os.path.exists(os.path.join(os.path.dirname(cpu.DROPIN_TEST), n)) for n in ("engine_ref", "engine_full"))


@pytest.mark.skipif(not HAVE, reason="engine binaries not built (needs the reference checkout)")
def test_reference_engine_with_every_operator_from_this_library():
    """The reference's transformer.cpp and model.cpp, unmodified, with none of its kernels."""
    cfg = tf.TllmConfig(**e2e.ARCHS["tiny"])
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "tiny.tllm")
        tf.write_tllm(path, tf.random_model(cfg, seed=7))
        res = e2e.run_engines(path, 1, 6, d, names=("engine_ref", "engine_full"))     # single-token steps only
        a, b = res["engine_ref"][1], res["engine_full"][1]
        assert np.isfinite(b).all()
        assert res["engine_ref"][0]["last_token"] == res["engine_full"][0]["last_token"]
        assert close(b, a, 5e-2)
        # a multi-token prefill: the reference's own attention kernel does not compute a softmax
        # there, so only this library's result is checked, against the oracle
        res = e2e.run_engines(path, 24, 0, d, names=("engine_full",))
        model = tf.read_tllm(path)
        want = LO.Transformer(model).forward(list(e2e.prompt_tokens(24, cfg.vocab_size)), 0)
        assert close(res["engine_full"][1], want, 3e-2)
