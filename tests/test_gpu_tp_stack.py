"""The tensor-parallel layer stack (ternary_llm_b200/tp_stack.py) on one GPU: with a single
rank it is the reference's layer loop on this library's kernels, so its residual stream,
pushed through the oracle's final norm and lm_head, must give the oracle's logits token by
token.  (The exchange between ranks is covered by tests/test_gpu_tp_allreduce.py on two
GPUs; the split of heads and columns over ranks by tests/test_tp_cpu.py.)"""
import numpy as np
import pytest
import torch

from oracle import layer_oracle as LO
from ternary_llm_b200 import tllm_format as tf
from ternary_llm_b200.tp_stack import StackConfig, TpLayerStack, layer_sources_from_model

pytestmark = pytest.mark.gpu


def _model():
    cfg = tf.TllmConfig(vocab_size=512, hidden_dim=256, intermediate_dim=512, n_layers=3, n_heads=4, n_kv_heads=2,
                        head_dim=64, max_seq_len=48, rope_theta=10000.0, rms_norm_eps=1e-5)
    return cfg, tf.random_model(cfg, seed=21)


def _logits(model, res):
    h, _ = LO.rmsnorm(res.astype(np.float16)[None, :], model.final_norm, model.config.rms_norm_eps)
    return LO.fp16_gemv(model.lm_head, h[0])


@pytest.mark.parametrize("batch", [1, 3])
def test_single_rank_stack_matches_the_layer_oracle(batch):
    cfg, model = _model()
    dev = torch.device("cuda", 0)
    sc = StackConfig(hidden=cfg.hidden_dim, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                     intermediate=cfg.intermediate_dim, max_seq_len=cfg.max_seq_len, rope_theta=cfg.rope_theta,
                     rms_norm_eps=cfg.rms_norm_eps)
    stack = TpLayerStack(sc, layer_sources_from_model(model, 0, 1, dev), 0, 1, dev, allreduce="none", batch=batch)
    emb = torch.from_numpy(model.embedding).to(dev)
    rng = np.random.default_rng(batch)
    seqs = rng.integers(0, cfg.vocab_size, (batch, 6))
    oracles = [LO.Transformer(model, int8_decode=False) for _ in range(batch)]
    for pos in range(seqs.shape[1]):
        x = emb[torch.from_numpy(seqs[:, pos]).to(dev)].contiguous()
        res = stack.step(x, pos).float().cpu().numpy()
        assert np.isfinite(res).all()
        for b in range(batch):
            want = oracles[b].forward([int(seqs[b, pos])], pos).astype(np.float32)
            got = _logits(model, res[b]).astype(np.float32)
            assert np.abs(got - want).max() <= 4e-2 * max(1.0, np.abs(want).max()), f"position {pos}, sequence {b}"
    with pytest.raises(ValueError):
        stack.step(x, cfg.max_seq_len)
