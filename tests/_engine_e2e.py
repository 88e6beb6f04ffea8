"""Helpers for the tests that run the REFERENCE engine's own Model/Transformer code
(oracle/engine_main.cpp, built into oracle/_ref/ by oracle/Makefile): the model
architectures used, the prompt ids that program draws, and a runner that starts the
built executables and parses their timing line and logits file."""
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

ARCHS = {
    "1b": dict(vocab_size=128256, hidden_dim=2048, intermediate_dim=8192, n_layers=16, n_heads=32, n_kv_heads=8,
               head_dim=64, max_seq_len=1024, rope_theta=500000.0, rms_norm_eps=1e-5),
    "tiny": dict(vocab_size=4096, hidden_dim=512, intermediate_dim=1024, n_layers=2, n_heads=8, n_kv_heads=2,
                 head_dim=64, max_seq_len=256, rope_theta=500000.0, rms_norm_eps=1e-5),
}


def prompt_tokens(n, vocab):
    """The prompt ids oracle/engine_main.cpp draws: std::mt19937(1234)() % vocab."""
    bg = np.random.MT19937()
    bg._legacy_seeding(1234)
    return (bg.random_raw(n) % np.uint64(vocab)).astype(np.int32)


def run_engines(model_path, n_prompt, n_decode, workdir, names=("engine_ref", "engine_tllm")):
    out = {}
    for name in names:
        exe = os.path.join(ROOT, "oracle", "_ref", name)
        logits = os.path.join(workdir, name + ".logits")
        r = subprocess.run([exe, model_path, str(n_prompt), str(n_decode), logits], capture_output=True, text=True,
                           timeout=1200)
        line = [l for l in r.stdout.splitlines() if l.startswith("prefill_ms")]
        if r.returncode != 0 or not line:
            raise RuntimeError(f"{name} failed: {r.stdout[-500:]} {r.stderr[-1500:]}")
        fields = dict(kv.split("=", 1) for kv in line[0].split() if "=" in kv)
        out[name] = (fields, np.fromfile(logits, dtype=np.float16).astype(np.float32))
    return out
