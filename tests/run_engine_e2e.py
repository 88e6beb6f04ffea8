#!/usr/bin/env python3
"""End-to-end decode of a random-init ternary model through the REFERENCE engine's own
Model/Transformer code (oracle/engine_main.cpp), once with the reference's ternary kernels
and once with libtllm_b200.so in their place.  Not a pytest module; run on a GPU machine:

    python tests/run_engine_e2e.py [--arch 1b|tiny] [--prompt 512] [--decode 128]

`1b` is the LLaMA-3.2-1B architecture of the benchmark definition (16 layers, hidden 2048,
32/8 heads of 64, intermediate 8192, vocab 128256, FP16 embedding and lm_head); the weights
are seeded random (W = 0.02*randn, ternarised per 128).  Prints both engines' timing lines
and the agreement of their final logits."""
import argparse
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from ternary_llm_b200 import tllm_format as tf  # noqa: E402

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


def own_decoder(path, n_prompt, n_decode, res):
    """The library's decoder on the same model and prompt: prefill, then the decode loop
    replayed as a CUDA graph (tllm_b200_decoder_generate)."""
    import torch

    import ternary_llm_b200 as tl
    model = tf.read_tllm(path)
    dec = tl.Decoder(model, int8_decode=True)
    prompt = torch.from_numpy(prompt_tokens(n_prompt, model.config.vocab_size)).cuda()
    dec.forward(prompt, 0)                       # warm-up (lazy set-up), then the timed pass
    torch.cuda.synchronize()
    dec.reset()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    logits = dec.forward(prompt, 0)
    e1.record()
    torch.cuda.synchronize()
    first = int(logits.float().argmax().item())
    last = first
    fields = {"prefill_ms": f"{e0.elapsed_time(e1):.3f}", "tok_per_s": "0", "last_token": str(first)}
    if n_decode > 0:
        dec.generate(first, n_prompt, min(4, n_decode))          # captures the step graph
        dec.reset()
        dec.forward(prompt, 0)
        toks, ms = dec.generate(first, n_prompt, n_decode)
        last = toks[-1]
        fields.update(decode_ms=f"{ms * n_decode:.3f}", tok_per_s=f"{1e3 / ms:.2f}", last_token=str(last))
        # logits after the last generated token's predecessor: rerun the last step eagerly
        lg = dec.forward(torch.tensor([toks[-2] if n_decode > 1 else first], dtype=torch.int32, device="cuda"),
                         n_prompt + n_decode - 1)
        logits = lg
    res["tllm_decoder"] = (fields, logits.float().cpu().numpy())
    dec.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", default="1b", choices=sorted(ARCHS))
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--decode", type=int, default=128)
    ap.add_argument("--full", action="store_true",
                    help="also run engine_full (every operator from libtllm_b200.so) and the library's own decoder")
    args = ap.parse_args()
    cfg = tf.TllmConfig(**ARCHS[args.arch])
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "model.tllm")
        t0 = time.time()
        tf.write_tllm(path, tf.random_model(cfg, seed=2026))
        print(f"wrote {path}: {os.path.getsize(path) / 1e6:.1f} MB in {time.time() - t0:.1f} s", flush=True)
        names = ("engine_ref", "engine_tllm") + (("engine_full",) if args.full else ())
        res = run_engines(path, args.prompt, args.decode, d, names)
        if args.full:
            own_decoder(path, args.prompt, args.decode, res)
    for name, (fields, _) in res.items():
        print(name, fields)
    a, b = res["engine_ref"][1], res["engine_tllm"][1]
    print(f"final logits: max |ref - tllm| = {np.abs(a - b).max():.4g}, max |ref| = {np.abs(a).max():.4g}, "
          f"same last token: {res['engine_ref'][0]['last_token'] == res['engine_tllm'][0]['last_token']}")
    r, t = float(res["engine_ref"][0]["tok_per_s"]), float(res["engine_tllm"][0]["tok_per_s"])
    if r > 0:
        print(f"decode tok/s: reference kernels {r:.1f}, libtllm_b200 {t:.1f}  ({t / r:.2f}x); "
              f"prefill ms: {res['engine_ref'][0]['prefill_ms']} vs {res['engine_tllm'][0]['prefill_ms']}")
    for name in ("engine_full", "tllm_decoder"):
        if name in res:
            c = res[name][1]
            print(f"{name}: max |ref - {name}| = {np.abs(a - c).max():.4g}, last token {res[name][0]['last_token']}, "
                  f"tok/s {res[name][0]['tok_per_s']}, prefill ms {res[name][0]['prefill_ms']}")


if __name__ == "__main__":
    main()
