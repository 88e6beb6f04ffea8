"""One rank's share of a LLaMA-style decoder layer stack under tensor parallelism
(the reference's layer loop, src/transformer.cpp:196-292, split over GPUs):

    q, k, v, gate, up   column-parallel: a rank holds n_heads/world query heads, n_kv_heads/world
                        KV heads (with their slice of the KV cache) and intermediate/world rows;
    o, down             row-parallel: a rank multiplies its slice of the input columns and the
                        partial vectors are summed over ranks -- by the GEMV kernel itself over
                        peer memory (ternary_gemv_packed_allreduce, one vector), or by a library
                        all-reduce of the FP16 result (several vectors, or on request).

The residual stream is replicated: every rank holds the full hidden vector and does the
(cheap) norms and residual adds itself.  Attention needs no exchange: a rank's query heads
only read the KV heads it holds.  One process per GPU; this class only sequences calls into
the C ABI on torch's current stream, so a whole step can be captured in a CUDA graph.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import layer_ops as L
from . import ops

_H = torch.float16


@dataclass
class StackConfig:
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    intermediate: int
    max_seq_len: int
    rope_theta: float = 500000.0
    rms_norm_eps: float = 1e-5

    def shard_shapes(self, world: int):
        """(name, rows, cols) of one rank's projections."""
        if self.n_heads % world or self.n_kv_heads % world or self.intermediate % world:
            raise ValueError(f"heads {self.n_heads}/{self.n_kv_heads} and intermediate {self.intermediate} "
                             f"must divide by the {world} ranks")
        q, kv = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        return [("q", q // world, self.hidden), ("k", kv // world, self.hidden), ("v", kv // world, self.hidden),
                ("o", self.hidden, q // world), ("gate", self.intermediate // world, self.hidden),
                ("up", self.intermediate // world, self.hidden), ("down", self.hidden, self.intermediate // world)]


def layer_sources_from_model(model, rank: int, world: int, device):
    """This rank's shards of a loaded model (tllm_format.TllmFile), layer by layer, in the form
    TpLayerStack takes: column shards are row ranges of the arrays, row shards column ranges on
    scale-group boundaries (tllm_format.shard_ternary)."""
    import numpy as np

    from . import tllm_format as tf

    def dev(a):
        a = np.ascontiguousarray(a)
        return torch.from_numpy(a.view(np.int32) if a.dtype == np.uint32 else a).to(device)

    for layer in model.layers:
        out = {"attn_norm": dev(layer["attn_norm"]), "ffn_norm": dev(layer["ffn_norm"])}
        for name in ("q", "k", "v", "o", "gate", "up", "down"):
            t = tf.shard_ternary(layer[name + "_proj"], name + "_proj", rank, world)
            out[name] = (dev(t.nonzero_masks), dev(t.sign_masks), dev(t.scales))
        yield out


class TpLayerStack:
    """layers: per layer a dict with this rank's shards "q","k","v","o","gate","up","down" as
    (nonzero_masks, sign_masks, scales) device tensors in the reference layout, and the FP16
    vectors "attn_norm", "ffn_norm" [hidden].  allreduce: "fused" (batch 1 only), "nccl", or
    "none" (world == 1).  `layers` may be a generator: the source arrays of a layer are repacked
    and can be dropped before the next layer is produced."""

    def __init__(self, cfg: StackConfig, layers, rank: int, world: int, device, group=None, allreduce: str = "fused",
                 batch: int = 1, weights_from: "TpLayerStack | None" = None):
        if allreduce == "fused" and batch != 1:
            raise ValueError("the fused all-reduce carries one vector; use allreduce='nccl' for a batch")
        if world == 1:
            allreduce = "none"
        self.cfg, self.rank, self.world, self.dev, self.batch = cfg, rank, world, device, batch
        self.group, self.mode = group, allreduce
        shapes = dict((n, (r, c)) for n, r, c in cfg.shard_shapes(world))
        self.hq, self.hkv = cfg.n_heads // world, cfg.n_kv_heads // world
        # weights_from: another stack of the same rank whose prepared weights are shared (layers is
        # ignored then): a second batch size on the same model
        self.layers = list(weights_from.layers) if weights_from is not None else []
        for src in (layers if weights_from is None else ()):
            def t(name):
                nz, sg, sc = src[name]
                return (nz, sg, sc) + shapes[name]
            qkv = ops.prepare_group([t("q"), t("k"), t("v")])
            o = ops.PreparedWeight(*t("o"), register=False, keep_source=False)
            gu = ops.prepare_group([t("gate"), t("up")])
            down = ops.PreparedWeight(*t("down"), register=False, keep_source=False)
            self.layers.append((qkv, o, gu, down, src["attn_norm"], src["ffn_norm"]))
        B, hd = batch, cfg.head_dim
        n = len(self.layers)
        z = lambda *s: torch.zeros(*s, dtype=_H, device=device)   # noqa: E731
        self.k_cache = z(n, B, self.hkv, cfg.max_seq_len, hd)
        self.v_cache = z(n, B, self.hkv, cfg.max_seq_len, hd)
        self.res, self.h = z(B, cfg.hidden), z(B, cfg.hidden)
        self.res2 = z(B, cfg.hidden)          # the residual stream alternates between res and res2 at batch 1
        self.q, self.k, self.v = z(B, self.hq * hd), z(B, self.hkv * hd), z(B, self.hkv * hd)
        self.attn, self.yo = z(B, self.hq * hd), z(B, cfg.hidden)
        self.g, self.u = z(B, cfg.intermediate // world), z(B, cfg.intermediate // world)
        self.act, self.yd = z(B, cfg.intermediate // world), z(B, cfg.hidden)
        self.ar = ops.FusedAllReduce(group, cfg.hidden, device) if allreduce == "fused" else None
        self.launches_per_step = 0
        self.out = self.res                   # what the last step returned

    # -- pieces -----------------------------------------------------------------------------
    def _column(self, ws, x, ys):
        if self.batch == 1:
            ops.ternary_gemv_packed_multi(ws, x, ys)        # one launch for the matrices that share x
            return 1
        for w, y in zip(ws, ys):
            self._matmul(w, x, y)
        return len(ws)

    def _matmul(self, w, x, y):
        if self.batch <= 16:
            ops.ternary_gemv_packed(w, x, y, self.batch)     # up to 8 vectors: streaming GEMV; above: tcgen05 kernel
        else:
            ops.ternary_gemm_packed(x, w, y, self.batch)

    def _row(self, w, x, y):
        if self.mode == "fused":
            ops.ternary_gemv_packed_allreduce(w, x, y, self.ar)
            return 1
        self._matmul(w, x, y)
        if self.mode == "nccl":
            import torch.distributed as dist
            dist.all_reduce(y, group=self.group)
            return 2
        return 1

    def step(self, x, pos: int):
        """One token per sequence at cache position `pos`: x [batch, hidden] FP16 (the same on
        every rank) -> the residual stream after the last layer (a view of an internal buffer)."""
        c, B, hd = self.cfg, self.batch, self.cfg.head_dim
        if pos < 0 or pos >= c.max_seq_len:
            raise ValueError(f"position {pos} outside the cache of {c.max_seq_len}")
        if B == 1:
            return self._step_one(x, pos)
        n = 0
        self.res.copy_(x.reshape(B, c.hidden))
        L.rmsnorm_forward(self.res, self.layers[0][4], self.h, None, None, B, c.hidden, c.rms_norm_eps)
        n += 2
        for li, (qkv, o, gu, down, _, ffn_norm) in enumerate(self.layers):
            n += self._column(qkv, self.h, [self.q, self.k, self.v])
            L.rope_append(self.q, self.k, self.v, self.k_cache[li], self.v_cache[li], B, 1, self.hq, self.hkv, hd,
                          pos, c.rope_theta, c.max_seq_len)
            L.attention_forward(self.q, self.k_cache[li], self.v_cache[li], self.attn, B, self.hq, self.hkv, hd,
                                1, pos + 1, c.max_seq_len)
            n += 2 + self._row(o, self.attn, self.yo)
            # res += o-projection; h = norm(res)
            L.rmsnorm_forward(self.yo, ffn_norm, self.h, self.res, self.res, B, c.hidden, c.rms_norm_eps)
            n += 1 + self._column(gu, self.h, [self.g, self.u])
            L.silu_mul_forward(self.g, self.u, self.act, self.act.numel())
            n += 1 + self._row(down, self.act, self.yd)
            if li + 1 < len(self.layers):
                L.rmsnorm_forward(self.yd, self.layers[li + 1][4], self.h, self.res, self.res, B, c.hidden,
                                  c.rms_norm_eps)
            else:
                L.add_forward(self.res, self.yd, self.res, self.res.numel())
            n += 1
        self.launches_per_step = n
        self.out = self.res
        return self.res

    def _step_one(self, x, pos: int):
        """Batch 1: six launches per layer.  The residual add and the RMSNorm in front of the
        column-parallel projections run inside their GEMV launch (ternary_gemv_packed_multi_norm),
        RoPE + cache append + attention are one launch; the residual stream alternates between
        two buffers because the fused launch must not overwrite the vector other CTAs still read."""
        c, hd = self.cfg, self.cfg.head_dim
        cur, nxt = self.res, self.res2
        cur.copy_(x.reshape(1, c.hidden))
        n = 1
        pending = None                       # the row-parallel result not yet added to the residual stream
        for li, (qkv, o, gu, down, attn_norm, ffn_norm) in enumerate(self.layers):
            if pending is None:
                ops.ternary_gemv_packed_multi_norm(qkv, cur[0], None, attn_norm, None, c.rms_norm_eps,
                                                   [self.q[0], self.k[0], self.v[0]])
            else:
                ops.ternary_gemv_packed_multi_norm(qkv, pending[0], cur[0], attn_norm, nxt[0], c.rms_norm_eps,
                                                   [self.q[0], self.k[0], self.v[0]])
                cur, nxt = nxt, cur
            L.attention_decode(self.q, self.k, self.v, self.k_cache[li], self.v_cache[li], self.attn, self.hq,
                               self.hkv, hd, pos, c.rope_theta, c.max_seq_len)
            n += 2 + self._row(o, self.attn, self.yo)
            ops.ternary_gemv_packed_multi_norm(gu, self.yo[0], cur[0], ffn_norm, nxt[0], c.rms_norm_eps,
                                               [self.g[0], self.u[0]])
            cur, nxt = nxt, cur
            L.silu_mul_forward(self.g, self.u, self.act, self.act.numel())
            n += 2 + self._row(down, self.act, self.yd)
            pending = self.yd
        L.add_forward(cur, self.yd, nxt, cur.numel())
        self.launches_per_step = n + 1
        self.out = nxt
        return nxt

    def weight_bytes(self) -> int:
        return sum(w.packed.numel() for (qkv, o, gu, down, _, _) in self.layers for w in (*qkv, o, *gu, down))
