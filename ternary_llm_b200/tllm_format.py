"""The .tllm container: header, section order, reader and a seeded random-init writer.

Layout (reference include/format.h:8-43, read by src/model.cpp:72-212, written by
ternarize/ternarize.py:73-111,254-349), little-endian:
  256-byte header: 15 x uint32 {magic 0x544C4C4D, version 1, arch, vocab, hidden,
      intermediate, n_layers, n_heads, n_kv_heads, max_seq_len, head_dim, rope_theta bits,
      group_size, rms_norm_eps bits, flags (bit 0: ternary lm_head)}, zero padded
  embedding  half [vocab, hidden]
  per layer: q, k, v, o, gate, up, down -- each as nonzero uint32 [out, in/32],
      sign uint32 [out, in/32], scales half [out, in/group] (in padded to 32) --
      then attn_norm half [hidden], ffn_norm half [hidden]
  final norm half [hidden]
  lm_head: half [vocab, hidden], or a ternary triple when flag bit 0 is set
  uint64 tokenizer length + blob (length 0 when absent)

Only the ternary projection sections feed the contraction path of this library; the
other sections are carried so that a file written here loads in the reference engine.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

from . import pack

MAGIC = 0x544C4C4D
VERSION = 1
HEADER_SIZE = 256
ARCH_LLAMA = 0
FLAG_LM_HEAD_TERNARY = 1
PROJ_NAMES = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def _f2u(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


def _u2f(x: int) -> float:
    return struct.unpack("<f", struct.pack("<I", x))[0]


def pad32(n: int) -> int:
    return (n + 31) // 32 * 32


@dataclass
class TllmConfig:
    vocab_size: int
    hidden_dim: int
    intermediate_dim: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    max_seq_len: int = 4096
    rope_theta: float = 500000.0
    group_size: int = 128
    rms_norm_eps: float = 1e-5
    lm_head_ternary: bool = False
    arch: int = ARCH_LLAMA

    def __post_init__(self):
        # the file stores these two as float32
        self.rope_theta = _u2f(_f2u(self.rope_theta))
        self.rms_norm_eps = _u2f(_f2u(self.rms_norm_eps))

    def proj_shapes(self):
        """(name, out_features, in_features padded to 32) in file order (src/model.cpp:139-153)."""
        q, kv = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        h, i = self.hidden_dim, self.intermediate_dim
        return [("q_proj", q, pad32(h)), ("k_proj", kv, pad32(h)), ("v_proj", kv, pad32(h)),
                ("o_proj", h, pad32(q)), ("gate_proj", i, pad32(h)), ("up_proj", i, pad32(h)),
                ("down_proj", h, pad32(i))]

    def pack_header(self) -> bytes:
        flags = FLAG_LM_HEAD_TERNARY if self.lm_head_ternary else 0
        raw = struct.pack("<15I", MAGIC, VERSION, self.arch, self.vocab_size, self.hidden_dim,
                          self.intermediate_dim, self.n_layers, self.n_heads, self.n_kv_heads,
                          self.max_seq_len, self.head_dim, _f2u(self.rope_theta), self.group_size,
                          _f2u(self.rms_norm_eps), flags)
        return raw + b"\x00" * (HEADER_SIZE - len(raw))

    @staticmethod
    def unpack_header(raw: bytes) -> "TllmConfig":
        if len(raw) < HEADER_SIZE:
            raise ValueError("short header")
        f = struct.unpack("<15I", raw[:60])
        if f[0] != MAGIC:
            raise ValueError(f"bad magic 0x{f[0]:08X}")
        if f[1] != VERSION:
            raise ValueError(f"unsupported version {f[1]}")
        return TllmConfig(arch=f[2], vocab_size=f[3], hidden_dim=f[4], intermediate_dim=f[5], n_layers=f[6],
                          n_heads=f[7], n_kv_heads=f[8], max_seq_len=f[9], head_dim=f[10],
                          rope_theta=_u2f(f[11]), group_size=f[12], rms_norm_eps=_u2f(f[13]),
                          lm_head_ternary=bool(f[14] & FLAG_LM_HEAD_TERNARY))


def ternary_bytes(out_f: int, in_f: int, gs: int) -> int:
    return 2 * out_f * (in_f // 32) * 4 + out_f * (in_f // gs) * 2


def expected_size(cfg: TllmConfig, tokenizer_bytes: int = 0) -> int:
    n = HEADER_SIZE + cfg.vocab_size * cfg.hidden_dim * 2
    per_layer = sum(ternary_bytes(o, i, cfg.group_size) for _, o, i in cfg.proj_shapes()) + 2 * cfg.hidden_dim * 2
    n += per_layer * cfg.n_layers + cfg.hidden_dim * 2
    n += ternary_bytes(cfg.vocab_size, pad32(cfg.hidden_dim), cfg.group_size) if cfg.lm_head_ternary \
        else cfg.vocab_size * cfg.hidden_dim * 2
    return n + 8 + tokenizer_bytes


@dataclass
class TernaryTensor:
    nonzero_masks: np.ndarray     # uint32 [out, in/32]
    sign_masks: np.ndarray        # uint32 [out, in/32]
    scales: np.ndarray            # float16 [out, in/group]

    @property
    def shape(self):
        return self.nonzero_masks.shape[0], self.nonzero_masks.shape[1] * 32


@dataclass
class TllmFile:
    config: TllmConfig
    embedding: np.ndarray
    layers: list = field(default_factory=list)      # dicts: 7 TernaryTensor + attn_norm, ffn_norm
    final_norm: np.ndarray = None
    lm_head: object = None                          # float16 array or TernaryTensor
    tokenizer: bytes = b""


def _write_ternary(f, t: TernaryTensor):
    f.write(np.ascontiguousarray(t.nonzero_masks, "<u4").tobytes())
    f.write(np.ascontiguousarray(t.sign_masks, "<u4").tobytes())
    f.write(np.ascontiguousarray(t.scales, "<f2").tobytes())


def write_tllm(path: str, m: TllmFile) -> None:
    cfg = m.config
    with open(path, "wb") as f:
        f.write(cfg.pack_header())
        f.write(np.ascontiguousarray(m.embedding, "<f2").tobytes())
        for layer in m.layers:
            for name in PROJ_NAMES:
                _write_ternary(f, layer[name])
            f.write(np.ascontiguousarray(layer["attn_norm"], "<f2").tobytes())
            f.write(np.ascontiguousarray(layer["ffn_norm"], "<f2").tobytes())
        f.write(np.ascontiguousarray(m.final_norm, "<f2").tobytes())
        if cfg.lm_head_ternary:
            _write_ternary(f, m.lm_head)
        else:
            f.write(np.ascontiguousarray(m.lm_head, "<f2").tobytes())
        f.write(struct.pack("<Q", len(m.tokenizer)))
        f.write(m.tokenizer)


def read_tllm(path: str) -> TllmFile:
    """Memory-maps the file; every array is a view into it."""
    buf = np.memmap(path, dtype=np.uint8, mode="r")
    cfg = TllmConfig.unpack_header(bytes(buf[:HEADER_SIZE]))
    if cfg.group_size <= 0 or cfg.group_size % 32:
        raise ValueError(f"bad group size {cfg.group_size}")
    pos = HEADER_SIZE

    def take(dtype, shape):
        nonlocal pos
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        if pos + n > buf.size:
            raise ValueError("file is shorter than its header implies")
        a = buf[pos:pos + n].view(dtype).reshape(shape)
        pos += n
        return a

    def take_ternary(out_f, in_f):
        return TernaryTensor(take("<u4", (out_f, in_f // 32)), take("<u4", (out_f, in_f // 32)),
                             take("<f2", (out_f, in_f // cfg.group_size)))

    m = TllmFile(cfg, take("<f2", (cfg.vocab_size, cfg.hidden_dim)))
    for _ in range(cfg.n_layers):
        layer = {name: take_ternary(o, i) for name, o, i in cfg.proj_shapes()}
        layer["attn_norm"] = take("<f2", (cfg.hidden_dim,))
        layer["ffn_norm"] = take("<f2", (cfg.hidden_dim,))
        m.layers.append(layer)
    m.final_norm = take("<f2", (cfg.hidden_dim,))
    m.lm_head = take_ternary(cfg.vocab_size, pad32(cfg.hidden_dim)) if cfg.lm_head_ternary \
        else take("<f2", (cfg.vocab_size, cfg.hidden_dim))
    if pos + 8 <= buf.size:
        n = struct.unpack("<Q", bytes(buf[pos:pos + 8]))[0]
        pos += 8
        m.tokenizer = bytes(buf[pos:pos + n])
    return m


def random_model(cfg: TllmConfig, seed: int, std: float = 0.02) -> TllmFile:
    """Seeded random-init model with the benchmark's weight distribution (W = std*randn,
    ternarised per group; norms = 1; FP16 embedding / lm_head = std*randn)."""
    rng = np.random.default_rng(seed)
    m = TllmFile(cfg, (rng.standard_normal((cfg.vocab_size, cfg.hidden_dim), dtype=np.float32) * std).astype(np.float16))
    for li in range(cfg.n_layers):
        layer = {}
        for pi, (name, o, i) in enumerate(cfg.proj_shapes()):
            nz, sg, sc = pack.random_ternary_weight(o, i, seed=seed * 100003 + li * 16 + pi, std=std)
            layer[name] = TernaryTensor(nz, sg, sc)
        layer["attn_norm"] = np.ones(cfg.hidden_dim, np.float16)
        layer["ffn_norm"] = np.ones(cfg.hidden_dim, np.float16)
        m.layers.append(layer)
    m.final_norm = np.ones(cfg.hidden_dim, np.float16)
    if cfg.lm_head_ternary:
        nz, sg, sc = pack.random_ternary_weight(cfg.vocab_size, pad32(cfg.hidden_dim), seed=seed * 100003 + 99991, std=std)
        m.lm_head = TernaryTensor(nz, sg, sc)
    else:
        m.lm_head = (rng.standard_normal((cfg.vocab_size, cfg.hidden_dim), dtype=np.float32) * std).astype(np.float16)
    return m


TP_COLUMN = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")   # output rows are split
TP_ROW = ("o_proj", "down_proj")                                      # input columns are split
TP_GROUPS = (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj"))  # share their input vector


def shard_ternary(t: TernaryTensor, name: str, rank: int, world: int, group_size: int = 128) -> TernaryTensor:
    """The part of projection `name` that rank `rank` of `world` tensor-parallel ranks holds.

    q, k, v, gate and up are column-parallel: a contiguous range of output rows of all three
    arrays (a pointer offset in the file's layout).  o and down are row-parallel: a range of
    input columns on group boundaries, i.e. strided slices of all three arrays; their partial
    results are summed across ranks.  The shards are views of `t`."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    rows, cols = t.shape
    if world == 1:
        return t
    if name in TP_COLUMN:
        if rows % world:
            raise ValueError(f"{name}: {rows} rows do not split over {world} ranks")
        r0, r1 = rank * (rows // world), (rank + 1) * (rows // world)
        return TernaryTensor(t.nonzero_masks[r0:r1], t.sign_masks[r0:r1], t.scales[r0:r1])
    if name in TP_ROW:
        if cols % (world * group_size):
            raise ValueError(f"{name}: {cols} columns do not split over {world} ranks on {group_size}-column groups")
        k0, k1 = rank * (cols // world), (rank + 1) * (cols // world)
        return TernaryTensor(t.nonzero_masks[:, k0 // 32:k1 // 32], t.sign_masks[:, k0 // 32:k1 // 32],
                             t.scales[:, k0 // group_size:k1 // group_size])
    raise ValueError(f"unknown projection {name}")


class _PinnedStager:
    """Host-to-device copies through two page-locked buffers used in turn: the copy of one
    array runs while the host gathers the next one (a row-parallel shard is a strided slice
    of the memory-mapped file) into the other buffer."""

    def __init__(self, torch, device, nbytes: int):
        self.torch, self.device = torch, device
        self.bufs = [torch.empty(max(nbytes, 16), dtype=torch.uint8).pin_memory() for _ in range(2)]
        self.events = [None, None]
        self.turn = 0

    def to_device(self, a: np.ndarray):
        torch = self.torch
        i, self.turn = self.turn, self.turn ^ 1
        if self.events[i] is not None:
            self.events[i].synchronize()          # the buffer's previous copy has left it
        n = a.nbytes
        host = self.bufs[i][:n]
        np.copyto(host.numpy().view(a.dtype).reshape(a.shape), a)
        dt = {"uint32": torch.int32, "float16": torch.float16}[a.dtype.name]
        with torch.cuda.device(self.device):      # the event must belong to the target device's stream
            out = torch.empty(a.shape, dtype=dt, device=self.device)
            out.view(torch.uint8).reshape(-1).copy_(host, non_blocking=True)
            self.events[i] = torch.cuda.Event()
            self.events[i].record()
        return out


def load_projections(path: str, device, register: bool = False, rank: int = 0, world: int = 1,
                     verify: bool = False, grouped: bool = False):
    """Reads a .tllm file and prepares every ternary projection on `device` for the
    streaming kernels (the load-time repack).  Returns (config, layers) where layers[i]
    maps a projection name to an ops.PreparedWeight.  Projections whose input width is
    not a multiple of 128 are rejected by the library (TllmError).

    rank, world: load only this tensor-parallel rank's shard of every projection
        (shard_ternary); nothing of the other ranks' parts is copied to the device.
    verify: unpack every prepared matrix again and compare it bit for bit with what was read.
    grouped: pack q|k|v and gate|up back to back, so that ternary_gemv_packed_multi runs
        each group as one launch (ops.prepare_group).
    The arrays go to the device through page-locked staging buffers."""
    import torch

    from . import ops
    if register and grouped:
        raise ValueError("grouped weights are not registered under their source arrays")
    m = read_tllm(path)
    gs = m.config.group_size
    shards = [{name: shard_ternary(layer[name], name, rank, world, gs) for name in PROJ_NAMES} for layer in m.layers]
    biggest = max(t.nonzero_masks.size * 4 for d in shards for t in d.values()) if shards else 0
    stager = _PinnedStager(torch, torch.device(device), biggest)

    def device_arrays(t):
        rows, cols = t.shape
        return (stager.to_device(t.nonzero_masks), stager.to_device(t.sign_masks), stager.to_device(t.scales),
                rows, cols)

    def check(w, src, what):
        nz, sg, sc = w.unpack()
        if not (torch.equal(nz, src[0]) and torch.equal(sg, src[1])
                and torch.equal(sc.view(torch.int16), src[2].view(torch.int16))):
            raise ValueError(f"{what}: the prepared matrix does not unpack to the arrays of the file")

    out = []
    # the library's kernels run on the CURRENT device: make the target device current for the
    # repack launches (and for the staging copies' events)
    with torch.cuda.device(torch.device(device)):
        for li, layer in enumerate(shards):
            d = {}
            todo = list(PROJ_NAMES)
            if grouped:
                for names in TP_GROUPS:
                    srcs = [device_arrays(layer[n]) for n in names]
                    for n, w, src in zip(names, ops.prepare_group(srcs), srcs):
                        d[n] = w
                        if verify:
                            check(w, src, f"layer {li} {n}")
                        todo.remove(n)
            for name in todo:
                src = device_arrays(layer[name])
                d[name] = ops.PreparedWeight(*src, register=register, keep_source=register)
                if verify:
                    check(d[name], src, f"layer {li} {name}")
            out.append(d)
    torch.cuda.synchronize(torch.device(device))
    return m.config, out
