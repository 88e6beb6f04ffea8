"""Host-side mirror of the reference's Transformer (include/transformer.h:15-27) on the
library's decoder (include/tllm_b200_layer.h): construct from a model, forward(token ids,
start_pos) -> logits of the last token, reset(), and generate() for the greedy decode loop
replayed as a CUDA graph.  The model's tensors are uploaded with torch; every operator runs
in libtllm_b200.so.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib
from .tllm_format import PROJ_NAMES, TernaryTensor, TllmFile, read_tllm


class _DevArray:
    """Zero-copy view of device memory for torch.as_tensor."""

    def __init__(self, ptr: int, n: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}


class Decoder:
    def __init__(self, model, device=None, int8_decode: bool = True, max_batch: int = 1):
        """max_batch > 1: room for that many independent sequences, each with its own KV cache
        (forward_seq for one of them, forward_batch for a lock-step decode of several)."""
        if isinstance(model, str):
            model = read_tllm(model)
        assert isinstance(model, TllmFile)
        self.config = cfg = model.config
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._keep = []          # tensors the decoder keeps pointers to (embedding, norms, FP16 lm_head)
        staging = []             # ternary source arrays, needed only until create() has repacked them

        def up(a, keep=True):
            if isinstance(a, torch.Tensor):          # already on the device (synth.random_device_model)
                t = a.to(self.device).contiguous()
            else:
                a = np.array(a)  # copy: file views are read-only maps
                if a.dtype == np.uint32:
                    a = a.view(np.int32)
                t = torch.from_numpy(a).to(self.device)
            (self._keep if keep else staging).append(t)
            return t.data_ptr()

        def tern(t: TernaryTensor):
            rows, cols = t.shape
            return _lib.TernaryWeightDesc(up(t.nonzero_masks, False), up(t.sign_masks, False), up(t.scales, False),
                                          rows, cols)

        layers = (_lib.LayerWeightsDesc * cfg.n_layers)()
        for i, layer in enumerate(model.layers):
            for name in PROJ_NAMES:
                setattr(layers[i], name, tern(layer[name]))
            layers[i].attn_norm_weight = up(layer["attn_norm"])
            layers[i].ffn_norm_weight = up(layer["ffn_norm"])
        d = _lib.ModelDesc()
        d.vocab_size, d.hidden_dim, d.intermediate_dim = cfg.vocab_size, cfg.hidden_dim, cfg.intermediate_dim
        d.n_layers, d.n_heads, d.n_kv_heads = cfg.n_layers, cfg.n_heads, cfg.n_kv_heads
        d.max_seq_len, d.head_dim, d.group_size = cfg.max_seq_len, cfg.head_dim, cfg.group_size
        d.rope_theta, d.rms_norm_eps = cfg.rope_theta, cfg.rms_norm_eps
        d.embedding_table = up(model.embedding)
        d.final_norm_weight = up(model.final_norm)
        if cfg.lm_head_ternary:
            d.lm_head_weight = None
            d.lm_head_ternary = tern(model.lm_head)
        else:
            d.lm_head_weight = up(model.lm_head)
        d.layers = layers
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            _lib.check(_lib.lib().tllm_b200_decoder_create_batched(ctypes.byref(d), 1 if int8_decode else 0,
                                                                   max_batch, ctypes.byref(handle)))
        self._h = handle
        self.max_batch = max_batch
        del staging

    def reset(self) -> None:
        _lib.check(_lib.lib().tllm_b200_decoder_reset(self._h, torch.cuda.current_stream().cuda_stream))

    @staticmethod
    def _check_tokens(token_ids):
        if not (token_ids.is_cuda and token_ids.dtype == torch.int32 and token_ids.is_contiguous()):
            raise TypeError("token_ids must be a contiguous int32 CUDA tensor")

    def forward(self, token_ids, start_pos: int) -> torch.Tensor:
        """token_ids: int32 CUDA tensor [n]; returns the FP16 logits of the last token
        (a view of the decoder's buffer, overwritten by the next call)."""
        return self.forward_seq(0, token_ids, start_pos)

    def forward_seq(self, seq: int, token_ids, start_pos: int) -> torch.Tensor:
        """forward for sequence `seq` of a batched decoder (its own KV cache)."""
        self._check_tokens(token_ids)
        out = ctypes.c_void_p()
        _lib.check(_lib.lib().tllm_b200_decoder_forward_seq(self._h, seq, token_ids.data_ptr(), token_ids.numel(),
                                                            start_pos, ctypes.byref(out),
                                                            torch.cuda.current_stream().cuda_stream))
        return torch.as_tensor(_DevArray(out.value, self.config.vocab_size, "<f2"), device=self.device)

    def forward_batch(self, token_ids, pos: int) -> torch.Tensor:
        """One lock-step decode step: token_ids[b] is the next token of sequence b, all at cache
        position pos.  Returns FP16 logits [batch, vocab] (a view of the decoder's buffer)."""
        self._check_tokens(token_ids)
        b = token_ids.numel()
        out = ctypes.c_void_p()
        _lib.check(_lib.lib().tllm_b200_decoder_forward_batch(self._h, token_ids.data_ptr(), b, pos, ctypes.byref(out),
                                                              torch.cuda.current_stream().cuda_stream))
        flat = torch.as_tensor(_DevArray(out.value, b * self.config.vocab_size, "<f2"), device=self.device)
        return flat.view(b, self.config.vocab_size)

    def generate(self, first_token: int, start_pos: int, n_steps: int):
        """Greedy continuation: returns (tokens [n_steps], ms per step measured on the device)."""
        toks = (ctypes.c_int * n_steps)()
        ms = ctypes.c_float()
        _lib.check(_lib.lib().tllm_b200_decoder_generate(self._h, int(first_token), start_pos, n_steps, toks,
                                                         ctypes.byref(ms)))
        return list(toks), ms.value

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.lib().tllm_b200_decoder_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
