"""Grouped-query attention over the cache, as a mixer: fused q/k/v projection, per-head
RMSNorm of q and k (when the spec names their weights), position encoding, keys and values
into the cache line, causal attention with an optional window, output projection added into
the residual. The steps are the reference's ``AttentionBlock`` (``decoder.pas:2625-2702``);
head h reads KV head h div (heads div kv_heads) (``backend.cpu.pas:1253``).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..errors import ConfigError, KernelError
from .base import MIXERS, CacheNeed, Part, TensorNeed
from .linear import Linear


class GqaAttention(Part):
    capturable = True

    def __init__(self, spec, prefix: str = "", positions=None):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.hd = int(p["heads"]), int(p["kv_heads"]), int(p["head_dim"])
        if self.nkv <= 0 or self.nh % self.nkv:
            raise ConfigError(f"{self.nh} heads on {self.nkv} KV heads")
        self.window = int(p.get("window", 0))
        self.scale = float(p["scale"])
        self.head_norm_eps = p.get("head_norm_eps")
        self.names = {k: prefix + v for k, v in p["names"].items()}
        self.position = (positions or {}).get(p.get("position", ""))
        if p.get("position") and self.position is None:
            raise ConfigError(f"the mixer names the position encoding \"{p['position']}\", "
                              "which the model does not define")
        self.qw, self.kvw = self.nh * self.hd, self.nkv * self.hd

    def tensors(self) -> List[TensorNeed]:
        n = self.names
        out = [TensorNeed(n["q"], (self.qw, self.hidden)),
               TensorNeed(n["k"], (self.kvw, self.hidden)),
               TensorNeed(n["v"], (self.kvw, self.hidden)),
               TensorNeed(n["o"], (self.hidden, self.qw))]
        if "q_norm" in n:
            out += [TensorNeed(n["q_norm"], (self.hd,), "vector"),
                    TensorNeed(n["k_norm"], (self.hd,), "vector")]
        return out

    def cache_need(self) -> CacheNeed:
        return CacheNeed(self.nkv, self.hd, self.window)

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        if self.hd % 16 or self.hd > 256:
            raise KernelError(
                f"heads of {self.hd} values are not supported by the attention kernels "
                "(a multiple of 16, at most 256)")
        n = self.names
        wq, wk, wv = weights[n["q"]], weights[n["k"]], weights[n["v"]]
        if wq.dtype == wk.dtype == wv.dtype:
            # one product for q, k and v: the rows of the three weights one after another
            self.qkv = Linear(torch.cat([wq, wk, wv], dim=0), rt)
            self.q_only = Linear(self.qkv.weight[:self.qw], rt)
            self.split = None
            if getattr(rt, "consume_weights", False):
                # the engine owns the tensors: the three originals go as soon as they are fused,
                # so that loading never holds much more than the model
                del wq, wk, wv
                for key in ("q", "k", "v"):
                    weights.pop(n[key], None)
        else:
            self.qkv = None
            self.split = [Linear(wq, rt), Linear(wk, rt), Linear(wv, rt)]
            self.q_only = self.split[0]
        self.o = Linear(weights[n["o"]], rt)
        self.q_norm = weights.get(n.get("q_norm", ""))
        self.k_norm = weights.get(n.get("k_norm", ""))

    def forward(self, h, x, step, line, state, writes_cache: bool):
        """Adds the mixer's output into x, or returns it as ``Pending`` split sums for the next
        norm to add (a decode step whose output product splits K)."""
        from .linear import Pending
        T = h.shape[0]
        nkv = self.nkv if writes_cache else 0
        width = self.qw + 2 * nkv * self.hd
        eps = float(self.head_norm_eps) if self.head_norm_eps is not None else 0.0
        inv_freq, rot_dim = (self.position.frequencies() if self.position is not None
                             else (None, 0))
        split_ok = (writes_cache and self.qkv is not None and rot_dim == self.hd
                    and self.hd in (64, 128, 256) and self.rt.dtype == torch.bfloat16)
        qkv = self.qkv(h, defer=True) if split_ok else None
        if isinstance(qkv, Pending):
            # the kernel that norms and rotates q and k adds the split sums up as it reads them
            q = torch.empty((T, self.qw), dtype=self.rt.dtype, device=h.device)
            K.qk_norm_rope_store(None, self.q_norm, self.k_norm, eps, inv_freq, rot_dim, step,
                                 line, self.nh, nkv, self.hd, True, partial=qkv.partial, q_out=q)
            attn = torch.empty((T, self.qw), dtype=self.rt.dtype, device=h.device)
            self.rt.attention(q, self.qw, attn, step, line, self.nh, self.nkv, self.hd,
                              self.window, self.scale)
            out = self.o(attn, add_into=x, defer=True)
            return out if isinstance(out, Pending) else None
        if qkv is not None:
            pass
        elif not writes_cache:
            qkv = self.q_only(h)
        elif self.qkv is not None:
            qkv = self.qkv(h)
        else:
            qkv = torch.empty((T, width), dtype=self.rt.dtype, device=h.device)
            self.split[0](h, out=qkv[:, :self.qw])
            self.split[1](h, out=qkv[:, self.qw:self.qw + self.kvw])
            self.split[2](h, out=qkv[:, self.qw + self.kvw:])
        K.qk_norm_rope_store(qkv, self.q_norm, self.k_norm, eps, inv_freq, rot_dim,
                             step, line, self.nh, nkv, self.hd, writes_cache)
        attn = torch.empty((T, self.qw), dtype=self.rt.dtype, device=h.device)
        self.rt.attention(qkv, width, attn, step, line, self.nh, self.nkv, self.hd,
                          self.window, self.scale)
        out = self.o(attn, add_into=x, defer=True)
        return out if isinstance(out, Pending) else None


MIXERS.register("gqa_attention", GqaAttention)
