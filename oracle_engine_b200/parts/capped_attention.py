"""Mixer `capped_attention`: grouped-query attention over the paged cache whose keys and values have head sizes of
their own, with a partial rotation, a cap on the scores and an optional window.

    q = Wq h [H, dk], k = Wk h [G, dk], v = Wv h [G, dv]                    (no bias)
    q, k: the first `rot` dimensions of each head turned by the token's position, dimension i < rot/2 paired with
          i + rot/2 (the position encoding's cos/sin table [positions, rot/2]); the other dimensions pass
    s_j = scale * q . k_j;  s_j <- cap * tanh(s_j / cap) if cap > 0;  keys pos - window < j <= pos (all j <= pos
          when window is 0);  softmax over those keys;  x += Wo concat_heads(sum_j p_j v_j)
Query head i reads key/value head i // (H / G).

The cache keeps per token two tensors: "k" (G, dk), the turned key, and "v" (G, dv).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import matmul_nt
from .registry import MIXERS, Part
from .spec import CacheNeed, TensorDecl

_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o"}


@MIXERS.register("capped_attention")
class CappedAttention(Part):
    graph_safe = True
    can_overwrite = True
    """params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale, softcap (0 or None: no cap),
    window (0 or None: all keys), position (a `rotary` encoding whose head_dim is the number of turned
    dimensions, or None), tensor_names (optional overrides)."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.H = int(self._need("num_heads"))
        self.G = int(self._need("num_kv_heads"))
        self.dk = int(self._need("key_dim"))
        self.dv = int(self._need("value_dim"))
        self.scale = float(self._need("scale"))
        self.cap = float(self.params.get("softcap") or 0.0)
        self.window = int(self.params.get("window") or 0)
        self.position = self.params.get("position")
        if self.H % self.G:
            raise ValueError(f"capped_attention: {self.H} heads are not a multiple of {self.G} key heads")
        if not (1 <= self.dk <= ops.MAX_HEAD_DIM and 1 <= self.dv <= ops.MAX_HEAD_DIM):
            raise ValueError(f"capped_attention: head sizes up to {ops.MAX_HEAD_DIM} are supported")
        self.rot = 0 if self.position is None else int(self.position.head_dim)
        if self.rot % 2 or self.rot > self.dk:
            raise ValueError(f"capped_attention: {self.rot} turned dimensions must be even and at most key_dim {self.dk}")
        self.names = {k: prefix + v for k, v in {**_NAMES, **self.params.get("tensor_names", {})}.items()}
        self.w_qkv = self.w_o = None

    def tensors(self):
        n = self.names
        return [TensorDecl(n["q"], (self.H * self.dk, self.D)), TensorDecl(n["k"], (self.G * self.dk, self.D)),
                TensorDecl(n["v"], (self.G * self.dv, self.D)), TensorDecl(n["o"], (self.D, self.H * self.dv))]

    def load(self, get):
        to, n = self.rt.to_compute, self.names
        self.w_qkv = torch.cat([to(get(n["q"])), to(get(n["k"])), to(get(n["v"]))], 0).contiguous()
        self.w_o = to(get(n["o"]))

    def cache_need(self):
        return CacheNeed("window" if self.window else "full",
                         (("k", (self.G, self.dk)), ("v", (self.G, self.dv))), self.window)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o) if t is not None)

    def cache_bytes_per_query(self, context):
        seen = min(context, self.window) if self.window else context
        return seen * self.G * (self.dk + self.dv) * (2 if self.rt.dtype == torch.bfloat16 else 4)

    def flops(self, start, count):
        products = 2.0 * self.D * (self.H * self.dk + self.G * (self.dk + self.dv) + self.H * self.dv)
        first, last = start + 1, start + count
        tri = lambda a, b: (a + b) * (b - a + 1) / 2.0 if b >= a else 0.0      # noqa: E731
        if self.window:
            w = self.window
            seen = tri(first, min(last, w)) + w * max(0, last - max(first, w + 1) + 1)
        else:
            seen = tri(first, last)
        return count * products + 2.0 * self.H * (self.dk + self.dv) * seen

    def first_weights(self):
        return self.w_qkv

    def forward(self, h, residual, ctx, cache, state, owns_cache=True, overwrite: bool = False):
        """overwrite: the output is written into `residual` (float32) instead of added."""
        if not owns_cache:
            raise ValueError("capped_attention: reading another entry's cache is not supported")
        T = h.shape[0]
        qw = self.H * self.dk
        qkv = self.rt.buffer("capped.qkv", T, qw + self.G * (self.dk + self.dv))
        matmul_nt(self.rt, qkv, h, self.w_qkv)
        cos, sin = self.position.tables() if self.rot else (None, None)
        kc, vc = cache.tensors["k"], cache.tensors["v"]
        o = self.rt.buffer("capped.o", T, self.H * self.dv)
        from . import attention_dispatch as ad
        ad.split_mixer_core(self.rt, o, qkv, cos, sin, self.rot, kc, vc, cache.tables, ctx, self.H, self.G, self.dk,
                            self.dv, self.window, self.scale, self.cap)
        matmul_nt(self.rt, residual, o, self.w_o, accumulate=not overwrite)
