"""Mixer `sink_attention`: grouped-query attention over the paged cache whose softmax has a sink and whose
values are its keys.

    q = Wq h, k = Wk h (no bias), v = k as projected (there is no value projection)
    q, k rotated by the position encoding (pairs (2i, 2i+1) of the first `dims` dimensions), then each head
    divided by its root mean square (no weight)
    s_j = scale * q . k_j for the keys j <= t of the sequence (or the last `window`)
    p_j = exp(s_j) / (1 + sum_j exp(s_j))          the sink: a key of score 0 that has no value
    x += Wo (sigmoid(Wg h) * concat_heads(sum_j p_j v_j))
Query head i reads key head i // (heads / kv_heads).

The cache keeps per token the tensor "kv" (2, kv_heads, head_dim): the rotated, normed key and the key as
projected (the value), which is the layout the attention kernels of this library read.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import matmul_nt
from .registry import MIXERS, Part
from .spec import TensorDecl, attention_cache_need

_NAMES = {"q": "q", "k": "k", "g": "g", "o": "o"}


@MIXERS.register("sink_attention")
class SinkAttention(Part):
    graph_safe = True
    """params: hidden_size, num_heads, num_kv_heads, head_dim, scale, eps (of the q/k norm), position (a
    `rotary_pairs` encoding or None), window (0 = all keys), gate (True: the output gate sigmoid(Wg h)),
    tensor_names (optional overrides)."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.H = int(self._need("num_heads"))
        self.G = int(self._need("num_kv_heads"))
        self.hd = int(self._need("head_dim"))
        self.scale = float(self._need("scale"))
        self.eps = float(self._need("eps"))
        self.window = int(self.params.get("window", 0) or 0)
        self.gate = bool(self.params.get("gate", True))
        self.position = self.params.get("position")
        if self.H % self.G:
            raise ValueError(f"sink_attention: {self.H} heads are not a multiple of {self.G} key heads")
        if self.hd % 2 or not 2 <= self.hd <= ops.MAX_HEAD_DIM:
            raise ValueError(f"sink_attention: head_dim {self.hd} must be even and at most {ops.MAX_HEAD_DIM}")
        self.names = {k: prefix + v for k, v in {**_NAMES, **self.params.get("tensor_names", {})}.items()}
        self.w_in = self.w_o = None

    def tensors(self):
        n, q, kv = self.names, self.H * self.hd, self.G * self.hd
        out = [TensorDecl(n["q"], (q, self.D)), TensorDecl(n["k"], (kv, self.D)), TensorDecl(n["o"], (self.D, q))]
        if self.gate:
            out.append(TensorDecl(n["g"], (q, self.D)))
        return out

    def load(self, get):
        to, n = self.rt.to_compute, self.names
        self.w_in = torch.cat([to(get(n[k])) for k in (("q", "k", "g") if self.gate else ("q", "k"))], 0).contiguous()
        self.w_o = to(get(n["o"]))

    def cache_need(self):
        return attention_cache_need(self.G, self.hd, self.window)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o) if t is not None)

    def cache_bytes_per_query(self, context):
        seen = min(context, self.window) if self.window else context
        return seen * 2 * self.G * self.hd * (2 if self.rt.dtype == torch.bfloat16 else 4)

    def flops(self, start, count):
        rows = (2 + int(self.gate)) * self.H + self.G
        first, last = start + 1, start + count
        tri = lambda a, b: (a + b) * (b - a + 1) / 2.0 if b >= a else 0.0      # noqa: E731
        if self.window:
            w = self.window
            seen = tri(first, min(last, w)) + w * max(0, last - max(first, w + 1) + 1)
        else:
            seen = tri(first, last)
        return count * 2.0 * self.D * rows * self.hd + 4.0 * self.H * self.hd * seen

    def first_weights(self):
        return self.w_in

    can_overwrite = True

    def forward(self, h, residual, ctx, cache, state, owns_cache=True, overwrite: bool = False):
        """overwrite: the output is written into `residual` (float32) instead of added."""
        T = h.shape[0]
        qw, kw = self.H * self.hd, self.G * self.hd
        width = qw + kw + (qw if self.gate else 0)
        if not owns_cache:
            raise ValueError("sink_attention: reading another entry's cache is not supported")
        qkg = self.rt.buffer("sink.qkg", T, width)
        matmul_nt(self.rt, qkg, h, self.w_in)
        inv_freq, dims = self.position.tables() if self.position is not None else (None, 0)
        ops.rot_norm_kv_write(qkg, inv_freq, dims, cache.kv, cache.tables, ctx.tok_seq, ctx.tok_pos, self.H, self.G,
                              self.hd, self.eps, True)
        o = self.rt.buffer("sink.o", T, qw)
        from . import attention_dispatch as ad
        ad.attend(self.rt, o, qkg, cache, ctx, self.H, self.G, self.hd, self.window, self.scale, sink=True)
        if self.gate:
            y = self.rt.buffer("sink.y", T, qw)
            ops.head_gate(y, o, qkg[:, qw + kw:], None, self.H, self.hd, False, "sigmoid")
            o = y
        matmul_nt(self.rt, residual, o, self.w_o, accumulate=not overwrite)
