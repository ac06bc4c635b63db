"""Mixer `retention`: linear attention with one fixed decay per head, no softmax and no denominator; a recurrent
layer whose memory is one matrix S [dk, dv] per head and sequence.

    q = Wq h, k = Wk h [H, dk], v = Wv h [H, dv], gate = silu(Wg h) [H dv]      (no bias)
    q, k: the first `rot` dimensions of each head turned by the token's position (dimension i < rot/2 paired with
          i + rot/2), then k times dk^(-1/2)
    S <- gamma_h S + k v^T;   o = S^T q                                     per head, S starts at zero
    x += Wo (concat_heads(o / sqrt(mean(o^2) + eps)) * gate)
The projections leave their product as float32 on both paths, so nothing that enters the recurrence is rounded to
16 bits; the turn, the scaling, S and the read-out are float32.  Two forms (csrc/retention.cu): a step in which
some sequence brings CHUNK_FROM tokens or more cuts every sequence's tokens into chunks of 32 and computes all
chunks side by side, only the state going from chunk to chunk (the same sums chunk by chunk); other steps, decoding
among them, take the tokens one by one.  Both leave the same state up to rounding.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import matmul_nt
from .registry import MIXERS, Part
from .spec import StateNeed, TensorDecl

_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o"}
CHUNK_FROM = 16         # a step whose longest sequence brings fewer tokens goes token by token


@MIXERS.register("retention")
class Retention(Part):
    graph_safe = True
    can_overwrite = True
    """params: hidden_size, num_heads, key_dim, value_dim, decay (one number per head), eps (of the read-out's
    norm), position (a `rotary` encoding whose head_dim is the number of turned dimensions, or None),
    tensor_names (optional overrides)."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.H = int(self._need("num_heads"))
        self.dk = int(self._need("key_dim"))
        self.dv = int(self._need("value_dim"))
        self.eps = float(self._need("eps"))
        self.decay_values = [float(g) for g in self._need("decay")]
        if len(self.decay_values) != self.H:
            raise ValueError(f"retention: {len(self.decay_values)} decays for {self.H} heads")
        if not 1 <= self.dk <= 256:
            raise ValueError("retention: key_dim up to 256 is supported")
        self.position = self.params.get("position")
        self.rot = 0 if self.position is None else int(self.position.head_dim)
        if self.rot % 2 or self.rot > self.dk:
            raise ValueError(f"retention: {self.rot} turned dimensions must be even and at most key_dim {self.dk}")
        self.names = {k: prefix + v for k, v in {**_NAMES, **self.params.get("tensor_names", {})}.items()}
        self.w_in = self.w_o = self.decay = None

    def tensors(self):
        n, qk, vv = self.names, self.H * self.dk, self.H * self.dv
        return [TensorDecl(n["q"], (qk, self.D)), TensorDecl(n["k"], (qk, self.D)), TensorDecl(n["v"], (vv, self.D)),
                TensorDecl(n["g"], (vv, self.D)), TensorDecl(n["o"], (self.D, vv))]

    def load(self, get):
        to, n = self.rt.to_compute, self.names
        self.w_in = torch.cat([to(get(n[k])) for k in ("q", "k", "v", "g")], 0).contiguous()
        self.w_o = to(get(n["o"]))
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(self.rt.device)

    def state_need(self):
        return {"S": StateNeed((self.H, self.dk, self.dv), torch.float32)}

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o) if t is not None)

    def cache_bytes_per_query(self, context):
        return 2 * 4 * self.H * self.dk * self.dv          # the state, read and written

    def flops(self, start, count):
        return count * (2.0 * self.D * (2 * self.H * self.dk + 3 * self.H * self.dv) + 4.0 * self.H * self.dk * self.dv)

    def first_weights(self):
        return self.w_in

    def forward(self, h, residual, ctx, cache, state, owns_cache=True, overwrite: bool = False):
        """overwrite: the output is written into `residual` (float32) instead of added."""
        T, f32 = h.shape[0], torch.float32
        qk, vv = self.H * self.dk, self.H * self.dv
        proj = self.rt.buffer("retention.in", T, 2 * qk + 2 * vv, dtype=f32)
        matmul_nt(self.rt, proj, h, self.w_in)
        cos, sin = self.position.tables() if self.rot else (None, None)
        o = self.rt.buffer("retention.o", T, vv, dtype=f32)
        scratch = None
        if ctx.max_qlen >= CHUNK_FROM:
            scratch = self.rt.buffer("retention.chunks", ops.retention_scratch(T, ctx.n_seqs, self.H, self.dk, self.dv),
                                     dtype=f32)
        ops.retention_scan(o, state["S"], proj, 0, qk, 2 * qk, cos, sin, self.rot, self.dk ** -0.5, self.decay, ctx,
                           self.H, self.dk, self.dv, scratch=scratch)
        y = self.rt.buffer("retention.y", T, vv)
        ops.head_gate(y, o, proj[:, 2 * qk + vv:], None, self.H, self.dv, True, "silu", self.eps)
        matmul_nt(self.rt, residual, y, self.w_o, accumulate=not overwrite)
