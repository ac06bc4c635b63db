"""Mixer `decay_time_mix`: time mixing with a data-dependent decay per key channel (in the manner of
RWKV's sixth version), a recurrent layer whose memory is one matrix S [d, d] per head and sequence.

With h the layer's input and h' the previous token's (zeros before a sequence's first token):
    m_s = h + (h' - h) * mu_s                      for s in r, k, v, g, w
    r, k, v = Wr m_r, Wk m_k, Wv m_v               heads x d
    gate = silu(Wg m_g);  w = exp(-exp(W2 tanh(W1 m_w) + w0))          w per head and key channel
    o = (S + diag(u) k v^T)^T r;  S <- diag(w) S + k v^T               u only for the current token
    x += Wo (concat_heads(o / sqrt(mean(o^2) + eps)) * w_norm * gate)
r, k, v and the decay's argument come out of their products in float32; S and h' are per-sequence state
(float32).  Prompts, pieces of prompts and single tokens run the same kernels.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import matmul_nt
from .registry import MIXERS, Part
from .spec import StateNeed, TensorDecl

_MIXES = ("r", "k", "v", "g", "w")
_NAMES = {"r": "r", "k": "k", "v": "v", "g": "g", "w1": "w1", "w2": "w2", "w0": "w0", "u": "u", "norm": "norm", "o": "o",
          **{"mu_" + s: "mu." + s for s in _MIXES}}


@MIXERS.register("decay_time_mix")
class DecayTimeMix(Part):
    graph_safe = True
    """params: hidden_size, num_heads, head_dim, eps (of the read-out's norm), decay_rank (the rank of the
    decay's two-matrix projection; None: the shape of `w1` in the file gives it), tensor_names (optional
    overrides)."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.H = int(self._need("num_heads"))
        self.d = int(self._need("head_dim"))
        self.rank = int(self.params.get("decay_rank") or -1)
        self.eps = float(self._need("eps"))
        if not 1 <= self.d <= 256:
            raise ValueError("decay_time_mix: head_dim up to 256 is supported")
        self.names = {k: prefix + v for k, v in {**_NAMES, **self.params.get("tensor_names", {})}.items()}
        self.w = {}

    def tensors(self):
        n, hd = self.names, self.H * self.d
        out = [TensorDecl(n["mu_" + s], (self.D,)) for s in _MIXES]
        out += [TensorDecl(n[s], (hd, self.D)) for s in ("r", "k", "v", "g")]
        out += [TensorDecl(n["w1"], (self.rank, self.D)), TensorDecl(n["w2"], (hd, self.rank)),
                TensorDecl(n["w0"], (hd,)), TensorDecl(n["u"], (self.H, self.d)),
                TensorDecl(n["norm"], (hd,), "ones_normal"), TensorDecl(n["o"], (self.D, hd))]
        return out

    def load(self, get):
        to, f32, n = self.rt.to_compute, self.rt.to_f32, self.names
        self.mu = torch.stack([f32(get(n["mu_" + s])) for s in _MIXES], 0).contiguous()
        self.w = {s: to(get(n[s])) for s in ("r", "k", "v", "g", "w1", "w2", "o")}
        self.rank = int(self.w["w1"].shape[0])
        if self.w["w2"].shape[1] != self.rank:
            raise ValueError(f"{n['w2']}: {self.w['w2'].shape[1]} columns, but {n['w1']} has {self.rank} rows")
        self.w0, self.u, self.norm_w = f32(get(n["w0"])), f32(get(n["u"])).reshape(-1), f32(get(n["norm"]))

    def state_need(self):
        return {"S": StateNeed((self.H, self.d, self.d), torch.float32), "prev": StateNeed((self.D,), torch.float32)}

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in self.w.values())

    def cache_bytes_per_query(self, context):
        return 2 * 4 * (self.H * self.d * self.d + self.D)

    def flops(self, start, count):
        hd = self.H * self.d
        return count * (2.0 * self.D * 5 * hd + 2.0 * max(self.rank, 0) * (self.D + hd) + 4.0 * hd * self.d)

    def first_weights(self):
        return self.w.get("r")

    can_overwrite = True

    def forward(self, h, residual, ctx, cache, state, owns_cache=True, overwrite: bool = False):
        """overwrite: the output is written into `residual` (float32) instead of added."""
        T, f32, hd = h.shape[0], torch.float32, self.H * self.d
        buf = self.rt.buffer
        mix = buf("mix.in", len(_MIXES), T, self.D)
        ops.token_shift_mix(mix, h, self.mu, state["prev"], ctx)
        ops.last_rows_to_state(state["prev"], h, ctx)
        r, k, v, g, z = (buf("mix." + n, T, hd, dtype=f32) for n in "rkvgz")
        for out, i, name in ((r, 0, "r"), (k, 1, "k"), (v, 2, "v"), (g, 3, "g")):
            matmul_nt(self.rt, out, mix[i], self.w[name])
        low = buf("mix.low", T, self.rank, dtype=f32)
        matmul_nt(self.rt, low, mix[4], self.w["w1"])
        th = buf("mix.tanh", T, self.rank)
        ops.tanh_rows(th, low)
        matmul_nt(self.rt, z, th, self.w["w2"])
        o = buf("mix.o", T, hd, dtype=f32)
        ops.decay_scan(o, state["S"], r, k, v, z, self.u, self.w0, ctx, self.H, self.d)
        y = buf("mix.y", T, hd)
        ops.head_gate(y, o, g, self.norm_w, self.H, self.d, True, "silu", self.eps)
        matmul_nt(self.rt, residual, y, self.w["o"], accumulate=not overwrite)
