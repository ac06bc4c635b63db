"""Mixer `gated_delta`: a gated delta rule, a recurrent layer whose memory is one matrix S [dk, dv] per
head and sequence.

With h the layer's input, per token:
    q~, k~, v~ = silu(conv(Wq h)), silu(conv(Wk h)), silu(conv(Wv h))   causal convolution over time, per channel
    q = unit(q~) * dk^-1/2,  k = unit(k~)          unit(a) = a / sqrt(|a|^2 + 1e-6), per head
    beta = sigmoid(Wb h),  g = exp(-exp(A_log) * softplus(Wa h + dt_bias))       one per value head
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    x += Wo (o / sqrt(mean(o^2) + eps) * w_norm * silu(Wg h))
q and k have kv_heads heads, v has heads heads; value head i reads q/k head i // (heads / kv_heads).

The six projections are one matrix product whose output is float32 (the decays, step sizes and
everything the recurrence reads stay in float32); S and the last taps - 1 projection rows are
per-sequence state (float32).  Prompts, pieces of prompts and single tokens run the same kernels.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import matmul_nt
from .registry import MIXERS, Part
from .spec import StateNeed, TensorDecl

_NAMES = {"q": "mix.q", "k": "mix.k", "v": "mix.v", "q_conv": "mix.q.conv", "k_conv": "mix.k.conv",
          "v_conv": "mix.v.conv", "b": "mix.b", "a": "mix.a", "A_log": "mix.A_log", "dt_bias": "mix.dt_bias",
          "g": "mix.g", "norm": "mix.norm", "o": "mix.o"}


@MIXERS.register("gated_delta")
class GatedDelta(Part):
    graph_safe = True
    """params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, conv_taps, eps (of the read-out's
    norm), tensor_names (optional overrides)."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.H = int(self._need("num_heads"))
        self.G = int(self._need("num_kv_heads"))
        self.dk = int(self._need("key_dim"))
        self.dv = int(self._need("value_dim"))
        self.taps = int(self._need("conv_taps"))
        self.eps = float(self._need("eps"))
        if self.H % self.G:
            raise ValueError(f"gated_delta: {self.H} heads are not a multiple of {self.G} key heads")
        if not (1 <= self.dk <= 256 and 1 <= self.dv <= 4096 and 1 <= self.taps <= 32):
            raise ValueError("gated_delta: key_dim up to 256, value_dim up to 4096 and 1..32 taps are supported")
        self.C = 2 * self.G * self.dk + self.H * self.dv                    # channels that pass the convolution
        self.P = self.C + self.H * self.dv + 2 * self.H                     # + gate, beta, a
        self.names = {k: prefix + v for k, v in {**_NAMES, **self.params.get("tensor_names", {})}.items()}
        self.w_in = self.w_o = None

    def tensors(self):
        n, qk, vv = self.names, self.G * self.dk, self.H * self.dv
        return [TensorDecl(n["q"], (qk, self.D)), TensorDecl(n["k"], (qk, self.D)), TensorDecl(n["v"], (vv, self.D)),
                TensorDecl(n["q_conv"], (qk, self.taps)), TensorDecl(n["k_conv"], (qk, self.taps)),
                TensorDecl(n["v_conv"], (vv, self.taps)), TensorDecl(n["b"], (self.H, self.D)),
                TensorDecl(n["a"], (self.H, self.D)), TensorDecl(n["A_log"], (self.H,)),
                TensorDecl(n["dt_bias"], (self.H,)), TensorDecl(n["g"], (vv, self.D)),
                TensorDecl(n["norm"], (self.dv,), "ones_normal"), TensorDecl(n["o"], (self.D, vv))]

    def load(self, get):
        to, f32, n = self.rt.to_compute, self.rt.to_f32, self.names
        self.w_in = torch.cat([to(get(n[k])) for k in ("q", "k", "v", "g", "b", "a")], 0).contiguous()
        self.conv_w = torch.cat([f32(get(n[k])) for k in ("q_conv", "k_conv", "v_conv")], 0).contiguous()
        self.A_log, self.dt_bias, self.norm_w = f32(get(n["A_log"])), f32(get(n["dt_bias"])), f32(get(n["norm"]))
        self.w_o = to(get(n["o"]))

    def state_need(self):
        return {"S": StateNeed((self.H, self.dk, self.dv), torch.float32),
                "conv": StateNeed((max(self.taps - 1, 1), self.C), torch.float32)}

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o) if t is not None)

    def state_bytes_per_query(self) -> int:
        """Bytes of state one sequence's token reads and writes."""
        return 2 * 4 * (self.H * self.dk * self.dv + max(self.taps - 1, 1) * self.C)

    def cache_bytes_per_query(self, context):
        return self.state_bytes_per_query()

    def flops(self, start, count):
        products = 2.0 * self.D * (self.P + self.H * self.dv)
        return count * (products + 6.0 * self.H * self.dk * self.dv)

    def first_weights(self):
        return self.w_in

    can_overwrite = True

    def forward(self, h, residual, ctx, cache, state, owns_cache=True, overwrite: bool = False):
        """overwrite: the output is written into `residual` (float32) instead of added."""
        T, f32 = h.shape[0], torch.float32
        vv = self.H * self.dv
        buf = self.rt.buffer
        proj = buf("delta.proj", T, self.P, dtype=f32)
        matmul_nt(self.rt, proj, h, self.w_in)
        qkv = buf("delta.qkv", T, self.C, dtype=f32)
        gb = buf("delta.gb", T, 2 * self.H, dtype=f32)
        ops.short_conv_prepare(qkv, gb, proj, self.conv_w, state["conv"], self.A_log, self.dt_bias, ctx, self.G,
                               self.H, self.dk, self.dv, self.dk ** -0.5)
        ops.conv_state_update(state["conv"], proj, self.C, self.taps, ctx)
        o = buf("delta.o", T, vv, dtype=f32)
        ops.delta_rule_scan(o, state["S"], qkv, gb, ctx, self.G, self.H, self.dk, self.dv)
        y = buf("delta.y", T, vv)
        ops.head_gate(y, o, proj[:, self.C:self.C + vv], self.norm_w, self.H, self.dv, True, "silu", self.eps)
        matmul_nt(self.rt, residual, y, self.w_o, accumulate=not overwrite)
