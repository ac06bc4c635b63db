"""Mixer `parallel_mixers`: several mixers side by side that read the same input; each one's output is
RMS-normed over the model width with a weight of its own, and the mean of the normed outputs is the
layer's output:   x += (1/n) sum_b norm_b(mixer_b(h)).

params: hidden_size, eps, branches: a list of {"tag", "kind", "params", "prefix", "out_norm"} (the registered
kind and parameters of the mixer, the tensor-name prefix below the layer's and the name of its output
norm's weight).  At most one branch may keep a paged cache (it gets the entry's); every branch's
per-sequence state is kept under "<tag>.<name>".
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .registry import MIXERS, Part
from .spec import TensorDecl


@MIXERS.register("parallel_mixers")
class ParallelMixers(Part):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.eps = float(self._need("eps"))
        table = self.params.get("position_table", {})
        self.branches = []
        for b in self._need("branches"):
            sub = dict(b["params"])
            if isinstance(sub.get("position"), str):
                sub["position"] = table[sub["position"]]
            mixer = MIXERS.get(b["kind"])(sub, prefix + b["prefix"], runtime)
            self.branches.append((b["tag"], mixer, prefix + b["out_norm"]))
        if not self.branches:
            raise ValueError("parallel_mixers: at least one branch is needed")
        if sum(1 for _, m, _ in self.branches if m.cache_need() is not None) > 1:
            raise ValueError("parallel_mixers: only one branch may keep a paged cache")
        self.graph_safe = all(getattr(m, "graph_safe", False) for _, m, _ in self.branches)
        self.out_w = {}

    def tensors(self):
        out = []
        for _, m, norm_name in self.branches:
            out += m.tensors() + [TensorDecl(norm_name, (self.D,), "ones_normal")]
        return out

    def load(self, get):
        for tag, m, norm_name in self.branches:
            m.load(get)
            self.out_w[tag] = self.rt.to_f32(get(norm_name))

    def cache_need(self):
        for _, m, _ in self.branches:
            if m.cache_need() is not None:
                return m.cache_need()
        return None

    def state_need(self):
        return {f"{tag}.{name}": need for tag, m, _ in self.branches for name, need in m.state_need().items()}

    def weight_bytes(self):
        return sum(m.weight_bytes() for _, m, _ in self.branches)

    def cache_bytes_per_query(self, context):
        return sum(m.cache_bytes_per_query(context) for _, m, _ in self.branches)

    def flops(self, start, count):
        return sum(m.flops(start, count) for _, m, _ in self.branches)

    def first_weights(self):
        f = getattr(self.branches[0][1], "first_weights", None)
        return f() if f is not None else None

    can_overwrite = True

    def forward(self, h, residual, ctx, cache, state, owns_cache=True, overwrite: bool = False):
        """overwrite: the output is written into `residual` (float32) instead of added."""
        coef = 1.0 / len(self.branches)
        y = self.rt.buffer("parallel.branch_out", h.shape[0], self.D, dtype=torch.float32)
        for i, (tag, m, _) in enumerate(self.branches):
            own = {name[len(tag) + 1:]: t for name, t in state.items() if name.startswith(tag + ".")}
            if getattr(m, "can_overwrite", False):
                m.forward(h, y, ctx, cache, own, owns_cache, overwrite=True)
            else:
                y.zero_()
                m.forward(h, y, ctx, cache, own, owns_cache)
            ops.rmsnorm_add(residual, y, self.out_w[tag], self.eps, coef, accumulate=not (overwrite and i == 0))
