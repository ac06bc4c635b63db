"""Mixer `parallel_mixers`: several mixers side by side that read the same input.  Two ways of putting their
outputs together:

* each one's output is RMS-normed over the model width with a weight of its own, and the mean of the normed
  outputs is the layer's output:   x += (1/n) sum_b norm_b(mixer_b(h))        (branches with "out_norm");
* a weighted sum of the outputs as they are:   x += sum_b c_b mixer_b(h)       (branches with "coef" and no
  "out_norm"); this form takes the block's `scale=(m, s)` and adds m * s * sum_b c_b mixer_b(h) in one kernel.

params: hidden_size, eps, branches: a list of {"tag", "kind", "params", "prefix", "out_norm" or "coef"} (the
registered kind and parameters of the mixer, the tensor-name prefix below the layer's, and the name of its output
norm's weight or its coefficient).  At most one branch may keep a paged cache (it gets the entry's); every
branch's per-sequence state is kept under "<tag>.<name>".
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
        self.eps = float(self.params.get("eps") or 0.0)
        table = self.params.get("position_table", {})
        self.branches = []
        self.coefs = []
        for b in self._need("branches"):
            sub = dict(b["params"])
            if isinstance(sub.get("position"), str):
                sub["position"] = table[sub["position"]]
            mixer = MIXERS.get(b["kind"])(sub, prefix + b["prefix"], runtime)
            normed = b.get("out_norm") is not None
            self.branches.append((b["tag"], mixer, prefix + b["out_norm"] if normed else None))
            self.coefs.append(None if normed else float(b.get("coef", 1.0)))
        if not self.branches:
            raise ValueError("parallel_mixers: at least one branch is needed")
        self.weighted = self.coefs[0] is not None
        if any((c is not None) != self.weighted for c in self.coefs):
            raise ValueError("parallel_mixers: either every branch has an output norm or none has")
        self.can_scale = self.weighted
        if sum(1 for _, m, _ in self.branches if m.cache_need() is not None) > 1:
            raise ValueError("parallel_mixers: only one branch may keep a paged cache")
        self.graph_safe = all(getattr(m, "graph_safe", False) for _, m, _ in self.branches)
        self.out_w = {}

    def tensors(self):
        out = []
        for _, m, norm_name in self.branches:
            out += m.tensors() + ([TensorDecl(norm_name, (self.D,), "ones_normal")] if norm_name else [])
        return out

    def load(self, get):
        for tag, m, norm_name in self.branches:
            m.load(get)
            if norm_name:
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

    def _branch_into(self, i, y, h, ctx, cache, state, owns_cache):
        tag, m, _ = self.branches[i]
        own = {name[len(tag) + 1:]: t for name, t in state.items() if name.startswith(tag + ".")}
        if getattr(m, "can_overwrite", False):
            m.forward(h, y, ctx, cache, own, owns_cache, overwrite=True)
        else:
            y.zero_()
            m.forward(h, y, ctx, cache, own, owns_cache)

    def _forward_weighted(self, h, residual, ctx, cache, state, owns_cache, overwrite, scale):
        mult, vec = scale if scale is not None else (1.0, None)
        if overwrite:
            residual.zero_()
        ys = []
        for i in range(len(self.branches)):
            y = self.rt.buffer(f"parallel.branch_out{i}", h.shape[0], self.D, dtype=torch.float32)
            self._branch_into(i, y, h, ctx, cache, state, owns_cache)
            ys.append(y)
        for i in range(0, len(ys), 2):               # two outputs a kernel
            two = i + 1 < len(ys)
            ops.scaled_add(residual, ys[i], vec, mult, self.coefs[i], ys[i + 1] if two else None,
                           self.coefs[i + 1] if two else 0.0)

    def forward(self, h, residual, ctx, cache, state, owns_cache=True, overwrite: bool = False, scale=None):
        """overwrite: the output is written into `residual` (float32) instead of added.  scale = (m, s): the output
        is multiplied by the constant m and, per channel, by the float32 vector s (or None) before it is added
        (the weighted form only)."""
        if self.weighted:
            return self._forward_weighted(h, residual, ctx, cache, state, owns_cache, overwrite, scale)
        if scale is not None:
            raise ValueError("parallel_mixers: branches with output norms take no scale")
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
