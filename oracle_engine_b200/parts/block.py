"""Arrangements of a layer's parts.  `pre_norm`: x += mixer(norm(x)); x += ffn(norm(x)),
the reference's layer (core/model.cpp:361-474).  The mixer and the feed-forward add their
outputs into the float32 residual stream themselves (fused into their last product).
`norm_after`: x += norm(mixer(x)); x += norm(ffn(x)): the sublayers read the residual stream itself and
their OUTPUT is normed before it is added; a sublayer adds its output into a zeroed float32 buffer.
`pre_norm_scaled`: x += m * s1 * mixer(norm(x)); x += m * s2 * ffn(norm(x)) with m one constant and s1, s2 one
weight per channel each (a layer scale)."""
from __future__ import annotations

import torch

from ..csrc import ops
from .registry import BLOCKS, Part
from .spec import TensorDecl


@BLOCKS.register("pre_norm")
class PreNormBlock:
    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward) if p is not None]

    def first_weights(self):
        """The weight matrix this block streams first (a hint for the part that runs before it), or None."""
        return _first_weights(self.mixer)

    def forward(self, x, ctx, cache, state, owns_cache=True):
        rt = getattr(self.mixer, "rt", None)
        after = getattr(rt, "next_weights", None)          # what the model says comes after this block
        h = self.mixer_norm.forward(x)
        if rt is not None:
            rt.next_weights = _first_weights(self.feed_forward) if self.feed_forward is not None else after
        self.mixer.forward(h, x, ctx, cache, state, owns_cache)
        if self.feed_forward is not None:
            h = self.ffn_norm.forward(x)
            if rt is not None:
                rt.next_weights = after
            self.feed_forward.forward(h, x, ctx)
        if rt is not None:
            rt.next_weights = None


@BLOCKS.register("norm_after")
class NormAfterBlock:
    """x <- x + norm_1(mixer(x)); x <- x + norm_2(ffn(x)) (the second only with a feed-forward)."""

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm):
        if mixer_norm is None or (feed_forward is not None and ffn_norm is None):
            raise ValueError("norm_after: every sublayer needs the norm of its output")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm

    def parts(self):
        return [p for p in (self.mixer, self.mixer_norm, self.feed_forward, self.ffn_norm) if p is not None]

    def first_weights(self):
        return _first_weights(self.mixer)

    def forward(self, x, ctx, cache, state, owns_cache=True):
        rt = self.mixer.rt
        rt.next_weights = None
        y = rt.buffer("sublayer_out", *x.shape, dtype=x.dtype)
        h = rt.activations(x)
        # a sublayer that can write its output (instead of adding it) saves the zeroing of the buffer
        if getattr(self.mixer, "can_overwrite", False):
            self.mixer.forward(h, y, ctx, cache, state, owns_cache, overwrite=True)
        else:
            y.zero_()
            self.mixer.forward(h, y, ctx, cache, state, owns_cache)
        self.mixer_norm.add_into(x, y, keep_cast=True)
        if self.feed_forward is not None:
            h = rt.activations(x)
            if getattr(self.feed_forward, "can_overwrite", False):
                self.feed_forward.forward(h, y, ctx, overwrite=True)
            else:
                y.zero_()
                self.feed_forward.forward(h, y, ctx)
            self.ffn_norm.add_into(x, y, keep_cast=True)


class ChannelScales(Part):
    """The per-channel weights of a block arrangement: params {"names": {key: tensor name under the prefix}, "size"}."""
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.size = int(self._need("size"))
        self.names = {k: prefix + v for k, v in self._need("names").items()}
        self.vec = {}

    def tensors(self):
        return [TensorDecl(n, (self.size,), "ones_normal") for n in self.names.values()]

    def load(self, get):
        self.vec = {k: self.rt.to_f32(get(n)) for k, n in self.names.items()}


@BLOCKS.register("pre_norm_scaled")
class PreNormScaledBlock:
    """x <- x + m * s1 * mixer(norm_1(x)); x <- x + m * s2 * ffn(norm_2(x)) (the second only with a feed-forward).
    params: hidden_size, residual_mult (m, default 1), mixer_scale / ffn_scale (tensor names of s1 / s2 under the
    layer's prefix; absent: no per-channel weight).  A sublayer that takes `scale=` applies m and s itself (in the
    kernel that adds its output); any other writes into a float32 buffer that one kernel scales and adds."""

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm, params, prefix, runtime):
        if mixer_norm is None or (feed_forward is not None and ffn_norm is None):
            raise ValueError("pre_norm_scaled: every sublayer needs the norm of its input")
        self.mixer, self.feed_forward, self.mixer_norm, self.ffn_norm = mixer, feed_forward, mixer_norm, ffn_norm
        self.rt = runtime
        self.mult = float(params.get("residual_mult", 1.0))
        names = {}
        if params.get("mixer_scale"):
            names["mixer"] = params["mixer_scale"]
        if feed_forward is not None and params.get("ffn_scale"):
            names["ffn"] = params["ffn_scale"]
        self.scales = ChannelScales({"names": names, "size": params["hidden_size"]}, prefix, runtime)

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward, self.scales)
                if p is not None]

    def first_weights(self):
        return _first_weights(self.mixer)

    def _sublayer(self, part, key, h, x, *args):
        vec = self.scales.vec.get(key)
        if getattr(part, "can_scale", False):
            part.forward(h, x, *args, scale=(self.mult, vec))
            return
        y = self.rt.buffer("sublayer_out", *x.shape, dtype=torch.float32)
        if getattr(part, "can_overwrite", False):
            part.forward(h, y, *args, overwrite=True)
        else:
            y.zero_()
            part.forward(h, y, *args)
        ops.scaled_add(x, y, vec, self.mult)

    def forward(self, x, ctx, cache, state, owns_cache=True):
        self.rt.next_weights = None
        self._sublayer(self.mixer, "mixer", self.mixer_norm.forward(x), x, ctx, cache, state, owns_cache)
        if self.feed_forward is not None:
            self._sublayer(self.feed_forward, "ffn", self.ffn_norm.forward(x), x, ctx)


def _first_weights(part):
    f = getattr(part, "first_weights", None)
    return f() if f is not None else None
