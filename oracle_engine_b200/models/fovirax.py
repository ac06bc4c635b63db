"""The Fovirax decoder as data: FoviraxConfig -> ModelSpec.

Every layer is x += m * s1 * mixer(norm1(x)); x += m * s2 * ffn(norm2(x)) (`pre_norm_scaled`; the norms' weights
are kept around zero, `rms_norm` with offset 1; the feed-forward is optional).  The mixer is the weighted sum of
two mixers that read the same input (`parallel_mixers` with coefficients): an attention with a window, capped
scores, keys and values of different head sizes and a partial rotation whose frequencies may be rescaled by
wavelength (`capped_attention`), and a retention with a fixed decay per head (`retention`).  The feed-forward is a
mixture of experts with a shared expert (`moe_swiglu`).  The schedule repeats the looped group of layers: the
repeated entries share weights and each has a cache and a state of its own.  A final norm and a head of its own.
Tensor names: `embed`, `head`, `final.norm`, `l<i>.norm1|norm2|ls1|ls2`, `l<i>.mix.left|right.*`, `l<i>.mlp.*`.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.fovirax import FoviraxConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

NO_POSITION_LIMIT = 1 << 30        # the design has no largest position; the cache's size bounds a sequence


def build_spec(cfg: FoviraxConfig, max_positions: int | None = None) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps
    max_pos = NO_POSITION_LIMIT if max_positions is None else min(max_positions, NO_POSITION_LIMIT)
    positions, layers = {}, []

    def norm(name):
        return PartSpec("rms_norm", {"size": D, "eps": eps, "name": name, "offset": 1.0})

    def position(rot):
        """The name of the rotary tables for this rotation; equal rotations share one."""
        if rot is None:
            return None
        sc = rot["scaling"]
        key = f"rot:{rot['dims']}:{rot['base']!r}:" + ("-" if sc is None else
                                                      f"{sc['factor']!r}:{sc['low']!r}:{sc['high']!r}:{sc['original']!r}")
        if key not in positions:
            scaling = None if sc is None else {"factor": sc["factor"], "low_freq_factor": sc["low"],
                                               "high_freq_factor": sc["high"],
                                               "original_max_position_embeddings": sc["original"]}
            positions[key] = PartSpec("rotary", {"head_dim": rot["dims"], "theta": rot["base"], "scaling": scaling,
                                                 "max_positions": max_pos})
        return key

    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        left, right = m["left"], m["right"]
        mixer = PartSpec("parallel_mixers", {"hidden_size": D, "eps": eps, "branches": [
            {"tag": "left", "kind": "capped_attention", "prefix": "mix.left.", "coef": m["left_scale"],
             "params": {"hidden_size": D, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"],
                        "key_dim": left["dim"], "value_dim": left["vdim"], "scale": left["scale"],
                        "softcap": left["softcap"], "window": (left["mask"] or {}).get("size", 0),
                        "position": position(left["rot"])}},
            {"tag": "right", "kind": "retention", "prefix": "mix.right.", "coef": m["right_scale"],
             "params": {"hidden_size": D, "num_heads": right["heads"], "key_dim": right["dim"],
                        "value_dim": right["vdim"], "decay": right["decay"], "eps": eps,
                        "position": position(right["rot"])}}]})
        mlp = layer["mlp"]
        ffn = None if mlp is None else PartSpec("moe_swiglu", {
            "hidden_size": D, "num_experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
            "expert_size": mlp["expert"]["ff"], "shared_size": (mlp["shared"] or {}).get("ff", 0)})
        layers.append(LayerSpec(
            prefix=f"l{i}.", mixer=mixer, feed_forward=ffn, mixer_norm=norm("norm1"),
            ffn_norm=None if mlp is None else norm("norm2"), block="pre_norm_scaled",
            block_params={"hidden_size": D, "residual_mult": cfg.residual_mult, "mixer_scale": "ls1",
                          "ffn_scale": "ls2"}))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab, max_positions=max_pos,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": D, "name": "embed"}),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": D, "tied": False, "name": "head"}),
        positions=positions, layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in cfg.layer_order()),
        # a layer without a feed-forward reads neither of these, whether its file holds them or not
        ignored_tensors=(".norm2", ".ls2"))


register_architecture("Fovirax", FoviraxConfig, build_spec)
