"""The Fuvipel decoder as data: FuvipelConfig -> ModelSpec.

Every layer norms what its sublayers return (`norm_after`): x += norm1(mixer(x)); x += norm2(ffn(x)), the
feed-forward being optional.  A "delta" layer's mixer is a gated delta rule (`gated_delta`); a "parallel"
layer's is the mean of two normed mixers that read the same input (`parallel_mixers`): an attention with
a sink whose values are its keys (`sink_attention`, rotated on interleaved pairs by `rotary_pairs`) and a
time mixing with per-channel decay (`decay_time_mix`).  The feed-forward is `relu2`.  A final RMS norm,
and the head is the embedding table.  Tensor names: `embed`, `final.norm`, `l<i>.norm1`, `l<i>.norm2`,
`l<i>.mix.*`, `l<i>.mlp.up`, `l<i>.mlp.down`.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.fuvipel import FuvipelConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

NO_POSITION_LIMIT = 1 << 30        # the design has no largest position; the cache's size bounds a sequence


def build_spec(cfg: FuvipelConfig, max_positions: int | None = None) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps
    positions, layers = {}, []

    def norm(name):
        return PartSpec("rms_norm", {"size": D, "eps": eps, "name": name})

    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        if layer["type"] == "delta":
            mixer = PartSpec("gated_delta", {"hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
                                             "key_dim": m["dim"], "value_dim": m["vdim"], "conv_taps": m["conv"],
                                             "eps": eps})
        else:
            left, right = m["left"], m["right"]
            pos = None
            if left["rot"] is not None and left["rot"]["dims"] > 0:
                pos = f"rot{i}"
                positions[pos] = PartSpec("rotary_pairs", {"dims": left["rot"]["dims"], "base": left["rot"]["base"]})
            mixer = PartSpec("parallel_mixers", {"hidden_size": D, "eps": eps, "branches": [
                {"tag": "left", "kind": "sink_attention", "prefix": "mix.left.", "out_norm": "mix.left.out",
                 "params": {"hidden_size": D, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"],
                            "head_dim": left["dim"], "scale": left["scale"], "eps": eps, "position": pos,
                            "window": 0, "gate": True}},
                {"tag": "right", "kind": "decay_time_mix", "prefix": "mix.right.", "out_norm": "mix.right.out",
                 "params": {"hidden_size": D, "num_heads": right["heads"], "head_dim": right["dim"], "eps": eps,
                            "decay_rank": right.get("rank")}}]})
        mlp = layer["mlp"]
        layers.append(LayerSpec(
            prefix=f"l{i}.", mixer=mixer,
            feed_forward=None if mlp is None else PartSpec("relu2", {
                "hidden_size": D, "intermediate_size": mlp["ff"],
                "tensor_names": {"up": "mlp.up", "down": "mlp.down"}}),
            mixer_norm=norm("norm1"), ffn_norm=None if mlp is None else norm("norm2"), block="norm_after"))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab,
        max_positions=NO_POSITION_LIMIT if max_positions is None else min(max_positions, NO_POSITION_LIMIT),
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": D, "name": "embed"}),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": D, "tied": True}),
        positions=positions, layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))))


register_architecture("Fuvipel", FuvipelConfig, build_spec)
