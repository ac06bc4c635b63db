"""FuvipelConfig: the sizes and constants of a Fuvipel decoder, read from config.json.

config.json of this design:
    architecture   "Fuvipel"
    vocab, width   sizes of the embedding table
    norm.eps       the epsilon of every root mean square of a layer
    layers         a list; each entry has `type` ("delta" or "parallel"), `mixer` (the mixer's sizes) and
                   `mlp` ({"kind": "dense", "ff": n} or null)
      delta        mixer: heads, kv_heads, dim, vdim, conv
      parallel     mixer: left {heads, kv_heads, dim, vdim, scale, rot {dims, base} or null},
                          right {heads, dim, optionally rank}
Nothing else is read; every key below the top level is checked, an unknown one is refused.  The design has no largest position, no stop tokens and
a head tied to the embedding table.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, _Reader


def _obj(raw, what):
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: `{what}` must be an object, got {raw!r}")
    return raw


def _only(raw: dict, what: str, allowed) -> None:
    extra = sorted(set(raw) - set(allowed))
    if extra:
        raise ConfigError(f"config.json: `{what}` has keys this design does not have: {', '.join(extra)}")


def _delta(raw, what) -> dict:
    raw = _obj(raw, what)
    _only(raw, what, ("heads", "kv_heads", "dim", "vdim", "conv"))
    r = _Reader(raw)
    m = {"heads": r.integer("heads"), "kv_heads": r.integer("kv_heads"), "dim": r.integer("dim"),
         "vdim": r.integer("vdim"), "conv": r.integer("conv")}
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: `{what}`: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
    return m


def _parallel(raw, what) -> dict:
    raw = _obj(raw, what)
    _only(raw, what, ("left", "right"))
    left, right = _obj(raw.get("left"), what + ".left"), _obj(raw.get("right"), what + ".right")
    _only(left, what + ".left", ("heads", "kv_heads", "dim", "vdim", "scale", "rot"))
    _only(right, what + ".right", ("heads", "dim", "rank"))
    rl, rr = _Reader(left), _Reader(right)
    lm = {"heads": rl.integer("heads"), "kv_heads": rl.integer("kv_heads"), "dim": rl.integer("dim"),
          "vdim": rl.integer("vdim"), "scale": rl.number("scale"), "rot": None}
    if lm["heads"] % lm["kv_heads"]:
        raise ConfigError(f"config.json: `{what}.left`: heads is not a multiple of kv_heads")
    if lm["vdim"] != lm["dim"]:
        raise ConfigError(f"config.json: `{what}.left`: vdim {lm['vdim']} differs from dim {lm['dim']}, but the "
                          f"values of this attention are its keys")
    if lm["dim"] % 2:
        raise ConfigError(f"config.json: `{what}.left.dim` must be even (rotated pairs)")
    if left.get("rot") is not None:
        rot = _obj(left["rot"], what + ".left.rot")
        _only(rot, what + ".left.rot", ("dims", "base"))
        rt = _Reader(rot)
        lm["rot"] = {"dims": rt.integer("dims", minimum=0), "base": rt.number("base")}
        if lm["rot"]["dims"] % 2 or lm["rot"]["dims"] > lm["dim"]:
            raise ConfigError(f"config.json: `{what}.left.rot.dims` must be even and at most dim")
    rm = {"heads": rr.integer("heads"), "dim": rr.integer("dim")}
    rank = rr.integer("rank", default=None, required=False)
    if rank is not None:
        rm["rank"] = rank
    return {"left": lm, "right": rm}


@dataclass(frozen=True)
class FuvipelConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: tuple              # of {"type", "mixer", "mlp"} with checked contents

    @staticmethod
    def from_dict(raw: dict) -> "FuvipelConfig":
        r = _Reader(raw)
        # top-level keys beyond these are a file's own notes (a name, a seed, a dtype) and are not read; inside
        # `norm`, a layer, a mixer or a feed-forward an unknown key would be a mechanism this code does not have
        norm = _obj(raw.get("norm"), "norm")
        _only(norm, "norm", ("eps",))
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: `layers` must be a list with at least one layer")
        out = []
        for i, layer in enumerate(layers):
            what = f"layers[{i}]"
            layer = _obj(layer, what)
            _only(layer, what, ("type", "mixer", "mlp"))
            kind = layer.get("type")
            if kind == "delta":
                mixer = _delta(layer.get("mixer"), what + ".mixer")
            elif kind == "parallel":
                mixer = _parallel(layer.get("mixer"), what + ".mixer")
            else:
                raise ConfigError(f"config.json: `{what}.type` must be \"delta\" or \"parallel\", got {kind!r}")
            mlp = layer.get("mlp")
            if mlp is not None:
                mlp = _obj(mlp, what + ".mlp")
                _only(mlp, what + ".mlp", ("kind", "ff"))
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: `{what}.mlp.kind` must be \"dense\", got {mlp.get('kind')!r}")
                mlp = {"kind": "dense", "ff": _Reader(mlp).integer("ff")}
            out.append({"type": kind, "mixer": mixer, "mlp": mlp})
        name = raw.get("architecture") or (raw.get("architectures") or ["Fuvipel"])[0]
        return FuvipelConfig(architecture=name, vocab=r.integer("vocab"), width=r.integer("width"),
                             norm_eps=_Reader(norm).number("eps"), layers=tuple(out))

    def to_dict(self) -> dict:
        """The config.json that `from_dict` reads back to an equal configuration."""
        import copy
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}
