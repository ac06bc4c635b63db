"""FoviraxConfig: the sizes and constants of a Fovirax decoder, read from config.json.

config.json of this design:
    architecture    "Fovirax"
    vocab, width    sizes of the embedding table
    norm.eps        the epsilon of every root mean square
    residual_mult   the constant every sublayer's output is multiplied by before it is added (default 1)
    loop            optional {start, stop, times}: layers start .. stop - 1 run `times` times as a group
    layers          a list; each entry has `type` ("parallel"), `mixer` and `mlp` (an object or null)
      mixer         left_scale, right_scale (default 1) and
        left        heads, kv_heads, dim, vdim, scale; optional softcap, mask {size}, rot {dims, base, optional
                    scaling {factor, low, high, original}}
        right       heads, dim, vdim, decay (one number per head); optional rot {dims, base, optional scaling}
      mlp           kind "moe", expert {ff}, router {experts, top}, optional shared {ff}
Every key below the top level is checked and an unknown one is refused: it would be a mechanism this code does not
have.  Top-level keys beyond these are a file's own notes.  The design has no largest position, no stop tokens and
a head of its own.
"""
from __future__ import annotations

import copy
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


def _rot(raw, what, dim):
    """None, or {"dims", "base", "scaling": None or {"factor", "low", "high", "original"}}."""
    if raw is None:
        return None
    raw = _obj(raw, what)
    _only(raw, what, ("dims", "base", "scaling"))
    r = _Reader(raw)
    out = {"dims": r.integer("dims", minimum=0), "base": r.number("base"), "scaling": None}
    if out["dims"] % 2 or out["dims"] > dim:
        raise ConfigError(f"config.json: `{what}.dims` must be even and at most the head's dim {dim}")
    if out["dims"] == 0:
        return None
    if raw.get("scaling") is not None:
        sc = _obj(raw["scaling"], what + ".scaling")
        _only(sc, what + ".scaling", ("factor", "low", "high", "original"))
        rs = _Reader(sc)
        out["scaling"] = {"factor": rs.number("factor"), "low": rs.number("low"), "high": rs.number("high"),
                          "original": rs.number("original")}
        if out["scaling"]["high"] == out["scaling"]["low"]:
            raise ConfigError(f"config.json: `{what}.scaling`: high and low must differ")
    return out


def _left(raw, what) -> dict:
    raw = _obj(raw, what)
    _only(raw, what, ("heads", "kv_heads", "dim", "vdim", "scale", "softcap", "mask", "rot"))
    r = _Reader(raw)
    m = {"heads": r.integer("heads"), "kv_heads": r.integer("kv_heads"), "dim": r.integer("dim"),
         "vdim": r.integer("vdim"), "scale": r.number("scale"),
         "softcap": r.number("softcap", default=None, required=False), "mask": None}
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: `{what}`: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
    if raw.get("mask") is not None:
        mask = _obj(raw["mask"], what + ".mask")
        _only(mask, what + ".mask", ("size",))
        m["mask"] = {"size": _Reader(mask).integer("size")}
    m["rot"] = _rot(raw.get("rot"), what + ".rot", m["dim"])
    return m


def _right(raw, what) -> dict:
    raw = _obj(raw, what)
    _only(raw, what, ("heads", "dim", "vdim", "decay", "rot"))
    r = _Reader(raw)
    m = {"heads": r.integer("heads"), "dim": r.integer("dim"), "vdim": r.integer("vdim")}
    decay = raw.get("decay")
    if not isinstance(decay, list) or len(decay) != m["heads"] or \
            not all(isinstance(g, (int, float)) and not isinstance(g, bool) for g in decay):
        raise ConfigError(f"config.json: `{what}.decay` must list one number per head ({m['heads']})")
    m["decay"] = [float(g) for g in decay]
    m["rot"] = _rot(raw.get("rot"), what + ".rot", m["dim"])
    return m


def _moe(raw, what) -> dict:
    raw = _obj(raw, what)
    _only(raw, what, ("kind", "expert", "router", "shared"))
    if raw.get("kind") != "moe":
        raise ConfigError(f"config.json: `{what}.kind` must be \"moe\", got {raw.get('kind')!r}")
    expert, router = _obj(raw.get("expert"), what + ".expert"), _obj(raw.get("router"), what + ".router")
    _only(expert, what + ".expert", ("ff",))
    _only(router, what + ".router", ("experts", "top"))
    out = {"kind": "moe", "expert": {"ff": _Reader(expert).integer("ff")},
           "router": {"experts": _Reader(router).integer("experts"), "top": _Reader(router).integer("top")},
           "shared": None}
    if out["router"]["top"] > out["router"]["experts"]:
        raise ConfigError(f"config.json: `{what}.router`: top exceeds experts")
    if raw.get("shared") is not None:
        shared = _obj(raw["shared"], what + ".shared")
        _only(shared, what + ".shared", ("ff",))
        out["shared"] = {"ff": _Reader(shared).integer("ff")}
    return out


@dataclass(frozen=True)
class FoviraxConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    loop: tuple | None         # (start, stop, times)
    layers: tuple              # of {"type", "mixer", "mlp"} with checked contents

    @staticmethod
    def from_dict(raw: dict) -> "FoviraxConfig":
        r = _Reader(raw)
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
            if layer.get("type") != "parallel":
                raise ConfigError(f"config.json: `{what}.type` must be \"parallel\", got {layer.get('type')!r}")
            mixer = _obj(layer.get("mixer"), what + ".mixer")
            _only(mixer, what + ".mixer", ("left", "right", "left_scale", "right_scale"))
            rm = _Reader(mixer)
            m = {"left": _left(mixer.get("left"), what + ".mixer.left"),
                 "right": _right(mixer.get("right"), what + ".mixer.right"),
                 "left_scale": rm.number("left_scale", default=1.0, required=False, positive=False),
                 "right_scale": rm.number("right_scale", default=1.0, required=False, positive=False)}
            mlp = None if layer.get("mlp") is None else _moe(layer["mlp"], what + ".mlp")
            out.append({"type": "parallel", "mixer": m, "mlp": mlp})
        loop = None
        if raw.get("loop") is not None:
            lp = _obj(raw["loop"], "loop")
            _only(lp, "loop", ("start", "stop", "times"))
            rl = _Reader(lp)
            loop = (rl.integer("start", minimum=0), rl.integer("stop", minimum=0), rl.integer("times", minimum=1))
            if not loop[0] <= loop[1] <= len(out):
                raise ConfigError(f"config.json: `loop` must name layers inside 0 .. {len(out)}")
        name = raw.get("architecture") or (raw.get("architectures") or ["Fovirax"])[0]
        return FoviraxConfig(architecture=name, vocab=r.integer("vocab"), width=r.integer("width"),
                             norm_eps=_Reader(norm).number("eps"),
                             residual_mult=r.number("residual_mult", default=1.0, required=False, positive=False),
                             loop=loop, layers=tuple(out))

    def layer_order(self) -> list:
        """The indices of the layers in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        a, b, times = self.loop
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    def to_dict(self) -> dict:
        """The config.json that `from_dict` reads back to an equal configuration."""
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
             "layers": copy.deepcopy(list(self.layers))}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d
