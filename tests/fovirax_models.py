"""Small Fovirax configurations for the tests, and a writer of model folders with weights that make faults show:
decays close to one come from the configuration; router weights are scaled up so that the experts' logits lie well
apart; layer scales and norm weights vary per channel."""
from pathlib import Path

import torch


def rot(dims, base, scaling=None):
    return {"dims": dims, "base": base, "scaling": scaling}


def scaling(factor, low, high, original):
    return {"factor": factor, "low": low, "high": high, "original": original}


def left(heads, kv_heads, dim, vdim, scale, softcap=None, window=None, rotation=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
            "mask": None if window is None else {"size": window}, "rot": rotation}


def right(heads, dim, vdim, decay, rotation=None):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": rotation}


def moe(experts, top, ff, shared=None):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top},
            "shared": None if shared is None else {"ff": shared}}


def layer(l, r, mlp=None, left_scale=1.0, right_scale=1.0):
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def config(vocab, width, eps, layers, residual_mult=None, loop=None):
    c = {"architecture": "Fovirax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if residual_mult is not None:
        c["residual_mult"] = residual_mult
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


# Wavelengths of the first rotation fall into all three bands of the rescaling (kept, blended, divided); the
# rotation is partial; key and value sizes differ both ways; a loop that does not start at the first layer; one
# layer without feed-forward, one without window, cap and rotation, one whose router chooses every expert.
V1 = config(300, 96, 1e-5, [
    layer(left(4, 2, 32, 16, 0.25, 8.0, 40, rot(16, 10000.0, scaling(4.0, 1.0, 4.0, 64))),
          right(3, 16, 24, [0.9, 0.99, 0.999], rot(8, 100.0)), moe(6, 2, 40, 24), 0.8, 1.3),
    layer(left(2, 2, 16, 48, 0.3), right(2, 32, 32, [0.97, 0.9995], rot(32, 500.0, scaling(2.0, 2.0, 8.0, 128)))),
    layer(left(3, 1, 24, 24, 0.2, 3.0, 7, rot(24, 77.0)), right(1, 8, 8, [1.0]), moe(4, 4, 16), 1.0, 0.5)],
    residual_mult=0.7, loop=(1, 3, 2))
# no loop, no residual constant, a width and head sizes that are no multiples of 8 (the products of the 32-bit kind
# on both paths), one expert per token, a window of one page exactly, a window of one (a token sees itself only)
V2 = config(257, 100, 3e-6, [
    layer(left(5, 5, 20, 12, 0.22, 30.0, 64, rot(10, 1000.0)), right(2, 10, 30, [0.95, 0.999], rot(4, 10.0)),
          moe(5, 1, 28, 36)),
    layer(left(2, 1, 34, 6, 0.17, None, 1, rot(34, 50000.0, scaling(8.0, 1.0, 4.0, 2048))), right(4, 12, 4, [0.5, 0.9, 0.99, 0.999]),
          moe(3, 2, 20))])
# whole model looped three times; windows just below and above a page; many experts (more than a warp's lanes)
V3 = config(150, 64, 1e-6, [
    layer(left(2, 1, 16, 32, 0.25, 10.0, 63, rot(16, 300.0)), right(2, 16, 16, [0.98, 0.999], rot(16, 1e6)),
          moe(40, 3, 8, 16), 0.6, 0.5),
    layer(left(4, 4, 8, 8, 0.35, 5.0, 65, rot(4, 20.0)), right(1, 32, 64, [0.995]), None, 1.5, 0.25)],
    residual_mult=0.5, loop=(0, 2, 3))
# peaked attention: a large scale under a wide cap, so that one key decides a query's output; a window that passes
# over page borders; nothing else in the layer hides the attention (the retention's weight is small)
SHARP = config(200, 64, 1e-5, [
    layer(left(4, 2, 32, 32, 2.0, 40.0, 100, rot(32, 10000.0)), right(1, 8, 8, [0.9]), None, 1.0, 0.05),
    layer(left(2, 2, 16, 16, 1.5, None, 33, rot(8, 100.0)), right(2, 16, 16, [0.99, 0.999], rot(16, 1000.0)),
          moe(4, 2, 32, 32), 1.0, 1.0)])
# retention alone decides: the attention's weight is small, the decays are close to one
LONG_MEMORY = config(180, 48, 1e-5, [
    layer(left(1, 1, 8, 8, 0.3, None, 4), right(3, 16, 16, [0.999, 0.9999, 1.0], rot(16, 10000.0)), None, 0.05, 1.0)])
# head sizes of real models at a width of 1,024: the tensor-core products and attention kernels
REAL = config(1000, 1024, 1e-6, [
    layer(left(8, 2, 128, 64, 0.09, 50.0, 256, rot(128, 500000.0, scaling(8.0, 1.0, 4.0, 8192))),
          right(8, 64, 128, [1 - 2.0 ** -(5 + i) for i in range(8)], rot(64, 10000.0)), moe(8, 2, 256, 512), 0.7, 0.7),
    layer(left(16, 16, 64, 64, 0.125, None, 100, rot(32, 10000.0)), right(4, 128, 64, [0.97, 0.99, 0.997, 0.999], rot(128, 1e6)),
          moe(16, 4, 128)),
    layer(left(4, 1, 64, 128, 0.125, 20.0, None, rot(64, 10000.0)), right(2, 256, 32, [0.99, 0.999]), None)],
    residual_mult=0.5, loop=(0, 1, 2))

ALL = {"V1": (V1, 3), "V2": (V2, 4), "V3": (V3, 5), "SHARP": (SHARP, 6), "LONG_MEMORY": (LONG_MEMORY, 8)}


def write(folder, raw, seed, std=0.1):
    """A model folder of seeded random weights, the router's scaled up."""
    from oracle_engine_b200.config.fovirax import FoviraxConfig
    from oracle_engine_b200.weights.random_init import write_model_folder
    from oracle_engine_b200.weights.safetensors_io import ModelFiles, write_safetensors
    folder = Path(folder)
    write_model_folder(folder, FoviraxConfig.from_dict(raw), seed=seed, std=std)
    files = ModelFiles(folder)
    tensors = {}
    for n in files.names():
        t = files.read(n).clone()
        f = t.float()
        if n.endswith(".router"):
            f = f * 4.0                           # logits well apart: few choices hang on a rounding
        tensors[n] = f.to(t.dtype)
    files.close()
    write_safetensors(folder / "model.safetensors", tensors)
    return str(folder)
