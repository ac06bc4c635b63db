"""Small Fuvipel configurations for the tests, and a writer of model folders with weights that make faults
show: slow decays (a recurrent state that remembers hundreds of tokens), mixing weights inside (0, 1)."""
from pathlib import Path

import torch


def delta(heads, kv_heads, dim, vdim, conv, ff=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def parallel(heads, kv_heads, dim, scale, rot, r_heads, r_dim, rank, ff=None):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "rot": rot},
                      "right": {"heads": r_heads, "dim": r_dim, "rank": rank}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(vocab, width, eps, layers):
    return {"architecture": "Fuvipel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# a parallel layer first, grouped keys, a partial rotation, three taps, feed-forwards on delta layers
F1 = config(300, 96, 1e-5, [
    parallel(4, 2, 32, 0.3, {"dims": 16, "base": 10000.0}, 3, 32, 8, ff=160),
    delta(4, 4, 16, 48, 3, ff=128),
    delta(2, 1, 64, 32, 2)])
# five taps, value heads three to a key head, head sizes that are no powers of two, a parallel layer
# without feed-forward, an attention without rotation, single heads
F2 = config(257, 120, 3e-6, [
    delta(6, 2, 24, 40, 5),
    parallel(6, 6, 48, 0.144, {"dims": 48, "base": 500.0}, 5, 24, 12),
    parallel(1, 1, 64, 0.5, None, 1, 64, 16, ff=200),
    delta(1, 1, 32, 32, 4, ff=64)])
# a width the tensor-core products refuse (no multiple of 8), one tap (no convolution state), odd vocabulary
F3 = config(131, 100, 1e-6, [
    delta(5, 5, 20, 12, 1, ff=72),
    parallel(5, 1, 20, 0.25, {"dims": 4, "base": 77.0}, 2, 50, 6, ff=40)])
# sizes that are no multiples of four (scalar staging in the scans, one lane per state column), an attention
# head size the tensor-core kernels do not take, six taps, a value size above the key size
F4 = config(97, 72, 2e-5, [
    delta(3, 1, 15, 10, 6),
    parallel(2, 1, 34, 0.2, {"dims": 10, "base": 1000.0}, 3, 30, 5, ff=50),
    delta(2, 2, 8, 70, 2, ff=36)])
# one kind of layer only: a model without any paged cache, and one without delta layers
DELTA_ONLY = config(150, 64, 1e-5, [delta(2, 1, 16, 24, 3, ff=80), delta(4, 4, 8, 8, 4)])
PARALLEL_ONLY = config(150, 64, 1e-5, [parallel(2, 2, 16, 0.4, {"dims": 8, "base": 300.0}, 2, 16, 4, ff=80),
                                       parallel(4, 1, 32, 0.2, None, 1, 32, 8)])
# peaked attention: one key decides a query's output, so a key that is lost or wrong shows
SHARP = config(200, 64, 1e-5, [
    parallel(4, 2, 32, 1.0, {"dims": 32, "base": 10000.0}, 2, 32, 8),
    delta(2, 2, 32, 32, 4, ff=96)])

# head sizes of real models (128 and 64: the tensor-memory prompt attention; 128 x 128 and 64 x 64 states)
REAL = config(1000, 1024, 1e-6, [
    parallel(8, 2, 128, 0.0884, {"dims": 96, "base": 250000.0}, 16, 64, 32, ff=2048),
    delta(8, 4, 128, 128, 4),
    parallel(6, 6, 64, 0.11, {"dims": 48, "base": 10000.0}, 4, 128, 16)])

ALL = {"F1": (F1, 3), "F2": (F2, 4), "F3": (F3, 5), "F4": (F4, 7), "SHARP": (SHARP, 6), "DELTA_ONLY": (DELTA_ONLY, 8),
       "PARALLEL_ONLY": (PARALLEL_ONLY, 9)}


def write(folder, raw, seed, std=0.1, long_memory=True):
    """A model folder of seeded random weights; with long_memory the decays are moved close to one."""
    from oracle_engine_b200.config.fuvipel import FuvipelConfig
    from oracle_engine_b200.weights.random_init import write_model_folder
    from oracle_engine_b200.weights.safetensors_io import ModelFiles, write_safetensors
    folder = Path(folder)
    write_model_folder(folder, FuvipelConfig.from_dict(raw), seed=seed, std=std)
    files = ModelFiles(folder)
    tensors = {}
    for n in files.names():
        t = files.read(n).clone()
        f = t.float()
        if long_memory and (n.endswith(".A_log") or n.endswith(".w0")):
            f = f * 5.0 - 3.5                      # decays between about 0.9 and 0.999
        if ".mu." in n:
            f = 0.5 + 2.0 * f                      # mixing weights around one half
        if n.endswith(".conv") or n.endswith(".u") or n.endswith(".dt_bias"):
            f = f * 5.0
        tensors[n] = f.to(t.dtype)
    files.close()
    write_safetensors(folder / "model.safetensors", tensors)
    return str(folder)
