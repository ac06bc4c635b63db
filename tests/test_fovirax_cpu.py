"""The Fovirax design without a GPU: configuration, the model as data (schedule, tensors, cache and state needs),
and the plain model's own mechanisms."""
import copy
import math

import pytest
import torch

import fovirax_models as fm
import plain_fovirax as pf


def _build(raw):
    from oracle_engine_b200.config.base import get_architecture
    from oracle_engine_b200.config.fovirax import FoviraxConfig
    from oracle_engine_b200.engine.runtime import Runtime
    from oracle_engine_b200.parts.model import DecoderModel
    cfg = FoviraxConfig.from_dict(raw)
    spec = get_architecture("Fovirax").build_spec(cfg)
    return cfg, spec, DecoderModel(spec, Runtime(torch.float32, torch.device("cpu")))


@pytest.mark.parametrize("name", list(fm.ALL) + ["REAL"])
def test_configuration_round_trip_and_schedule(name):
    raw = fm.REAL if name == "REAL" else fm.ALL[name][0]
    from oracle_engine_b200.config.fovirax import FoviraxConfig
    cfg, spec, model = _build(raw)
    assert FoviraxConfig.from_dict(cfg.to_dict()) == cfg
    assert [e.layer for e in spec.schedule] == pf.layer_order(raw)
    # every run of a layer has a cache and a state of its own; repeated runs share the weights
    assert len(model.cache_needs()) == len(model.state_needs()) == len(spec.schedule)
    assert len({d.name for d in model.tensors()}) == len(model.tensors())


def test_declared_tensors_cache_and_state():
    cfg, spec, model = _build(fm.V1)
    shapes = {d.name: tuple(d.shape) for d in model.tensors()}
    assert shapes["l0.mix.left.q"] == (4 * 32, 96) and shapes["l0.mix.left.k"] == (2 * 32, 96)
    assert shapes["l0.mix.left.v"] == (2 * 16, 96) and shapes["l0.mix.left.o"] == (96, 4 * 16)
    assert shapes["l0.mix.right.q"] == (3 * 16, 96) and shapes["l0.mix.right.v"] == (3 * 24, 96)
    assert shapes["l0.mix.right.g"] == (3 * 24, 96) and shapes["l0.mix.right.o"] == (96, 3 * 24)
    assert shapes["l0.mlp.router"] == (6, 96) and shapes["l0.mlp.e5.down"] == (96, 40)
    assert shapes["l0.mlp.shared.sg"] == (1, 96) and shapes["l0.mlp.shared.gate"] == (24, 96)
    assert shapes["l0.ls1"] == shapes["l0.ls2"] == shapes["l0.norm2"] == (96,)
    assert "l1.mlp.router" not in shapes and "l1.ls2" not in shapes and "l1.norm2" not in shapes
    assert "l2.mlp.shared.sg" not in shapes and shapes["head"] == (300, 96) and shapes["final.norm"] == (96,)
    needs = model.cache_needs()
    assert needs[0].kind == "window" and needs[0].window == 40 and dict(needs[0].tensors) == {"k": (2, 32), "v": (2, 16)}
    assert needs[1].kind == "full" and dict(needs[1].tensors) == {"k": (2, 16), "v": (2, 48)}
    assert needs[1] == needs[3] and needs[2] == needs[4]            # the looped layers' second runs
    state = model.state_needs()
    assert state[0]["right.S"].shape == (3, 16, 24) and state[2]["right.S"].shape == (1, 8, 8)


def test_unknown_and_wrong_keys_are_refused():
    from oracle_engine_b200.config.base import ConfigError
    from oracle_engine_b200.config.fovirax import FoviraxConfig
    for path, value in [(("layers", 0, "mixer", "left", "sink"), True), (("layers", 0, "mlp", "router", "bias"), 1),
                        (("layers", 0, "type"), "delta"), (("layers", 0, "mixer", "right", "decay"), [0.5]),
                        (("layers", 0, "mixer", "left", "rot", "dims"), 34), (("loop", "stop"), 9),
                        (("layers", 0, "mlp", "kind"), "dense"), (("norm", "kind"), "layer")]:
        raw = copy.deepcopy(fm.V1)
        node = raw
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError):
            FoviraxConfig.from_dict(raw)
    raw = copy.deepcopy(fm.V1)
    raw["notes"] = "a file's own"                   # top-level keys beyond the design's are not read
    FoviraxConfig.from_dict(raw)


def test_library_frequencies_agree_with_plain():
    """The table builder of the package against the plain rescaling, in all three bands."""
    from oracle_engine_b200.parts.positions import rotary_inv_freq
    r = fm.V1["layers"][0]["mixer"]["left"]["rot"]
    sc = r["scaling"]
    got = rotary_inv_freq(r["dims"], r["base"], {"factor": sc["factor"], "low_freq_factor": sc["low"],
                                                 "high_freq_factor": sc["high"],
                                                 "original_max_position_embeddings": sc["original"]})
    want = pf.frequencies(r)
    plain = pf.frequencies({"dims": r["dims"], "base": r["base"]})
    assert torch.allclose(got, want, rtol=1e-12)
    ratio = (want / plain).tolist()
    assert ratio[0] == 1.0 and ratio[-1] == 1.0 / sc["factor"] and any(1.0 / sc["factor"] < x < 1.0 for x in ratio)


def test_plain_mechanisms():
    torch.manual_seed(0)
    # the rotation keeps lengths, leaves the dimensions behind `dims` alone and pairs i with i + dims/2
    a = torch.randn(5, 2, 12, dtype=torch.float64)
    pos = torch.arange(3, 8)
    b = pf.rotate(a, pos, {"dims": 8, "base": 100.0})
    assert torch.allclose((a * a).sum(-1), (b * b).sum(-1)) and torch.equal(a[..., 8:], b[..., 8:])
    one = torch.zeros(1, 1, 12, dtype=torch.float64)
    one[0, 0, 1] = 1.0
    t = pf.rotate(one, torch.tensor([2]), {"dims": 8, "base": 100.0})[0, 0]
    ang = 2 * 100.0 ** (-2.0 / 8)
    assert abs(t[1] - math.cos(ang)) < 1e-12 and abs(t[5] - math.sin(ang)) < 1e-12 and t[[0, 2, 3, 4, 6, 7]].abs().max() == 0
    # routing: the largest logits, weights that sum to one and follow the logits' order
    idx, wt = pf.route(torch.tensor([[0.1, 2.0, -1.0, 1.5]], dtype=torch.float64), 2)
    assert idx.tolist() == [[1, 3]] and abs(wt.sum().item() - 1) < 1e-12
    assert abs(wt[0, 0].item() - 1 / (1 + math.exp(-0.5))) < 1e-12
    # retention with one head: o_t = sum_j gamma^(t-j) (q_t . k_j) v_j / sqrt(d) before the norm
    D, d, dv, T = 6, 4, 3, 7
    W = {"q": torch.randn(d, D, dtype=torch.float64), "k": torch.randn(d, D, dtype=torch.float64),
         "v": torch.randn(dv, D, dtype=torch.float64), "g": torch.randn(dv, D, dtype=torch.float64),
         "o": torch.eye(dv, dtype=torch.float64)}
    h = torch.randn(T, D, dtype=torch.float64)
    m = {"heads": 1, "dim": d, "vdim": dv, "decay": [0.8], "rot": None}
    got = pf.retention(h, W, "", m, 1e-6)
    q, k, v = h @ W["q"].T, h @ W["k"].T / 2.0, h @ W["v"].T
    o = torch.stack([sum(0.8 ** (t - j) * (q[t] @ k[j]) * v[j] for j in range(t + 1)) for t in range(T)])
    want = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-6) * pf.silu(h @ W["g"].T)
    assert torch.allclose(got, want, atol=1e-12)
    # the window: with a window of one a token's attention is its own value
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": dv, "scale": 0.5, "softcap": 2.0, "mask": {"size": 1}, "rot": None}
    assert torch.allclose(pf.window_attention(h, W, "", m), h @ W["v"].T, atol=1e-12)
