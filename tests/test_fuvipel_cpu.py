"""The Fuvipel design without a GPU: its config.json reader, its model description, random model folders
and the plain model's own mechanisms."""
import copy
import json

import pytest
import torch

import fuvipel_models as fm
import plain_fuvipel as pf


def test_config_round_trip_and_refusals():
    from oracle_engine_b200.config.base import ConfigError
    from oracle_engine_b200.config.fuvipel import FuvipelConfig
    for raw, _ in fm.ALL.values():
        cfg = FuvipelConfig.from_dict(raw)
        assert FuvipelConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
        assert cfg.vocab == raw["vocab"] and cfg.width == raw["width"] and cfg.norm_eps == raw["norm"]["eps"]
    noted = dict(copy.deepcopy(fm.F1), seed=3, name="a note")          # a file's own notes at the top level are not read
    assert FuvipelConfig.from_dict(noted) == FuvipelConfig.from_dict(fm.F1)
    bad = copy.deepcopy(fm.F1)
    bad["layers"][1]["type"] = "conv"
    with pytest.raises(ConfigError, match="type"):
        FuvipelConfig.from_dict(bad)
    bad = copy.deepcopy(fm.F1)
    bad["layers"][0]["mixer"]["left"]["vdim"] = 48
    with pytest.raises(ConfigError, match="vdim"):
        FuvipelConfig.from_dict(bad)
    bad = copy.deepcopy(fm.F1)
    bad["layers"][0]["mixer"]["left"]["window"] = 128
    with pytest.raises(ConfigError, match="window"):
        FuvipelConfig.from_dict(bad)
    bad = copy.deepcopy(fm.F1)
    bad["layers"][2]["mlp"] = {"kind": "routed", "ff": 8}
    with pytest.raises(ConfigError, match="kind"):
        FuvipelConfig.from_dict(bad)
    bad = copy.deepcopy(fm.F1)
    del bad["norm"]["eps"]
    with pytest.raises(ConfigError, match="eps"):
        FuvipelConfig.from_dict(bad)


def test_spec_declares_the_designs_tensors_caches_and_state(tmp_path):
    from oracle_engine_b200.config.base import load_config
    from oracle_engine_b200.engine.runtime import Runtime
    from oracle_engine_b200.parts.model import DecoderModel
    folder = fm.write(tmp_path / "m", fm.F1, 1)
    cfg, arch = load_config(folder)
    assert arch.name == "Fuvipel"
    model = DecoderModel(arch.build_spec(cfg, None), Runtime(torch.float32, torch.device("cpu")))
    names = {d.name: tuple(d.shape) for d in model.tensors()}
    stored = pf.read_safetensors(tmp_path / "m" / "model.safetensors")
    assert set(names) == set(stored)
    assert all(tuple(stored[n].shape) == s for n, s in names.items())
    assert names["l0.mix.left.k"] == (2 * 32, 96) and names["l0.mix.right.u"] == (3, 32)
    assert names["l1.mix.q.conv"] == (4 * 16, 3) and names["l1.mix.norm"] == (48,) and "l2.norm2" not in names
    assert "l0.mix.left.v" not in names                       # the values are the keys
    needs = model.cache_needs()
    assert needs[1] is None and needs[2] is None and needs[0].tensors == (("kv", (2, 2, 32)),)
    state = model.state_needs()
    assert state[0]["right.S"].shape == (3, 32, 32) and state[0]["right.prev"].shape == (96,)
    assert state[1]["S"].shape == (4, 16, 48) and state[1]["conv"].shape == (2, 2 * 4 * 16 + 4 * 48)
    assert model.stages() == [(True, 0, len(cfg.layers) + 2)]  # every part can be captured in a CUDA graph


def test_a_size_only_the_file_gives(tmp_path):
    """Without `rank` in config.json the decay projection's rank is the shape of its tensors."""
    from oracle_engine_b200.config.base import load_config
    from oracle_engine_b200.engine.runtime import Runtime
    from oracle_engine_b200.parts.model import DecoderModel
    from oracle_engine_b200.weights.loader import check_tensors
    folder = fm.write(tmp_path / "m", fm.F1, 1)
    raw = json.loads((tmp_path / "m" / "config.json").read_text())
    del raw["layers"][0]["mixer"]["right"]["rank"]
    (tmp_path / "m" / "config.json").write_text(json.dumps(raw))
    cfg, arch = load_config(folder)
    model = DecoderModel(arch.build_spec(cfg, None), Runtime(torch.float32, torch.device("cpu")))
    decl = {d.name: tuple(d.shape) for d in model.tensors()}
    assert decl["l0.mix.right.w1"] == (-1, 96) and decl["l0.mix.right.w2"] == (3 * 32, -1)
    stored = pf.read_safetensors(tmp_path / "m" / "model.safetensors")
    check_tensors({n: (torch.bfloat16, tuple(t.shape)) for n, t in stored.items()}, model.tensors())


def test_plain_mechanisms():
    torch.manual_seed(0)
    # the sink: with all scores equal to zero every one of n keys weighs 1 / (n + 1)
    D, d = 8, 4
    W = {"q": torch.zeros(d, D, dtype=pf.F64), "k": torch.randn(d, D, dtype=pf.F64),
         "g": torch.zeros(d, D, dtype=pf.F64), "o": torch.eye(d, dtype=pf.F64)}
    h = torch.randn(5, D, dtype=pf.F64)
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": d, "scale": 1.0, "rot": None}
    out = pf.sink_attention(h, W, "", m, 1e-6)
    k = h @ W["k"].T
    for t in range(5):
        assert torch.allclose(out[t], 0.5 * k[:t + 1].sum(0) / (t + 2))
    # a rotation keeps lengths, and the dimensions beyond `dims` pass unchanged
    a = torch.randn(3, 2, 8, dtype=pf.F64)
    r = pf.rotate_pairs(a, torch.tensor([0, 5, 900]), 4, 100.0)
    assert torch.equal(r[0], a[0]) and torch.equal(r[..., 4:], a[..., 4:])
    assert torch.allclose(r.norm(dim=-1), a.norm(dim=-1))
    # the convolution's last column weighs the current token, and nothing comes before the start
    seq = torch.arange(1.0, 5.0, dtype=pf.F64)[:, None]
    assert pf.short_conv(seq, torch.tensor([[100.0, 10.0, 1.0]], dtype=pf.F64)).flatten().tolist() == [1, 12, 123, 234]


def test_plain_model_runs_on_a_random_folder(tmp_path):
    folder = fm.write(tmp_path / "m", fm.F2, 2)
    plain = pf.PlainFuvipel(folder)
    toks = list(range(1, 30))
    layers = []
    lg = plain.forward(toks, layers)
    assert lg.shape == (29, 257) and torch.isfinite(lg).all() and len(layers) == 4
    # causal: a position's logits do not depend on what follows
    assert torch.allclose(plain.forward(toks[:11])[-1], lg[10])
