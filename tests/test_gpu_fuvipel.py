"""The Fuvipel design on the GPU against the plain float64 model of tests/plain_fuvipel.py: every layer by
itself, whole prompts, token-by-token decoding, prompts in pieces, ragged batches, reused slots, keys at
page borders under a peaked softmax, and greedy generation through Engine.generate and the command line."""
import subprocess
import sys

import numpy as np
import pytest
import torch

import fuvipel_models as fm
import helpers
import plain_fuvipel as pf

pytestmark = pytest.mark.gpu

# A position's error is the root mean square over the vocabulary of the difference of its logits, relative to
# the root mean square of the request's logits.  float32: rounding of a few hundred fused multiply-adds per
# value; bfloat16: activations rounded to 2^-9 relative at every product, a few dozen products deep.
TOL = {"float32": 1e-4, "bfloat16": 5e-2}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (raw, seed) in fm.ALL.items():
        d = fm.write(tmp_path_factory.mktemp(f"fuvipel_{name}"), raw, seed)
        out[name] = (d, pf.PlainFuvipel(d))
    return out


def _engine(folder, dtype, **kw):
    from oracle_engine_b200.engine.engine import Engine
    kw.setdefault("max_tokens", 1024)
    return Engine.from_pretrained(folder, dtype=dtype, **kw)


def _compare(got, plain, requests, tol, what, cache={}):
    for i, toks in enumerate(requests):
        key = (id(plain), tuple(toks))
        if key not in cache:
            cache[key] = plain.logits(toks).numpy()
        want = cache[key]
        assert not np.isnan(got[i]).any(), f"{what}: request {i} has positions without logits"
        err = np.sqrt(((got[i] - want) ** 2).mean(axis=1)) / np.sqrt((want ** 2).mean())
        assert err.max() < tol, f"{what}: request {i} (len {len(toks)}) first bad position " \
                                f"{int((err >= tol).argmax())}, worst {int(err.argmax())}: {err.max()}"


@pytest.mark.parametrize("name", ["F1", "F2", "F3", "F4"])
def test_every_layer_by_itself_float32(models, name):
    """The residual stream after each layer of a whole prompt, in float32, against the plain model."""
    from oracle_engine_b200 import SequenceStep
    folder, plain = models[name]
    eng = _engine(folder, "float32", use_graphs=False)
    seen = []
    for layer in eng.model.layers:
        def fwd(x, *a, _orig=layer.forward, **k):
            _orig(x, *a, **k)
            seen.append(x.detach().double().cpu())
        layer.forward = fwd
    toks = helpers.random_tokens(150, plain.cfg["vocab"], 9)
    slot = eng.alloc()
    eng.step([SequenceStep(slot, toks, [len(toks) - 1])])
    want = []
    plain.forward(toks, want)
    assert len(seen) == len(want) == len(plain.cfg["layers"])
    for i, (a, b) in enumerate(zip(seen, want)):
        err = (a - b).abs().max().item()
        assert err < 2e-4 * max(1.0, b.abs().max().item()), f"{name}: layer {i} ({plain.cfg['layers'][i]['type']}) differs by {err}"


@pytest.mark.parametrize("branch", ["left", "right"])
def test_each_branch_of_a_parallel_layer_alone(tmp_path, branch):
    """With the other branch's output projection at zero, a parallel layer is one mixer (times one half)."""
    from oracle_engine_b200.weights.safetensors_io import ModelFiles, write_safetensors
    folder = fm.write(tmp_path / "m", fm.F2, 21)
    files = ModelFiles(folder)
    tensors = {n: files.read(n).clone() for n in files.names()}
    files.close()
    other = "right" if branch == "left" else "left"
    for n in tensors:
        if n.endswith(f"mix.{other}.o"):
            tensors[n].zero_()
    write_safetensors(tmp_path / "m" / "model.safetensors", tensors)
    plain = pf.PlainFuvipel(folder)
    toks = helpers.random_tokens(90, plain.cfg["vocab"], 5)
    for dtype in ("float32", "bfloat16"):
        eng = _engine(folder, dtype)
        steps = helpers.whole_steps([toks])
        got = helpers.collect(steps, helpers.TraceRunner(eng, tmp_path / dtype).run(steps), [toks])
        _compare(got, plain, [toks], TOL[dtype], f"{branch} alone {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["F1", "F2", "F3", "F4"])
def test_whole_decoded_pieces_and_batches_agree_with_plain(models, tmp_path, name, dtype):
    folder, plain = models[name]
    vocab = plain.cfg["vocab"]
    lens = [130, 65, 1, 200, 37, 2, 64, 129]
    requests = [helpers.random_tokens(n, vocab, 300 + i) for i, n in enumerate(lens)]
    eng = _engine(folder, dtype)
    runs = {}
    # each alone and whole; each alone decoded token by token from the first token (or after a prompt)
    runs["whole"] = helpers.whole_steps(requests)
    runs["decoded"] = helpers.tail_steps(requests, 1000)
    runs["tail"] = helpers.tail_steps(requests, 40)
    # in pieces down to two tokens and one
    runs["pieces"] = helpers.piece_steps(requests, [helpers.cut(n, [2, 37, 1, 64, 3, 65]) for n in lens], batch_size=1)
    # ragged batches of three, prompts then one token each; the next batch takes the slots they leave
    runs["batched"] = helpers.batched_steps(requests, [max(1, n - 20) for n in lens], 3)
    # steps that mix a prompt piece of one request with single tokens of others
    runs["mixed"] = helpers.piece_steps(requests, [helpers.cut(n, [1, 1, 30, 1, 2, 70][i % 3:] + [5]) for i, n in enumerate(lens)],
                                        batch_size=3)
    got = {}
    for k, steps in runs.items():
        got[k] = helpers.collect(steps, helpers.TraceRunner(eng, tmp_path / k).run(steps), requests)
        eng.cache.check()
        assert eng.cache.slots.n_free == eng.cache.n_slots
    for k in got:
        _compare(got[k], plain, requests, TOL[dtype], f"{name} {dtype} {k}")
    if dtype == "float32":
        # a position's logits do not depend on the cut or the batch: the same instructions in the same order
        for k in got:
            for i in range(len(requests)):
                assert np.array_equal(got["whole"][i], got[k][i]), f"{name} float32: {k} differs from whole, request {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["DELTA_ONLY", "PARALLEL_ONLY"])
def test_models_of_one_kind_of_layer(models, tmp_path, name, dtype):
    """Only recurrent layers (no paged cache at all) and only parallel layers: prompts, decoding, a ragged batch."""
    folder, plain = models[name]
    lens = [70, 3, 130]
    requests = [helpers.random_tokens(n, plain.cfg["vocab"], 610 + i) for i, n in enumerate(lens)]
    eng = _engine(folder, dtype, max_tokens=512)
    assert len(eng.cache.groups) == (0 if name == "DELTA_ONLY" else 2)         # two attentions of different key sizes
    for k, steps in {"tail": helpers.tail_steps(requests, 10), "batched": helpers.batched_steps(requests, [60, 1, 66], 3)}.items():
        got = helpers.collect(steps, helpers.TraceRunner(eng, tmp_path / k).run(steps), requests)
        _compare(got, plain, requests, TOL[dtype], f"{name} {dtype} {k}")
    eng.cache.check()
    assert eng.cache.slots.n_free == eng.cache.n_slots


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_and_page_borders_under_a_peaked_softmax(models, tmp_path, dtype):
    """Prompts that end just before, at and just after a page border, decoded across the next one, with an
    attention in which single keys (far ones too) decide: a lost or misplaced key changes the logits."""
    folder, plain = models["SHARP"]
    vocab = plain.cfg["vocab"]
    # the softmax is peaked: the largest weight of the last token's heads is well above uniform
    toks = helpers.random_tokens(300, vocab, 77)
    W, m = plain.W, plain.cfg["layers"][0]["mixer"]["left"]
    x = W["embed"][torch.as_tensor(toks)]
    q = (x @ W["l0.mix.left.q"].T).reshape(300, m["heads"], m["dim"])
    k = (x @ W["l0.mix.left.k"].T).reshape(300, m["kv_heads"], m["dim"])
    pos = torch.arange(300)
    qn = pf.rms(pf.rotate_pairs(q, pos, m["rot"]["dims"], m["rot"]["base"]), plain.eps)
    kn = pf.rms(pf.rotate_pairs(k, pos, m["rot"]["dims"], m["rot"]["base"]), plain.eps)
    s = (kn[:, 0] @ qn[-1, 0]) * m["scale"]
    p = torch.exp(s - s.max())
    assert (p / p.sum()).max() > 0.2 and int(s.argmax()) < 250
    lens = [63, 64, 65, 127, 128, 129, 300]
    requests = [toks[:n] for n in lens]
    eng = _engine(folder, dtype)
    runs = {"whole": helpers.whole_steps(requests),
            "tail": helpers.tail_steps(requests, 6),
            "pieces": helpers.piece_steps(requests, [helpers.cut(n, [62, 2, 1, 63, 64]) for n in lens], batch_size=2)}
    for kname, steps in runs.items():
        got = helpers.collect(steps, helpers.TraceRunner(eng, tmp_path / kname).run(steps), requests)
        _compare(got, plain, requests, TOL[dtype] * 2, f"SHARP {dtype} {kname}")
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_head_sizes(tmp_path, dtype):
    """Head sizes 128 and 64 at a width of 1,024: in bfloat16 the prompts go through the tensor-core products and
    the tensor-memory attention, decoding through the kernel that splits the keys; states of 128 x 128."""
    folder = fm.write(tmp_path / "m", fm.REAL, 31, std=0.05)
    plain = pf.PlainFuvipel(folder)
    lens = [333, 70, 200]
    requests = [helpers.random_tokens(n, 1000, 800 + i) for i, n in enumerate(lens)]
    eng = _engine(folder, dtype, max_tokens=2048)
    runs = {"batched": helpers.batched_steps(requests, [n - 6 for n in lens], 3),
            "pieces": helpers.piece_steps(requests, [helpers.cut(n, [150, 2, 100]) for n in lens], batch_size=1)}
    for k, steps in runs.items():
        got = helpers.collect(steps, helpers.TraceRunner(eng, tmp_path / k).run(steps), requests)
        _compare(got, plain, requests, TOL[dtype], f"REAL {dtype} {k}")
    # decoding over a handful of keys, where the sink is a large share of the softmax's denominator: one request
    # and three together, from the first token on (the decode kernels, with and without split keys)
    short = [r[:9] for r in requests]
    for k, steps in {"short_alone": helpers.tail_steps(short[:1], 1000),
                     "short_batch": helpers.batched_steps(short, [1, 2, 3], 3)}.items():
        reqs = short[:1] if k == "short_alone" else short
        got = helpers.collect(steps, helpers.TraceRunner(eng, tmp_path / k).run(steps), reqs)
        _compare(got, plain, reqs, TOL[dtype], f"REAL {dtype} {k}")
    eng.check_device_errors()
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slots_and_pages_are_used_again(models, tmp_path, dtype):
    """Two slots for six requests: a request that starts in a slot another left reads nothing of it."""
    folder, plain = models["F1"]
    vocab = plain.cfg["vocab"]
    lens = [70, 40, 90, 66, 5, 120]
    requests = [helpers.random_tokens(n, vocab, 500 + i) for i, n in enumerate(lens)]
    eng = _engine(folder, dtype, max_tokens=256, n_slots=2)
    steps = helpers.batched_steps(requests, [max(1, n - 8) for n in lens], 2)
    got = helpers.collect(steps, helpers.TraceRunner(eng, tmp_path / "t").run(steps), requests)
    _compare(got, plain, requests, TOL[dtype], f"reuse {dtype}")
    eng.cache.check()
    assert eng.cache.slots.n_free == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_generate(models, dtype):
    """Greedy generation through Engine.generate (scheduler, sampler, step ahead) against the plain model."""
    from oracle_engine_b200 import GenParams
    folder, plain = models["F2"]
    vocab = plain.cfg["vocab"]
    eng = _engine(folder, dtype)
    prompts = [helpers.random_tokens(n, vocab, 40 + i) for i, n in enumerate((1, 9, 70))]
    n_new = 80
    got = eng.generate(prompts, GenParams.greedy(n_new, ignore_eos=True))
    assert [len(g) for g in got] == [n_new] * 3
    margin = 1e-3 if dtype == "float32" else 2 * TOL[dtype]
    for p, g in zip(prompts, got):
        lg = plain.logits(list(p) + list(g))
        for j, tok in enumerate(g):
            row = lg[len(p) + j - 1]
            assert row.max().item() - row[tok].item() <= margin, f"{dtype}: token {j} of a prompt of {len(p)}"
    # a budget of prompt tokens per step: the 70-token prompt goes through in portions beside decoding rows
    again = eng.generate(prompts, GenParams.greedy(12, ignore_eos=True), max_step_tokens=16)
    if dtype == "float32":
        assert again == [g[:12] for g in got]
    eng.cache.check()
    assert eng.cache.slots.n_free == eng.cache.n_slots


def test_command_lines(models, tmp_path):
    """bin/trace_run and bin/oracle load the design by its config.json."""
    folder, plain = models["F3"]
    vocab = plain.cfg["vocab"]
    requests = [helpers.random_tokens(n, vocab, 900 + i) for i, n in enumerate((20, 66))]
    steps = helpers.batched_steps(requests, [15, 60], 2)
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        helpers.run_trace_cli(folder, dtype, steps, out, 256)
        files = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab) for s in steps}
        got = helpers.collect(steps, files, requests)
        _compare(got, plain, requests, TOL[dtype], f"trace_run {dtype}")
    prompt = requests[0][:12]
    r = subprocess.run([sys.executable, str(helpers.ROOT / "bin" / "oracle"), "-m", folder, "--tokens",
                        ",".join(map(str, prompt)), "-n", "6", "--temp", "0", "--dtype", "float32", "--ignore-eos"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [int(t) for t in r.stdout.split()] == pf.generate(plain, prompt, 6)
