"""A plain, slow Fovirax: one function per mechanism, float64 on the CPU.

It shares no code with the package: it reads config.json and the safetensors file by itself
(through torch only) and follows the equations below literally.

Notation.  x_t is the residual stream at token t (width D), p its position in its sequence.
    N(x; w) = x / sqrt(mean(x^2) + eps) * (1 + w)                     the norm's weight is kept around zero
    layer:   x <- x + m * s1 * M(N(x; w1));   x <- x + m * s2 * F(N(x; w2))       (F only if the layer has one)
with m one number of the model and s1, s2 one vector of the layer each.  The layers named by `loop`
(start .. stop - 1) run `times` times as a group before the layers behind them run.

Mixer "parallel":  M(h) = a * A(h) + b * R(h), a and b from the configuration.
  A, windowed grouped-query attention with capped scores.  q = Wq h [H, d], k = Wk h [G, d], v = Wv h [G, dv].
    rot(u, p): the first `dims` dimensions of a head are paired (i, i + dims/2) and each pair is turned by the
    angle p * f_i, f_i = base^(-2i/dims), the f_i optionally rescaled by wavelength (three bands).
    s_j = c * tanh(scale * rot(q, t) . rot(k_j, j) / c) for t - window < j <= t;  softmax over those j;
    A = Wo concat_h sum_j p_j v_j.
  R, retention.  q = Wq h, k = Wk h [H, d], v = Wv h [H, dv], q and k turned as above, k times d^(-1/2);
    S <- gamma_h S + k v^T;  o = S^T q;  R = Wo (concat_h o / sqrt(mean(o^2) + eps) * silu(Wg h)).

Feed-forward "moe":  z = Wr h; the `top` largest z choose experts, their weights are the softmax over those
z alone; F = sum_e w_e E_e(h) + sigmoid(Wsg h) * E_shared(h), with E(h) = Wdown (silu(Wgate h) * (Wup h)).

Logits = Whead N(x; w_final).
"""
import json
import math
import struct
from pathlib import Path

import torch

F64 = torch.float64


def read_safetensors(path):
    raw = Path(path).read_bytes()
    n = struct.unpack("<Q", raw[:8])[0]
    head = json.loads(raw[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    out = {}
    for name, info in head.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = bytearray(raw[8 + n + lo: 8 + n + hi])
        t = torch.frombuffer(buf, dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t.to(F64) if t.is_floating_point() else t.clone()
    return out


def norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def frequencies(rot):
    """The turning rates f_i of a rotation, i < dims/2, after the optional rescaling by wavelength."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        out = []
        for fi in f:
            wave = 2.0 * math.pi / fi
            if wave < sc["original"] / sc["high"]:
                out.append(fi)
            elif wave > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * fi / sc["factor"] + s * fi)
        f = out
    return torch.tensor(f, dtype=F64)


def rotate(a, pos, rot):
    """a [T, heads, d], pos [T]: dimension i < dims/2 is paired with i + dims/2."""
    if not rot or not rot.get("dims"):
        return a
    half = rot["dims"] // 2
    ang = pos.to(F64)[:, None] * frequencies(rot)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = a[..., :half], a[..., half:2 * half]
    out = a.clone()
    out[..., :half] = u * c - v * s
    out[..., half:2 * half] = v * c + u * s
    return out


def window_attention(h, W, p, m, pos0=0):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(pos0, pos0 + T)
    q = rotate((h @ W[p + "q"].T).reshape(T, H, d), pos, m.get("rot"))
    k = rotate((h @ W[p + "k"].T).reshape(T, G, d), pos, m.get("rot"))
    v = (h @ W[p + "v"].T).reshape(T, G, dv)
    cap = m.get("softcap")
    window = (m.get("mask") or {}).get("size")
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        lo = 0 if not window else max(0, t - window + 1)
        for hh in range(H):
            g = hh // (H // G)
            s = (k[lo:t + 1, g] @ q[t, hh]) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            o[t, hh] = torch.softmax(s, 0) @ v[lo:t + 1, g]
    return o.reshape(T, H * dv) @ W[p + "o"].T


def retention(h, W, p, m, eps, pos0=0):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(pos0, pos0 + T)
    q = rotate((h @ W[p + "q"].T).reshape(T, H, d), pos, m.get("rot"))
    k = rotate((h @ W[p + "k"].T).reshape(T, H, d), pos, m.get("rot")) * d ** -0.5
    v = (h @ W[p + "v"].T).reshape(T, H, dv)
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for hh in range(H):
            S[hh] = m["decay"][hh] * S[hh] + torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ q[t, hh]
    y = norm(o, None, eps).reshape(T, H * dv) * silu(h @ W[p + "g"].T)
    return y @ W[p + "o"].T


def parallel_mixer(h, W, p, m, eps):
    return m["left_scale"] * window_attention(h, W, p + "left.", m["left"]) + \
        m["right_scale"] * retention(h, W, p + "right.", m["right"], eps)


def expert(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(z, top):
    """z [T, E] -> (indices [T, top], weights [T, top]): the largest `top`, softmax over them alone."""
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, -1)


def moe(h, W, p, m):
    T = h.shape[0]
    idx, wt = route(h @ W[p + "router"].T, m["router"]["top"])
    out = torch.zeros(T, W[p + "e0.down"].shape[0], dtype=F64)
    for t in range(T):
        for j in range(idx.shape[1]):
            out[t] += wt[t, j] * expert(h[t:t + 1], W, f"{p}e{int(idx[t, j])}.")[0]
    if m.get("shared"):
        out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * expert(h, W, p + "shared.")
    return out


def layer_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


class PlainFovirax:
    def __init__(self, folder):
        self.cfg = json.loads((Path(folder) / "config.json").read_text())
        self.W = read_safetensors(Path(folder) / "model.safetensors")
        self.eps = float(self.cfg["norm"]["eps"])

    def forward(self, tokens, layers_out=None):
        """tokens: list of ids -> logits [T, vocab] (float64).  layers_out: a list that receives the residual
        stream after every layer run."""
        W, eps, cfg = self.W, self.eps, self.cfg
        m = cfg.get("residual_mult", 1.0)
        x = W["embed"][torch.as_tensor(tokens)]
        for i in layer_order(cfg):
            layer, p = cfg["layers"][i], f"l{i}."
            assert layer["type"] == "parallel"
            y = parallel_mixer(norm(x, W[p + "norm1"], eps), W, p + "mix.", layer["mixer"], eps)
            x = x + m * W[p + "ls1"] * y
            if layer.get("mlp") is not None:
                assert layer["mlp"]["kind"] == "moe"
                x = x + m * W[p + "ls2"] * moe(norm(x, W[p + "norm2"], eps), W, p + "mlp.", layer["mlp"])
            if layers_out is not None:
                layers_out.append(x.clone())
        return norm(x, W["final.norm"], eps) @ W["head"].T

    def logits(self, tokens):
        return self.forward(tokens)


def generate(model, prompt, n):
    """n greedy tokens (first maximum), recomputing the whole sequence for each."""
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(torch.argmax(model.forward(seq)[-1]).item()))
    return seq[len(prompt):]
