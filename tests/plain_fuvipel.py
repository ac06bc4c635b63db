"""A plain, slow Fuvipel: one function per mechanism, float64 on the CPU, token by token.

It shares no code with the package: it reads config.json and the safetensors file by
itself (through torch only) and follows the equations below literally.

Notation.  x_t is the residual stream at token t (width D).  A layer is
    x <- x + N1(M(x));   x <- x + N2(F(x))          (the second only if it has a feed-forward)
with N(y) = y / sqrt(mean(y^2) + eps) * w.  The sublayers read x itself.

Mixer "delta" (gated delta rule), per token with input h:
    q~ = conv(Wq h), k~ = conv(Wk h), v~ = conv(Wv h)      causal, per channel, then silu
    q = unit(q~) / sqrt(dk), k = unit(k~)                  unit(a) = a / sqrt(|a|^2 + 1e-6), per head
    beta = sigmoid(Wb h), g = exp(-exp(A) softplus(Wa h + dt))        one per value head
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q     S is [dk, dv] per value head
    y = Wo (rms(o) * w_norm * silu(Wg h))

Mixer "parallel": y = (N_left(A(h)) + N_right(R(h))) / 2 with
  A, attention with a sink: q = Wq h, k = Wk h, values = k as projected; q, k rotated on the first
    `dims` dimensions (pairs (2i, 2i+1), angle p * base^(-2i/dims)), then divided by their root mean
    square per head; s_j = scale q.k_j for j <= t; p_j = exp(s_j) / (1 + sum_j exp(s_j));
    A = Wo (sigmoid(Wg h) * concat_h sum_j p_j v_j).
  R, time mixing with per-channel decay: with h' the previous token's h (0 at the start),
    m_s = h + (h' - h) mu_s for s in r, k, v, g, w; r, k, v = W m; gate = silu(Wg m_g);
    w = exp(-exp(W2 tanh(W1 m_w) + w0));
    o = (S + diag(u) k v^T)^T r;  S <- diag(w) S + k v^T;
    R = Wo (rms_per_head(o) * w_norm * gate).

Feed-forward "dense": F(h) = Wdown relu(Wup h)^2.  Logits = E N_final(x) with E the embedding table.
"""
import json
import math
import struct
from pathlib import Path

import torch

F64 = torch.float64


def read_safetensors(path):
    """name -> float64 tensor (bfloat16 / float32 / float16 payloads)."""
    raw = Path(path).read_bytes()
    n = struct.unpack("<Q", raw[:8])[0]
    head = json.loads(raw[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16}
    out = {}
    for name, info in head.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = bytearray(raw[8 + n + lo: 8 + n + hi])
        out[name] = torch.frombuffer(buf, dtype=kinds[info["dtype"]]).reshape(info["shape"]).to(F64)
    return out


def rms(y, eps):
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def short_conv(seq, taps_w):
    """seq [T, C], taps_w [C, taps] (last column weighs the current token), zeros before the start."""
    T, C = seq.shape
    taps = taps_w.shape[1]
    out = torch.zeros_like(seq)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += taps_w[:, j] * seq[s]
    return out


def delta_mixer(h, W, p, m, eps):
    """h [T, D]; W the tensors; p the prefix '<layer>.mix.'; m the mixer's sizes."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, dk)
    k = silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, dk)
    v = silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) / math.sqrt(dk)
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    g = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    gate = silu(h @ W[p + "g"].T).reshape(T, H, dv)
    S = torch.zeros(H, dk, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for hh in range(H):
            kh, qh = k[t, hh // (H // G)], q[t, hh // (H // G)]
            S[hh] = g[t, hh] * S[hh]
            u = beta[t, hh] * (v[t, hh] - S[hh].T @ kh)
            S[hh] = S[hh] + torch.outer(kh, u)
            o[t, hh] = S[hh].T @ qh
    y = rms(o, eps) * W[p + "norm"] * gate
    return y.reshape(T, H * dv) @ W[p + "o"].T


def rotate_pairs(a, pos, dims, base):
    """a [T, heads, d]: pairs (2i, 2i+1) of the first `dims` dimensions turned by pos * base^(-2i/dims)."""
    out = a.clone()
    for i in range(dims // 2):
        ang = pos.to(F64) * (base ** (-2.0 * i / dims))
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        u, v = a[..., 2 * i], a[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def sink_attention(h, W, p, m, eps, pos0=0):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(pos0, pos0 + T)
    q = (h @ W[p + "q"].T).reshape(T, H, d)
    kraw = (h @ W[p + "k"].T).reshape(T, G, d)
    rot = m.get("rot")
    qr, kr = q, kraw
    if rot:
        qr = rotate_pairs(q, pos, rot["dims"], rot["base"])
        kr = rotate_pairs(kraw, pos, rot["dims"], rot["base"])
    qn, kn = rms(qr, eps), rms(kr, eps)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            s = (kn[:t + 1, g] @ qn[t, hh]) * m["scale"]
            e = torch.exp(s)
            pr = e / (1.0 + e.sum())
            o[t, hh] = pr @ kraw[:t + 1, g]
    gate = torch.sigmoid(h @ W[p + "g"].T)
    return (o.reshape(T, H * dv) * gate) @ W[p + "o"].T


def time_mix(h, W, p, m, eps):
    T, D = h.shape
    H, d = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, D, dtype=F64), h[:-1]], 0)
    mix = {s: h + (prev - h) * W[p + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ W[p + "r"].T).reshape(T, H, d)
    k = (mix["k"] @ W[p + "k"].T).reshape(T, H, d)
    v = (mix["v"] @ W[p + "v"].T).reshape(T, H, d)
    gate = silu(mix["g"] @ W[p + "g"].T)
    w = torch.exp(-torch.exp(torch.tanh(mix["w"] @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).reshape(T, H, d)
    u = W[p + "u"]
    S = torch.zeros(H, d, d, dtype=F64)
    o = torch.zeros(T, H, d, dtype=F64)
    for t in range(T):
        for hh in range(H):
            kv = torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = (S[hh] + u[hh][:, None] * kv).T @ r[t, hh]
            S[hh] = w[t, hh][:, None] * S[hh] + kv
    y = rms(o, eps).reshape(T, H * d) * W[p + "norm"] * gate
    return y @ W[p + "o"].T


def parallel_mixer(h, W, p, m, eps):
    a = rms(sink_attention(h, W, p + "left.", m["left"], eps), eps) * W[p + "left.out"]
    b = rms(time_mix(h, W, p + "right.", m["right"], eps), eps) * W[p + "right.out"]
    return 0.5 * (a + b)


def dense_ff(h, W, p):
    z = torch.relu(h @ W[p + "up"].T)
    return (z * z) @ W[p + "down"].T


MIXERS = {"delta": delta_mixer, "parallel": parallel_mixer}


class PlainFuvipel:
    def __init__(self, folder):
        self.cfg = json.loads((Path(folder) / "config.json").read_text())
        self.W = read_safetensors(Path(folder) / "model.safetensors")
        self.eps = float(self.cfg["norm"]["eps"])

    def forward(self, tokens, layers_out=None):
        """tokens: list of ids -> logits [T, vocab] (float64).  layers_out: a list that receives the
        residual stream after every layer."""
        W, eps = self.W, self.eps
        x = W["embed"][torch.as_tensor(tokens)]
        for i, layer in enumerate(self.cfg["layers"]):
            p = f"l{i}."
            y = MIXERS[layer["type"]](x, W, p + "mix.", layer["mixer"], eps)
            x = x + rms(y, eps) * W[p + "norm1"]
            if layer.get("mlp") is not None:
                assert layer["mlp"]["kind"] == "dense"
                x = x + rms(dense_ff(x, W, p + "mlp."), eps) * W[p + "norm2"]
            if layers_out is not None:
                layers_out.append(x.clone())
        return (rms(x, eps) * W["final.norm"]) @ W["embed"].T

    def logits(self, tokens):
        return self.forward(tokens)


def generate(model, prompt, n):
    """n greedy tokens (first maximum), recomputing the whole sequence for each."""
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(torch.argmax(model.forward(seq)[-1]).item()))
    return seq[len(prompt):]
