"""A plain, slow implementation of the Sogutar decoder, one function per mechanism, in float64 (or any torch dtype) on
the CPU. It shares no code with the package: it takes config.json as a dict and the tensors by name and loops over
tokens, heads and experts. The engine's tests compare against it.

Notation: T tokens, D width, H heads, G key/value heads, dk query/key size of a head, dv value size of a head, E experts.
The stream starts as LN(embed[token]); a layer is  x += mixer(LN(x)) + ff(LN(x))  with ONE layer norm (weight, no bias)
that both sub-layers read; the mixer is windowed softmax attention (its keys and values possibly borrowed from an
earlier layer) or retention (a matrix of state a head with a fixed decay); the feed-forward is dense (silu) or a
mixture of clamped experts with identity experts and a gated shared expert; logits = cap * tanh(embed LN(x) / cap).
Every function that keeps something between calls takes a dict `st` and leaves what the next call needs there, so whole
prompts, portions and single tokens all go through the same code.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch


# ---------------------------------------------------------------------------- files
def read_safetensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in head.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw, kind = data[lo:hi], info["dtype"]
        if kind == "BF16":
            t = torch.from_numpy((np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).copy())
        elif kind == "F32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy())
        elif kind == "I32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<i4").copy())
        else:
            raise ValueError(f"{name}: dtype {kind}")
        out[name] = t.reshape(info["shape"])
    return out


def read_model(model_dir, dtype=torch.float64):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    return cfg, {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}


# ---------------------------------------------------------------------------- small pieces
ROUNDING = None  # a function or None: with it, the operands of matrix products are rounded as a 16-bit engine rounds them


def _r(x):
    return x if ROUNDING is None else ROUNDING(x)


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last dimension, var the mean of the squared deviations; no bias."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def frequencies(rot):
    """The dims/2 turning rates of a rotation {dims, base, optional scaling {factor, low, high, original}}."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = sc["factor"], sc["low"], sc["high"], sc["original"]
        out = []
        for fi in f:
            wavelength = 2.0 * math.pi / fi
            if wavelength < orig / high:
                out.append(fi)
            elif wavelength > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wavelength - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=torch.float64)


def rotate(x, pos, rot):
    """x [heads, dk] at position pos: the pair (i, i + dims/2) of the first `dims` numbers of every head turns by pos * f_i."""
    if not rot or not rot.get("dims"):
        return x
    half = rot["dims"] // 2
    a = pos * frequencies(rot)
    c, s = torch.cos(a).to(x.dtype), torch.sin(a).to(x.dtype)
    out = x.clone()
    u, v = x[:, :half], x[:, half:2 * half]
    out[:, :half] = u * c - v * s
    out[:, half:2 * half] = v * c + u * s
    return out


# ---------------------------------------------------------------------------- windowed softmax attention
def attention(h, w, p, m, eps, st, kv_st=None):
    """h [T, D] -> [T, D]. m: heads, kv_heads, dim, vdim, scale, rot, optional mask {size}, optional kv_from.
    st keeps this layer's keys and values (after norm and rotation) of the whole sequence; a layer with kv_from reads
    kv_st, the dict of the layer it names, which has already taken this call's tokens in."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size = (m.get("mask") or {}).get("size", 0)
    own = kv_st is None
    T = h.shape[0]
    pos0 = st.get("n", 0)
    out = torch.zeros(T, H * dv, dtype=h.dtype)
    for t in range(T):
        pos = pos0 + t
        q = w[p + "q"] @ h[t]
        q = rotate((rms(q, eps) * w[p + "q.norm"]).view(H, dk), pos, m.get("rot"))
        q = _r(q)
        if own:
            k = w[p + "k"] @ h[t]
            k = rotate((rms(k, eps) * w[p + "k.norm"]).view(G, dk), pos, m.get("rot"))
            v = (w[p + "v"] @ h[t]).view(G, dv)
            st.setdefault("k", []).append(_r(k))
            st.setdefault("v", []).append(_r(v))
        src = st if own else kv_st
        lo = max(0, pos - size + 1) if size else 0
        K = torch.stack(src["k"][lo:pos + 1])  # [n, G, dk]
        V = torch.stack(src["v"][lo:pos + 1])
        for a in range(H):
            g = a // (H // G)
            s = (K[:, g] @ q[a]) * m["scale"]
            pr = torch.softmax(s, dim=0)
            out[t, a * dv:(a + 1) * dv] = _r(pr) @ V[:, g]
    st["n"] = pos0 + T
    return _r(out) @ w[p + "o"].T


# ---------------------------------------------------------------------------- retention
def retention(h, w, p, m, eps, st):
    """h [T, D] -> [T, D]. m: heads, dim, vdim, decay (a number a head), rot. Per head S <- decay S + k v^T with k rotated and
    times dk^(-1/2); o = S^T q with q rotated; o / rms(o) per head; times silu(W_g h); W_o."""
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos0 = st.get("n", 0)
    S = st.get("S")
    if S is None:
        S = torch.zeros(H, dk, dv, dtype=h.dtype)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    out = torch.zeros(T, H * dv, dtype=h.dtype)
    for t in range(T):
        pos = pos0 + t
        q = rotate((w[p + "q"] @ h[t]).view(H, dk), pos, m.get("rot"))
        k = rotate((w[p + "k"] @ h[t]).view(H, dk), pos, m.get("rot")) * dk ** -0.5
        v = (w[p + "v"] @ h[t]).view(H, dv)
        S = decay[:, None, None] * S + k[:, :, None] * v[:, None, :]
        o = torch.einsum("hkv,hk->hv", S, q)
        o = rms(o, eps).reshape(H * dv)
        out[t] = o * silu(w[p + "g"] @ h[t])
    st["S"], st["n"] = S, pos0 + T
    return _r(out) @ w[p + "o"].T


# ---------------------------------------------------------------------------- feed-forward
def dense_ff(h, w, p):
    return _r(silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def clamped_expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, -limit, limit)
    return _r(g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(h, w, p, r):
    """-> for every token the chosen router outputs (a list of `top` indices) and their weights."""
    z = h @ w[p + "router"].T  # [T, E + identity]
    s = torch.softmax(z, dim=-1)
    choice = s + w[p + "correction"]
    picks, weights = [], []
    for t in range(h.shape[0]):
        c = choice[t].clone()
        mine = []
        for _ in range(r["top"]):
            e = int(torch.argmax(c))
            mine.append(e)
            c[e] = -math.inf
        sc = s[t, mine]
        picks.append(mine)
        weights.append(sc / (sc.sum() + 1e-20) * r["scale"])
    return picks, weights


def moe_ff(h, w, p, f):
    r = f["router"]
    E = r["experts"]
    picks, weights = route(h, w, p, r)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, g in zip(picks[t], weights[t]):
            if e >= E:  # an identity expert: the input itself
                out[t] += g * h[t]
            else:
                out[t] += g * clamped_expert(h[t:t + 1], w, f"{p}e{e}.", f["expert"]["limit"])[0]
    sh = f.get("shared")
    if sh:
        gate = sigmoid(h @ w[p + "shared.sg"].T)  # [T, 1]
        out = out + gate * clamped_expert(h, w, p + "shared.", sh["limit"])
    return out


# ---------------------------------------------------------------------------- the model
class Plain:
    """The whole model with everything a sequence carries. run(tokens) takes the sequence's next tokens and returns their
    logits [T, vocab]; after it, `streams` holds the stream behind every layer for those tokens."""

    def __init__(self, cfg, w):
        self.cfg, self.w = cfg, w
        self.st = [dict() for _ in cfg["layers"]]
        self.streams = []

    def run(self, tokens):
        cfg, w = self.cfg, self.w
        eps = cfg["norm"]["eps"]
        x = layer_norm(w["embed"][torch.as_tensor(tokens, dtype=torch.long)], w["embed.norm"], eps)
        self.streams = []
        for i, l in enumerate(cfg["layers"]):
            p, m = f"l{i}.", l["mixer"]
            h = _r(layer_norm(x, w[p + "norm1"], eps))
            if l["type"] == "attention":
                j = m.get("kv_from")
                a = attention(h, w, p + "mix.", m, eps, self.st[i], None if j is None else self.st[j])
            elif l["type"] == "retention":
                a = retention(h, w, p + "mix.", m, eps, self.st[i])
            else:
                raise ValueError(l["type"])
            f = l.get("mlp")
            if f is None:
                b = 0.0
            elif f["kind"] == "dense":
                b = dense_ff(h, w, p + "mlp.")
            else:
                b = moe_ff(h, w, p + "mlp.", f)
            x = x + (a + b)
            self.streams.append(x.clone())
        y = _r(layer_norm(x, w["final.norm"], eps))
        logits = y @ w["embed"].T
        cap = cfg.get("logit_softcap")
        if cap:
            logits = cap * torch.tanh(logits / cap)
        return logits


def forward(cfg, w, ids, after_layers=None):
    """Logits [T, vocab] of a whole sequence; after_layers (a list) receives the stream behind every layer."""
    m = Plain(cfg, w)
    out = m.run(list(ids))
    if after_layers is not None:
        after_layers.extend(m.streams)
    return out


def greedy(cfg, w, prompt, n_new):
    """prompt + n_new tokens, each the first index of the largest logit; the sequence's keys and states are carried."""
    m = Plain(cfg, w)
    out = list(prompt)
    logits = m.run(out)
    for _ in range(n_new):
        out.append(int(torch.argmax(logits[-1])))
        logits = m.run(out[-1:])
    return out
