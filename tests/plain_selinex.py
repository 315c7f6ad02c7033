"""A plain, slow implementation of the Selinex decoder, one function per mechanism, in float64 (or any torch
dtype) on the CPU. It shares no code with the package: it takes config.json as a dict and the tensors by name
and loops over tokens, heads and experts. The engine's tests compare against it.

Notation: T tokens, D width, H heads, G key/value heads, dk query/key size of a head, dv value size of a head,
E experts. A layer:  x += m * norm_b(sublayer(norm_a(x)))  for the mixer and then for the feed-forward, every norm
with the weight 1 + w. Mixers: two side by side (windowed softmax attention beside a linear recurrence with a decay per key
channel, or rotated windowed attention beside a token-shift recurrence with a bonus for the current token) or a gated
delta rule behind short convolutions. Every function that keeps something between calls takes a dict `st` and leaves
what the next call needs there, so whole prompts, portions and single tokens all go through the same code.
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
        base = 8 + n
        out = {}
        for name, info in head.items():
            if name == "__metadata__":
                continue
            lo, hi = info["data_offsets"]
            f.seek(base + lo)
            raw = f.read(hi - lo)
            dt = info["dtype"]
            if dt == "BF16":
                a = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
                t = torch.from_numpy(a.view(np.float32).copy())
            elif dt == "F32":
                t = torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy())
            elif dt == "I32":
                t = torch.from_numpy(np.frombuffer(raw, dtype="<i4").copy())
            else:
                raise ValueError(f"{name}: dtype {dt}")
            out[name] = t.reshape(info["shape"])
    return out


def read_model(model_dir, dtype=torch.float64):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    return cfg, {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}


# ---------------------------------------------------------------------------- small pieces
ROUNDING = None  # a function, or None. A 16-bit engine rounds the operands of its matrix products (a sublayer's input, queries, keys and
# values, what enters an output projection or an expert's last matrix); with ROUNDING set, the same happens here, everything else
# staying in the precision of the weights: the difference to a run without it is the error that rounding alone causes.


def _r(x):
    return x if ROUNDING is None else ROUNDING(x)


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


# ---------------------------------------------------------------------------- windowed softmax attention
def rotate(x, pos, dims, base):
    """x [heads, dk] at position pos: pairs (i, i + dims/2) of the first `dims` numbers of every head turn by pos * base^(-2i/dims)."""
    if not dims:
        return x
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    a = (pos * f)
    c, s = torch.cos(a).to(x.dtype), torch.sin(a).to(x.dtype)
    out = x.clone()
    u, v = x[:, :half], x[:, half:dims]
    out[:, :half] = u * c - v * s
    out[:, half:dims] = v * c + u * s
    return out


def window_attention(h, w, p, m, st, gated):
    """h [T, D] -> [T, D]. m: heads, kv_heads, dim, vdim, scale, optional rot {dims, base}, optional mask {size}.
    st keeps every key and value of the sequence; the window is applied when they are read."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot, size = m.get("rot"), (m.get("mask") or {}).get("size", 0)
    T = h.shape[0]
    pos0 = st.get("n", 0)
    out = torch.zeros(T, H * dv, dtype=h.dtype)
    for t in range(T):
        pos = pos0 + t
        q = (w[p + "q"] @ h[t]).view(H, dk)
        k = (w[p + "k"] @ h[t]).view(G, dk)
        v = (w[p + "v"] @ h[t]).view(G, dv)
        if rot:
            q, k = rotate(q, pos, rot["dims"], rot["base"]), rotate(k, pos, rot["dims"], rot["base"])
        q, k, v = _r(q), _r(k), _r(v)
        st.setdefault("k", []).append(k)
        st.setdefault("v", []).append(v)
        lo = max(0, pos - size + 1) if size else 0
        K, V = torch.stack(st["k"][lo:pos + 1]), torch.stack(st["v"][lo:pos + 1])  # [S, G, *]
        gate = sigmoid(w[p + "g"] @ h[t]) if gated else None                       # one number a head
        for a in range(H):
            b = a // (H // G)
            pr = torch.softmax((K[:, b] @ q[a]) * m["scale"], dim=0)
            o = pr @ V[:, b]
            if gated:
                o = o * gate[a]
            out[t, a * dv:(a + 1) * dv] = o
    st["n"] = pos0 + T
    return _r(out) @ w[p + "o"].t()


# ---------------------------------------------------------------------------- recurrence with a decay per key channel
def decayed_linear_attention(h, w, p, m, st, eps):
    """S <- diag(alpha) S + k v^T; o = S^T q, alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau) per head and key channel."""
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    T = h.shape[0]
    S = st.get("S")
    if S is None:
        S = torch.zeros(H, dk, dv, dtype=h.dtype)
    out = torch.zeros(T, H * dv, dtype=h.dtype)
    for t in range(T):
        q = (w[p + "q"] @ h[t]).view(H, dk) * dk ** -0.5
        k = (w[p + "k"] @ h[t]).view(H, dk)
        v = (w[p + "v"] @ h[t]).view(H, dv)
        z = w[p + "a2"] @ (w[p + "a1"] @ h[t]) + w[p + "a2.b"]
        alpha = (sigmoid(z) ** (1.0 / tau)).view(H, dk)
        S = alpha[:, :, None] * S + k[:, :, None] * v[:, None, :]
        o = torch.einsum("hkv,hk->hv", S, q)
        o = rms(o, eps) * w[p + "norm"]
        out[t] = o.reshape(-1) * silu(w[p + "g"] @ h[t])
    st["S"] = S
    return _r(out) @ w[p + "o"].t()


# ---------------------------------------------------------------------------- token-shift recurrence with a bonus
def token_shift_recurrence(h, w, p, m, st, eps):
    """Every projection reads h + (h_prev - h) * mu of its own; o = (S + diag(u) k v^T)^T r, then S <- diag(decay) S + k v^T."""
    H, dk = m["heads"], m["dim"]
    T, D = h.shape
    S = st.get("S")
    if S is None:
        S = torch.zeros(H, dk, dk, dtype=h.dtype)
    prev = st.get("prev")
    if prev is None:
        prev = torch.zeros(D, dtype=h.dtype)
    out = torch.zeros(T, H * dk, dtype=h.dtype)
    u = w[p + "u"].view(H, dk)
    for t in range(T):
        mix = {s: _r(h[t] + (prev - h[t]) * w[p + "mu." + s]) for s in "rkvgw"}
        r = (w[p + "r"] @ mix["r"]).view(H, dk)
        k = (w[p + "k"] @ mix["k"]).view(H, dk)
        v = (w[p + "v"] @ mix["v"]).view(H, dk)
        gate = silu(w[p + "g"] @ mix["g"])
        decay = torch.exp(-torch.exp(w[p + "w2"] @ torch.tanh(w[p + "w1"] @ mix["w"]) + w[p + "w0"])).view(H, dk)
        kv = k[:, :, None] * v[:, None, :]
        o = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r)
        S = decay[:, :, None] * S + kv
        o = rms(o, eps).reshape(-1) * w[p + "norm"]
        out[t] = o * gate
        prev = h[t]
    st["S"], st["prev"] = S, prev
    return _r(out) @ w[p + "o"].t()


# ---------------------------------------------------------------------------- gated delta rule
def short_conv_silu(x, weight, st, key):
    """x [T, C], weight [C, taps]: out[t, c] = silu(sum_j weight[c, j] * x[t - (taps - 1) + j, c]), so tap taps - 1 meets the token itself;
    inputs before the sequence's first token are zero; st keeps the last taps - 1 inputs for the next call."""
    taps = weight.shape[1]
    tail = st.get(key)
    if tail is None:
        tail = torch.zeros(taps - 1, x.shape[1], dtype=x.dtype)
    padded = torch.cat([tail, x], dim=0)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        out[t] = (padded[t:t + taps] * weight.t()).sum(0)
    st[key] = padded[padded.shape[0] - (taps - 1):] if taps > 1 else tail
    return silu(out)


def gated_delta(h, w, p, m, st, eps):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = short_conv_silu(h @ w[p + "q"].t(), w[p + "q.conv"], st, "cq").view(T, G, dk)
    k = short_conv_silu(h @ w[p + "k"].t(), w[p + "k.conv"], st, "ck").view(T, G, dk)
    v = short_conv_silu(h @ w[p + "v"].t(), w[p + "v.conv"], st, "cv").view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = st.get("S")
    if S is None:
        S = torch.zeros(H, dk, dv, dtype=h.dtype)
    out = torch.zeros(T, H * dv, dtype=h.dtype)
    for t in range(T):
        beta = sigmoid(w[p + "b"] @ h[t])
        g = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(w[p + "a"] @ h[t] + w[p + "dt_bias"]))
        o = torch.zeros(H, dv, dtype=h.dtype)
        for a in range(H):
            b = a // (H // G)
            Sa = g[a] * S[a]
            u = beta[a] * (v[t, a] - Sa.t() @ k[t, b])
            Sa = Sa + k[t, b][:, None] * u[None, :]
            o[a] = Sa.t() @ q[t, b]
            S[a] = Sa
        o = rms(o, eps) * w[p + "norm"]
        out[t] = o.reshape(-1) * silu(w[p + "g"] @ h[t])
    st["S"] = S
    return _r(out) @ w[p + "o"].t()


# ---------------------------------------------------------------------------- mixers of a layer
def mixer(kind, h, w, p, m, st, eps):
    if kind == "delta":
        return gated_delta(h, w, p, m, st, eps)
    left, right = st.setdefault("left", {}), st.setdefault("right", {})
    if kind == "parallel":
        a = window_attention(h, w, p + "left.", m["left"], left, gated=True)
        b = decayed_linear_attention(h, w, p + "right.", m["right"], right, eps)
        return m["left_scale"] * a + m["right_scale"] * b
    if kind == "parallel_2":
        a = window_attention(h, w, p + "left.", m["left"], left, gated=False)
        b = token_shift_recurrence(h, w, p + "right.", m["right"], right, eps)
        return 0.5 * (rms(a, eps) * w[p + "left.out"] + rms(b, eps) * w[p + "right.out"])
    raise ValueError(kind)


# ---------------------------------------------------------------------------- feed-forwards
def dense_ff(h, w, p, f):
    lim = f["limit"]
    g = torch.clamp(h @ w[p + "gate"].t(), max=lim)
    u = torch.clamp(h @ w[p + "up"].t(), -lim, lim)
    return _r(g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].t()


def choose_experts(z, correction, top, groups, keep):
    """z [E] router logits -> (chosen expert indices, their weights)."""
    s = sigmoid(z)
    choice = s + correction
    E = z.shape[0]
    if groups and keep < groups:
        per = E // groups
        score = torch.stack([torch.sort(choice[i * per:(i + 1) * per], descending=True).values[:2].sum() for i in range(groups)])
        kept = torch.argsort(score, descending=True, stable=True)[:keep].tolist()
        masked = torch.full_like(choice, float("-inf"))
        for i in kept:
            masked[i * per:(i + 1) * per] = choice[i * per:(i + 1) * per]
        choice = masked
    chosen = torch.argsort(choice, descending=True, stable=True)[:top]
    return chosen, s[chosen]


def routed_ff(h, w, p, f):
    r = f["router"]
    gr = r.get("groups") or {}
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, share = choose_experts(w[p + "router"] @ h[t], w[p + "correction"], r["top"], gr.get("count", 0), gr.get("keep", 0))
        for e, g in zip(chosen.tolist(), share):
            q = f"{p}e{e}."
            out[t] += g * (w[q + "down"] @ _r(silu(w[q + "gate"] @ h[t]) * (w[q + "up"] @ h[t])))
    return out


# ---------------------------------------------------------------------------- the model
def layer_order(cfg):
    L = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(L))
    return list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], L))


class Sequence:
    """One sequence's state: what every run of a layer keeps."""

    def __init__(self, cfg):
        self.runs = [dict() for _ in layer_order(cfg)]


def forward(cfg, w, tokens, seq=None, after_layers=None):
    """Runs `tokens` (the next ones of `seq`, a fresh sequence if None) -> logits [T, vocab]. after_layers: a list that receives
    the stream after every run."""
    if seq is None:
        seq = Sequence(cfg)
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for r, i in enumerate(layer_order(cfg)):
        l, p = cfg["layers"][i], f"l{i}."
        y = mixer(l["type"], _r(norm_one_plus(x, w[p + "norm1"], eps)), w, p + "mix.", l["mixer"], seq.runs[r], eps)
        x = x + m * norm_one_plus(y, w[p + "norm1b"], eps)
        f = l.get("mlp")
        if f:
            hh = _r(norm_one_plus(x, w[p + "norm2"], eps))
            y = dense_ff(hh, w, p + "mlp.", f) if f["kind"] == "dense" else routed_ff(hh, w, p + "mlp.", f)
            x = x + m * norm_one_plus(y, w[p + "norm2b"], eps)
        if after_layers is not None:
            after_layers.append(x.clone())
    return _r(norm_one_plus(x, w["final.norm"], eps)) @ w["embed"].t()


def greedy(cfg, w, prompt, n_new):
    seq = Sequence(cfg)
    out = list(prompt)
    logits = forward(cfg, w, prompt, seq)
    for _ in range(n_new):
        out.append(int(torch.argmax(logits[-1])))
        logits = forward(cfg, w, out[-1:], seq)
    return out
