"""Tiny Selinex configurations and their weights for the tests. The configurations differ from one another in every size
and option, and no two sizes that could be mixed up are equal within one of them (query heads != key/value heads, key size !=
value size, rotated part != key size, window != page, taps != rank, groups kept != groups; one layer without a feed-forward,
one router without groups, one with a group an expert; loops over a part of the layers, over all of them, and none).

The weights are made here by rules of the test's own (not the package's random-weights mode), so that every tensor matters:
norm weights around zero, corrections large enough to change a choice and to make choice scores negative, feed-forward gates wide
enough to meet their limit, decays from fast to very slow (a state that is lost or reset shows hundreds of tokens later),
bonuses and blend weights away from 0 and 1. `sharp=True` scales the attention's query weights so that the softmax of most heads
rests on one or two keys, wherever they are: a key that is lost, shifted, read from a wrong page or let through a window's edge
moves the logits."""
from __future__ import annotations

import json
import math
import os

import torch


def _att(heads, kv_heads, dim, vdim, scale, window=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def _pair(left, heads, dim, vdim, tau, left_scale, right_scale):
    return {"left": left, "right": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "left_scale": left_scale, "right_scale": right_scale}


def _pair2(left, heads, dim):
    return {"left": left, "right": {"heads": heads, "dim": dim}}


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(ff, experts, top, groups=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


# ranks of the low-rank decay maps: no key of config.json; make_tensors draws the maps with these first dimensions
RANKS = {"sa": {1: 5, 2: 3}, "sb": {0: 16, 1: 8}, "sc": {0: 2, 2: 7}}

# A: nothing a multiple of 8; delta with shared query/key heads, a pair with a gate a head, a pair with a partly rotated head and no
#    feed-forward, a delta with a single tap and a router without groups; layers 1 and 2 run three times; pages of 4
SELINEX_A = {"architecture": "Selinex", "vocab": 301, "width": 72, "norm": {"eps": 1e-5}, "residual_mult": 0.6, "max_positions": 512,
             "loop": {"start": 1, "stop": 3, "times": 3},
             "layers": [{"type": "delta", "mixer": _delta(4, 2, 12, 10, 3), "mlp": _moe(20, 6, 2, (3, 2))},
                        {"type": "parallel", "mixer": _pair(_att(6, 2, 24, 10, 0.21, 13), 3, 20, 14, 7.0, 1.3, 0.7), "mlp": _dense(44, 0.8)},
                        {"type": "parallel_2", "mixer": _pair2(_att(4, 4, 12, 18, 0.3, 9, (8, 777.0)), 5, 14), "mlp": None},
                        {"type": "delta", "mixer": _delta(3, 3, 18, 6, 1), "mlp": _moe(12, 5, 1)}]}
# B: sizes the tensor-core products and attention take (multiples of 16, heads of 32 / 64 / 128); no loop, multiplier 1; pages of 16
SELINEX_B = {"architecture": "Selinex", "vocab": 512, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 1.0, "max_positions": 1024,
             "layers": [{"type": "parallel_2", "mixer": _pair2(_att(4, 2, 64, 64, 0.125, 48, (32, 250000.0)), 2, 64), "mlp": _dense(256, 2.0)},
                        {"type": "parallel", "mixer": _pair(_att(4, 4, 32, 128, 0.18, 40), 4, 32, 16, 4.0, 0.9, 1.1), "mlp": _moe(64, 8, 2, (4, 3))},
                        {"type": "delta", "mixer": _delta(4, 2, 32, 64, 4), "mlp": _moe(64, 16, 4, (4, 1))}]}
# C: one key/value head for five query heads, a window of one page, a window of a single key, one head of state, groups of one expert,
#    two taps, tau 1, attention without a window; the whole model runs twice; pages of 8
SELINEX_C = {"architecture": "Selinex", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 1.3, "max_positions": 400,
             "loop": {"start": 0, "stop": 3, "times": 2},
             "layers": [{"type": "parallel", "mixer": _pair(_att(5, 1, 16, 6, 0.4, 8), 1, 24, 10, 1.0, 1.0, 2.0), "mlp": _moe(16, 6, 2, (6, 2))},
                        {"type": "delta", "mixer": _delta(2, 1, 20, 12, 2), "mlp": _dense(40, 0.5)},
                        {"type": "parallel_2", "mixer": _pair2(_att(2, 2, 10, 14, 0.35, None, (10, 300.0)), 3, 6), "mlp": _moe(24, 3, 3)}]}
# D: a window of one key beside a long one
SELINEX_D = {"architecture": "Selinex", "vocab": 64, "width": 40, "norm": {"eps": 1e-6}, "residual_mult": 0.9, "max_positions": 300,
             "layers": [{"type": "parallel_2", "mixer": _pair2(_att(2, 1, 8, 12, 0.5, 1, (4, 50.0)), 2, 12), "mlp": _dense(24, 1.0)},
                        {"type": "parallel", "mixer": _pair(_att(3, 3, 12, 8, 0.3, 70), 2, 8, 20, 3.0, 0.5, 0.5), "mlp": None}]}
RANKS["sd"] = {0: 4, 1: 6}

SELINEX = {"sa": (SELINEX_A, 4), "sb": (SELINEX_B, 16), "sc": (SELINEX_C, 8), "sd": (SELINEX_D, 4)}  # name -> (config.json, page size)


def ranks_of(cfg):
    for name, (c, _) in SELINEX.items():
        if c is cfg:
            return RANKS[name]
    return {}


def make_tensors(cfg, seed, dtype, sharp=False, ranks=None):
    """name -> tensor, as a checkpoint stores them (matrices in `dtype`; the same for vectors: the reader widens)."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]
    ranks = ranks_of(cfg) if ranks is None else ranks
    t = {}

    def lin(name, out, inp, gain=1.0):
        t[name] = torch.randn(out, inp, generator=g) * (gain / math.sqrt(inp))

    def around_zero(name, n):
        t[name] = 0.2 * torch.randn(n, generator=g)

    def near_one(name, n):
        t[name] = 1.0 + 0.2 * torch.randn(n, generator=g)

    def slow_to_fast(n):
        """n decays between 0.5 and 0.999, the distances from 1 spread evenly on a logarithmic scale."""
        return 1.0 - torch.exp(torch.rand(n, generator=g) * math.log(500.0) + math.log(1e-3))

    def attention(p, m, gated):
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        lin(p + "q", H * dk, D); lin(p + "k", G * dk, D); lin(p + "v", G * dv, D); lin(p + "o", D, H * dv)
        if sharp:
            t[p + "q"] *= 6.0 / (m["scale"] * math.sqrt(dk))  # scores with a spread of about 6
        if gated:
            lin(p + "g", H, D, gain=2.0)

    t["embed"] = torch.randn(V, D, generator=g) * 0.5
    around_zero("final.norm", D)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        q = p + "mix."
        around_zero(p + "norm1", D)
        around_zero(p + "norm1b", D)
        if l["type"] == "delta":
            H, G, dk, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            lin(q + "q", G * dk, D); lin(q + "k", G * dk, D); lin(q + "v", H * dv, D); lin(q + "g", H * dv, D); lin(q + "o", D, H * dv)
            for s, c in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                t[q + s + ".conv"] = torch.randn(c, K, generator=g) * (0.8 / math.sqrt(K))
            lin(q + "b", H, D, gain=1.5); lin(q + "a", H, D, gain=0.5)
            rate = torch.exp(torch.rand(H, generator=g) * math.log(200.0) + math.log(0.01))  # exp(A_log): 0.01 .. 2
            t[q + "A_log"] = torch.log(rate)
            step = torch.exp(torch.rand(H, generator=g) * math.log(50.0) + math.log(0.02))   # softplus(dt_bias): 0.02 .. 1
            t[q + "dt_bias"] = torch.log(torch.expm1(step))
            near_one(q + "norm", dv)
        else:
            gated = l["type"] == "parallel"
            attention(q + "left.", m["left"], gated)
            r, rp, R = m["right"], q + "right.", ranks.get(i, 16)
            H, dk = r["heads"], r["dim"]
            if gated:
                dv = r["vdim"]
                lin(rp + "q", H * dk, D); lin(rp + "k", H * dk, D); lin(rp + "v", H * dv, D); lin(rp + "g", H * dv, D); lin(rp + "o", D, H * dv)
                near_one(rp + "norm", dv)
                lin(rp + "a1", R, D); lin(rp + "a2", H * dk, R, gain=0.5)
                a = slow_to_fast(H * dk) ** r["tau"]           # sigmoid(bias) = decay^tau
                t[rp + "a2.b"] = torch.log(a) - torch.log1p(-a)
            else:
                for s in "rkvgw":
                    t[rp + "mu." + s] = 0.1 + 0.8 * torch.rand(D, generator=g)
                for s in "rkvg":
                    lin(rp + s, H * dk, D)
                lin(rp + "o", D, H * dk)
                lin(rp + "w1", R, D); lin(rp + "w2", H * dk, R, gain=0.5)
                t[rp + "w0"] = torch.log(-torch.log(slow_to_fast(H * dk)))
                t[rp + "u"] = 0.5 * torch.randn(H, dk, generator=g) + 0.3
                near_one(rp + "norm", H * dk)
                near_one(q + "left.out", D); near_one(q + "right.out", D)
        f = l.get("mlp")
        if f:
            around_zero(p + "norm2", D)
            around_zero(p + "norm2b", D)
            if f["kind"] == "dense":
                lin(p + "mlp.gate", f["ff"], D, gain=1.5); lin(p + "mlp.up", f["ff"], D, gain=1.5); lin(p + "mlp.down", D, f["ff"])
            else:
                E = f["router"]["experts"]
                lin(p + "mlp.router", E, D, gain=2.0)
                t[p + "mlp.correction"] = torch.randn(E, generator=g) * 0.4 - 0.3
                for k in range(E):
                    lin(f"{p}mlp.e{k}.gate", f["expert"]["ff"], D); lin(f"{p}mlp.e{k}.up", f["expert"]["ff"], D)
                    lin(f"{p}mlp.e{k}.down", D, f["expert"]["ff"])
    return {k: v.to(dtype).contiguous() for k, v in t.items()}


def write_model(path, cfg, dtype, seed=11, sharp=False, ranks=None):
    from llmengine.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), make_tensors(cfg, seed, dtype, sharp, ranks))
    return path
