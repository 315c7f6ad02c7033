"""Tiny Sogutar configurations and their weights for the tests. The configurations differ from one another in every size and
option, and no two sizes that could be mixed up are equal within one of them (query heads != key/value heads, key size != value
size, rotated part != key size, window != page; layers that begin with a retention layer or an attention layer; layers that read
another layer's keys and values through a window wider or narrower than the owner's; routers with and without identity experts and
shared experts; a layer without a feed-forward; logits with and without a cap).

The weights are made here by rules of the test's own (not the package's random-weights mode), so that every tensor matters: norm
weights spread around one, corrections large enough to change a choice, feed-forward gates wide enough to meet their limits on both
sides, router logits that let identity experts win for some tokens, decays from fast to very slow (a state that is lost or reset
shows hundreds of tokens later). `sharp=True` scales the queries' norm weights so that the softmax of most heads rests on one or
two keys, wherever they are: a key that is lost, shifted, read from a wrong page or let through a window's edge moves the logits."""
from __future__ import annotations

import json
import math
import os

import torch


def att(heads, kv_heads, dim, vdim, scale, window=None, rot=None, scaling=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def ret(heads, dim, vdim, decay, rot=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, limit, experts, identity, top, scale, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
    if shared:
        f["shared"] = {"ff": shared[0], "limit": shared[1]}
    return f


# A: nothing a multiple of 8. Begins with retention; attention with 6 heads on 2, a part of each head rotated with stretched
#    frequencies; a layer that borrows layer 1's keys through a WIDER window than layer 1's own; a layer without a feed-forward;
#    one identity expert; pages of 4
SOGUTAR_A = {"architecture": "Sogutar", "vocab": 301, "width": 72, "norm": {"eps": 1e-5}, "logit_softcap": 9.0, "max_positions": 600,
             "layers": [{"type": "retention", "mixer": ret(3, 20, 14, (0.9, 0.99, 0.999), (12, 5000.0)), "mlp": moe(20, 0.8, 5, 1, 2, 1.7, (28, 1.1))},
                        {"type": "attention", "mixer": att(6, 2, 24, 10, 0.21, 13, (8, 777.0), (3.0, 1.0, 3.0, 40)), "mlp": dense(44)},
                        {"type": "retention", "mixer": ret(2, 12, 18, (0.5, 0.9995), None), "mlp": None},
                        {"type": "attention", "mixer": att(6, 2, 24, 10, 0.3, 21, (8, 777.0), (3.0, 1.0, 3.0, 40), kv_from=1), "mlp": moe(12, 1.5, 3, 0, 1, 1.0)}]}
# B: sizes the tensor-core products and attention take (multiples of 16, heads of 32 / 64 / 128). Begins with attention; two
#    identity experts; no cap on the logits; a borrower with a NARROWER window; pages of 16
SOGUTAR_B = {"architecture": "Sogutar", "vocab": 512, "width": 128, "norm": {"eps": 1e-6}, "max_positions": 1024,
             "layers": [{"type": "attention", "mixer": att(4, 2, 64, 64, 0.125, 48, (32, 250000.0), (8.0, 1.0, 4.0, 64)), "mlp": dense(256)},
                        {"type": "retention", "mixer": ret(4, 32, 96, (0.96875, 0.99, 0.998, 0.9995), (32, 5e5)), "mlp": moe(48, 1.25, 6, 2, 3, 2.5, (128, 2.0))},
                        {"type": "attention", "mixer": att(4, 4, 32, 128, 0.18, 40, (16, 10000.0)), "mlp": moe(64, 2.0, 16, 0, 4, 1.0, (64, 1.0))},
                        {"type": "attention", "mixer": att(4, 2, 64, 64, 0.1, 17, (32, 250000.0), (8.0, 1.0, 4.0, 64), kv_from=0), "mlp": dense(128)},
                        {"type": "retention", "mixer": ret(2, 64, 128, (0.9, 0.9999), (16, 100.0)), "mlp": dense(384)}]}
# C: one key/value head for five query heads, a window of one page, a window of a single key, attention without a window and
#    without rotation, one head of state, every expert chosen, two layers that borrow the same layer's keys; pages of 8
SOGUTAR_C = {"architecture": "Sogutar", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "logit_softcap": 4.0, "max_positions": 400,
             "layers": [{"type": "attention", "mixer": att(5, 1, 16, 6, 0.4, 8, (16, 300.0)), "mlp": moe(16, 0.6, 2, 1, 3, 0.5)},
                        {"type": "retention", "mixer": ret(1, 20, 12, (0.97,), (20, 50.0)), "mlp": dense(40)},
                        {"type": "attention", "mixer": att(5, 1, 16, 6, 0.35, 1, (16, 300.0), kv_from=0), "mlp": dense(24)},
                        {"type": "attention", "mixer": att(2, 2, 10, 14, 0.3, None, None), "mlp": moe(24, 3.0, 4, 3, 2, 3.0, (16, 0.7))},
                        {"type": "attention", "mixer": att(5, 1, 16, 6, 0.5, None, (16, 300.0), kv_from=0), "mlp": None}]}

SOGUTAR = {"ga": (SOGUTAR_A, 4), "gb": (SOGUTAR_B, 16), "gc": (SOGUTAR_C, 8)}  # name -> (config.json, page size)


def make_tensors(cfg, seed, dtype, sharp=False):
    """name -> tensor, as a checkpoint stores them (everything in `dtype`: the reader widens what it wants wider)."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]
    t = {}

    def lin(name, out, inp, gain=1.0):
        t[name] = torch.randn(out, inp, generator=g) * (gain / math.sqrt(inp))

    def near_one(name, n, spread=0.2):
        t[name] = 1.0 + spread * torch.randn(n, generator=g)

    t["embed"] = torch.randn(V, D, generator=g) * 0.5 + 0.1  # rows with a mean: the embedding's norm has something to take off
    near_one("embed.norm", D)
    near_one("final.norm", D)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        q = p + "mix."
        near_one(p + "norm1", D)
        if l["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            lin(q + "q", H * dk, D); lin(q + "o", D, H * dv)
            near_one(q + "q.norm", H * dk, 0.3)
            if sharp:
                t[q + "q.norm"] *= 6.0 / (m["scale"] * math.sqrt(dk))  # scores with a spread of about 6
            if m.get("kv_from") is None:
                lin(q + "k", G * dk, D); lin(q + "v", G * dv, D)
                near_one(q + "k.norm", G * dk, 0.3)
        else:
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            lin(q + "q", H * dk, D); lin(q + "k", H * dk, D); lin(q + "v", H * dv, D); lin(q + "g", H * dv, D, gain=1.5); lin(q + "o", D, H * dv)
        f = l.get("mlp")
        if f and f["kind"] == "dense":
            lin(p + "mlp.gate", f["ff"], D, gain=1.5); lin(p + "mlp.up", f["ff"], D, gain=1.5); lin(p + "mlp.down", D, f["ff"])
        elif f:
            r = f["router"]
            E, n_out = r["experts"], r["experts"] + r["identity"]
            lin(p + "mlp.router", n_out, D, gain=2.0)
            t[p + "mlp.correction"] = torch.randn(n_out, generator=g) * 0.3
            for k in range(E):
                lin(f"{p}mlp.e{k}.gate", f["expert"]["ff"], D, gain=1.5); lin(f"{p}mlp.e{k}.up", f["expert"]["ff"], D, gain=1.5)
                lin(f"{p}mlp.e{k}.down", D, f["expert"]["ff"])
            if f.get("shared"):
                ff = f["shared"]["ff"]
                lin(p + "mlp.shared.gate", ff, D, gain=1.5); lin(p + "mlp.shared.up", ff, D, gain=1.5); lin(p + "mlp.shared.down", D, ff)
                lin(p + "mlp.shared.sg", 1, D, gain=2.0)
    return {k: v.to(dtype).contiguous() for k, v in t.items()}


def write_model(path, cfg, dtype, seed=11, sharp=False):
    from llmengine.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), make_tensors(cfg, seed, dtype, sharp))
    return path
