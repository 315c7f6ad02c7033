"""Selinex on the GPU against the plain implementation (tests/plain_selinex.py): each mechanism alone (windowed attention with
and without rotation and a gate a head, the three linear-state mixers, the pair and its two ways of becoming one, the clamped
feed-forward, the sigmoid router with groups, the block with norms on both sides of a sublayer), then whole models through the
engine's step function in true 32-bit and in bfloat16: whole prompts, prompts followed by token-by-token decoding, portions
down to two tokens, batches of unequal requests, pages and state slots that are given back and used again, attention made
sharp so that a key that is lost or let through a window's edge shows, decays so slow that a lost state shows hundreds of
tokens later, long decoding, greedy generation through the scheduler, and replay through bin/trace_run."""
import copy
import json
import math

import numpy as np
import pytest
import torch

import llmengine
import plain_selinex as P
from gpu_helpers import DEV, Harness
from llmengine.config.selinex import SelinexConfig
from llmengine.models.selinex import describe_selinex
from llmengine.ops import get_ops
from llmengine.parts import LayerCache, build_part
from llmengine.parts.registry import part_class
from tiny import MIXED_SIZES_LONG, Trace, random_ids, round64, run_trace, trace_mixed, trace_portions, trace_tail, trace_whole
from tiny_selinex import RANKS, SELINEX, SELINEX_A, SELINEX_B, SELINEX_C, SELINEX_D, _att, _delta, _dense, _moe, _pair, _pair2, \
    make_tensors, ranks_of, write_model

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
NAMES = {torch.float32: "fp32", torch.bfloat16: "bf16"}


def close(got, want, dt, what="", tol32=1e-4, tol16=4e-2):
    """float32: element by element; bfloat16: the root mean square of the difference against that of the values."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    if dt == torch.float32:
        err = np.abs(got - want).max() / max(1.0, np.abs(want).max())
        assert err < tol32, f"{what}: float32 differs by {err:.3e}"
    else:
        err = np.sqrt(((got - want) ** 2).mean()) / max(np.sqrt((want ** 2).mean()), 1e-6)
        assert err < tol16, f"{what}: bfloat16 differs by {err:.3e} of the values' size"


def rounded_forward(pc, pw, ids):
    """The plain implementation with the operands of its matrix products rounded to bfloat16, as a 16-bit engine rounds them:
    its distance from the plain logits is the error that rounding alone causes in this model, on these tokens."""
    P.ROUNDING = lambda x: x.to(torch.bfloat16).to(x.dtype)
    try:
        return P.forward(pc, pw, ids).numpy()
    finally:
        P.ROUNDING = None


def rows_close(got, want, dt, what="", rounded=None):
    """Logits of a request, a row a position. float32: as close(). bfloat16: a row's error is the root mean square of its
    difference against that of all values. How large rounding alone makes it depends on the model (every sublayer's result is
    normalised before it is added, so nothing that is added is small; a router's choice between two experts that nearly tie can
    flip, and a recurrent state then colours the rows after it), so the measure is the plain implementation with the same
    roundings (`rounded`): the median row and the worst row in ten stay within 3 times its."""
    if dt == torch.float32:
        return close(got, want, dt, what)
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    size = max(np.sqrt((want ** 2).mean()), 1e-6)
    e = np.sqrt(((got - want) ** 2).mean(1)) / size
    n = np.sqrt(((np.asarray(rounded, dtype=np.float64) - want) ** 2).mean(1)) / size
    for q in (50, 90):
        a, b = np.percentile(e, q), np.percentile(n, q)
        assert a < 3 * b + 5e-3, f"{what}: bfloat16 rows differ by {a:.3e} of the values' size (percentile {q}); rounding alone: {b:.3e}"


def whole(delta):
    return delta if delta.dim() == 2 else delta.sum(0)


def with_ranks(cfg):
    """The configuration with the ranks that a model folder's tensor shapes would add."""
    c = copy.deepcopy(cfg)
    for i, r in ranks_of(cfg).items():
        c["layers"][i]["mixer"]["right"]["rank"] = r
    return c


def one_layer(layer, width=80, eps=1e-5, mult=0.8):
    return {"architecture": "Selinex", "vocab": 64, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "max_positions": 2048,
            "layers": [layer]}


def layer_tensors(cfg, i, dt, sharp=False, seed=5):
    """The tensors of layer i as the file would hold them -> (float64 for the plain side, on the device as the loader hands them
    over: matrices in the engine's precision, everything else float32, the block's description)."""
    t = {k: v for k, v in make_tensors(cfg, seed, dt, sharp).items() if k.startswith(f"l{i}.")}
    spec = describe_selinex(SelinexConfig.from_dict(with_ranks(cfg))).layers[i]
    needs = {n.name: n for n in part_class("block", spec.kind).tensor_needs(spec)}
    dev = {k: v.to(DEV, dt if needs[k].precision == "compute" else torch.float32) for k, v in t.items() if k in needs}
    return {k: v.double() for k, v in t.items()}, dev, spec


def mixer_harness(dt, page, part, pages=160):
    h = Harness(dt, page=page, pages=pages)
    c = LayerCache(group=0)
    for need in part.cache_needs():
        if hasattr(need, "head_dim"):
            c.k = torch.zeros(pages + 1, need.num_kv_heads, page, need.head_dim, dtype=dt, device=DEV)
            c.v = torch.zeros(pages + 1, need.num_kv_heads, page, need.value_dim, dtype=dt, device=DEV)
            c.window = need.window
        else:
            c.states[need.name] = torch.zeros((5,) + tuple(need.shape), dtype=need.dtype, device=DEV)
    return h, c


def loaded_mixer(dt, spec, dev, page=4, pages=160):
    part = build_part("mixer", spec, Harness(dt).env)
    h, cache = mixer_harness(dt, page, part, pages)
    part = build_part("mixer", spec, h.env)
    part.load(dev)
    return part, h, cache


PORTIONS = ((0, 1), (1, 3), (3, 4), (4, 21), (21, 22), (22, 24), (24, 70), (70, 71), (71, 72), (72, 100))


def run_block(block, stream, ctx, cache):
    """The block on a float32 stream -> the stream behind it (what the block left pending added)."""
    from llmengine.parts.base import Residual
    res = block.forward(Residual(stream), ctx, cache)
    if res.pending is not None:
        get_ops().residual_add(res.h, res.pending)
    return res.h


def run_in_portions(part, h, cache, x, plain_step, dt, portions=PORTIONS, **tol):
    for lo, hi in portions:
        got = whole(part.forward(x[lo:hi].to(DEV), h.ctx([(1, hi - lo, [])]), cache)).cpu()
        close(got, plain_step(x[lo:hi].double()), dt, f"positions {lo}..{hi}", **tol)


# ---------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("E,top,groups,keep,n", [(6, 2, 3, 2, 40), (16, 4, 4, 3, 33), (4, 4, 2, 2, 5), (9, 3, 3, 1, 17), (5, 1, 1, 1, 9),
                                                 (64, 8, 8, 4, 12), (6, 2, 6, 2, 21), (12, 3, 1, 1, 8)])
def test_sigmoid_router_with_groups_alone(E, top, groups, keep, n):
    """Choice scores that the correction makes negative; a group counts by its two largest (its only one, when a group is one
    expert); groups that are dropped although they hold the largest score; weights are the scores without the correction, not
    divided by their sum."""
    g = torch.Generator().manual_seed(E * 7 + top)
    x, wr = torch.randn(n, 24, generator=g), torch.randn(E, 24, generator=g) * 0.6
    corr = torch.randn(E, generator=g) * 0.4 - 0.9
    idx = torch.empty(n, top, dtype=torch.int32, device=DEV)
    share = torch.empty(n, top, dtype=torch.float32, device=DEV)
    get_ops().route_grouped(x.to(DEV), wr.to(DEV), corr.to(DEV), top, groups, keep, 0.0, idx, share, score="sigmoid", group_top=2,
                            normalize=False)
    z = x.double() @ wr.double().T
    negative = 0
    for t in range(n):
        chosen, wts = P.choose_experts(z[t], corr.double(), top, groups, keep)
        assert idx[t].tolist() == chosen.tolist(), f"token {t}"
        np.testing.assert_allclose(share[t].cpu().numpy(), wts.numpy(), rtol=2e-5)
        negative += int(((P.sigmoid(z[t]) + corr.double())[chosen] < 0).any())
    assert negative > 0, "the case is meant to choose experts whose choice score is negative"


FF_CASES = [(SELINEX_A, 0, 19), (SELINEX_A, 1, 4), (SELINEX_A, 3, 70), (SELINEX_B, 0, 150), (SELINEX_B, 1, 9), (SELINEX_B, 2, 33),
            (SELINEX_C, 0, 1), (SELINEX_C, 1, 40), (SELINEX_C, 2, 7)]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cfg,i,n", FF_CASES, ids=["a0", "a1", "a3", "b0", "b1", "b2", "c0", "c1", "c2"])
def test_feed_forward_alone(dt, cfg, i, n):
    """Dense: gates and ups beyond the limit on both sides (the gate has no lower limit). Routed: every expert is chosen (c2)."""
    cpu, dev, spec = layer_tensors(cfg, i, dt)
    h = Harness(dt)
    part = build_part("feed_forward", spec.feed_forward, h.env)
    part.load(dev)
    x = (1.5 * torch.randn(n, cfg["width"], generator=torch.Generator().manual_seed(8))).to(dt)
    got = whole(part.forward(x.to(DEV), h.ctx([(1, n, [])]))).cpu()
    f = cfg["layers"][i]["mlp"]
    if f["kind"] == "dense":
        gate = x.double() @ cpu[f"l{i}.mlp.gate"].T
        if n > 8:
            assert (gate > f["limit"]).any() and (gate < -f["limit"]).any(), "the case is meant to meet the limit"
        close(got, P.dense_ff(x.double(), cpu, f"l{i}.mlp.", f), dt)
    else:
        close(got, P.routed_ff(x.double(), cpu, f"l{i}.mlp.", f), dt)


def _attention_layer(heads, kv_heads, dim, vdim, window, rot, gated):
    left = _att(heads, kv_heads, dim, vdim, dim ** -0.5, window, rot)
    if gated:
        return one_layer({"type": "parallel", "mixer": _pair(left, 2, 16, 16, 2.0, 1.0, 1.0), "mlp": None})
    return one_layer({"type": "parallel_2", "mixer": _pair2(left, 2, 16), "mlp": None})


ATTENTION_CASES = [(SELINEX_A, 1), (SELINEX_A, 2), (SELINEX_B, 0), (SELINEX_B, 1), (SELINEX_C, 0), (SELINEX_C, 2), (SELINEX_D, 0),
                   (_attention_layer(6, 2, 64, 32, 16, (24, 1000.0), False), 0), (_attention_layer(8, 1, 128, 128, None, None, True), 0),
                   (_attention_layer(2, 2, 32, 128, 7, (32, 5e5), False), 0), (_attention_layer(12, 3, 128, 64, 21, None, True), 0)]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cfg,i", ATTENTION_CASES, ids=["a1", "a2", "b0", "b1", "c0", "c2", "d0", "64x32", "128x128", "32x128", "128x64"])
@pytest.mark.parametrize("sharp", [False, True])
def test_window_attention_alone(dt, cfg, i, sharp):
    """The pair's left side by itself over a prompt portion, then over single tokens and further portions that read the first one's
    cache rows: windows shorter than a portion, of one page, of one key, and none; rotation of a part of a head, of all of it,
    and none; a gate a head or none."""
    cpu, dev, spec = layer_tensors(cfg, i, dt, sharp)
    part, h, cache = loaded_mixer(dt, spec.mixer.left, dev)
    l = cfg["layers"][i]
    x = (2 * torch.randn(100, cfg["width"], generator=torch.Generator().manual_seed(6))).to(dt)
    state = {}
    run_in_portions(part, h, cache, x, lambda xs: P.window_attention(xs, cpu, f"l{i}.mix.left.", l["mixer"]["left"], state,
                                                                      gated=l["type"] == "parallel"), dt)


def _probe_weights(cpu, dev, prefix, H, G, dk, dt, strength):
    """Every query head asks along the model's first direction and every key answers along the second, with nothing else in
    either: a token whose input has the first direction set looks for the tokens whose input has the second one set."""
    D = cpu[prefix + "q"].shape[1]
    q, k = torch.zeros(H * dk, D, dtype=torch.float64), torch.zeros(G * dk, D, dtype=torch.float64)
    q[::dk, 0], k[::dk, 1] = strength, 1.0
    for name, w in ((prefix + "q", q), (prefix + "k", k)):
        cpu[name], dev[name] = w.to(dt).double(), w.to(DEV, dt)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("window,page", [(13, 4), (16, 16), (40, 16), (1, 4), (300, 16)])
@pytest.mark.parametrize("decoded", [False, True])
def test_a_marked_key_just_inside_and_just_outside_the_window(dt, window, page, decoded):
    """Hundreds of tokens of which one is marked; later tokens ask for it with a score that stands far out. The one that is
    `window - 1` behind it sees it and returns its value, the next one does not; the same when the asking tokens are decoded
    one by one, and when the marked key lies on a page's last or first row."""
    cfg = _attention_layer(4, 2, 16, 24, window, None, False)
    cpu, dev, spec = layer_tensors(cfg, 0, dt)
    _probe_weights(cpu, dev, "l0.mix.left.", 4, 2, 16, dt, 60.0 / 0.25)
    T = 420
    part, h, cache = loaded_mixer(dt, spec.mixer.left, dev, page=page, pages=T // page + 4)
    for marked in (page * 5 - 1, page * 5, 77):
        g = torch.Generator().manual_seed(marked)
        x = torch.randn(T, cfg["width"], generator=g)
        x[:, :2] = 0
        x[marked, 1] = 1.0                      # the key that is looked for
        x[marked, 2:] *= 3.0                    # and what it carries
        asking = [marked + window - 1, marked + window, marked + 150]
        for a in asking:
            if a < T and a != marked:
                x[a, 0] = 1.0
        x = x.to(dt)
        state, m = {}, cfg["layers"][0]["mixer"]["left"]
        want = P.window_attention(x.double(), cpu, "l0.mix.left.", m, state, gated=False)
        cut = marked + 1 if decoded else T
        got = [whole(part.forward(x[:cut].to(DEV), h.ctx([(marked + 1, cut, [])]), cache)).cpu()]
        for t in range(cut, min(T, marked + window + 2)):
            got.append(whole(part.forward(x[t:t + 1].to(DEV), h.ctx([(marked + 1, 1, [])]), cache)).cpu())
        got = torch.cat(got)
        close(got, want[:got.shape[0]], dt, f"marked key at {marked}")
        h.cm.release(marked + 1)
        if window > 1:  # the test tells the two apart: the value of the marked key is there, and one token later it is not
            v = (cpu["l0.mix.left.v"] @ x[marked].double()).view(2, 24)
            inside = marked + window - 1
            alone = torch.cat([v[a // 2] for a in range(4)]) @ cpu["l0.mix.left.o"].T
            assert float((want[inside] - alone).norm()) < 0.05 * float(alone.norm())
            if inside + 1 < T:
                assert float((want[inside + 1] - alone).norm()) > 0.5 * float(alone.norm())


RECURRENT_CASES = [(SELINEX_A, 0), (SELINEX_A, 1), (SELINEX_A, 2), (SELINEX_A, 3), (SELINEX_B, 0), (SELINEX_B, 1), (SELINEX_B, 2),
                   (SELINEX_C, 0), (SELINEX_C, 1), (SELINEX_C, 2), (SELINEX_D, 0), (SELINEX_D, 1),
                   (one_layer({"type": "delta", "mixer": _delta(4, 1, 128, 128, 4), "mlp": None}, width=96), 0),
                   (one_layer({"type": "parallel", "mixer": _pair(_att(2, 1, 16, 16, 0.25, 5), 2, 100, 36, 16.0, 1.0, 1.0), "mlp": None}), 0),
                   (one_layer({"type": "parallel_2", "mixer": _pair2(_att(2, 1, 16, 16, 0.25, 5), 1, 72), "mlp": None}), 0)]
RECURRENT_IDS = ["a0", "a1", "a2", "a3", "b0", "b1", "b2", "c0", "c1", "c2", "d0", "d1", "delta128", "decay100", "shift72"]


def _recurrent_part(cfg, i):
    """(the description of layer i's recurrent mixer, its plain function, its tensor prefix)"""
    l = cfg["layers"][i]
    if l["type"] == "delta":
        return (lambda spec: spec.mixer), P.gated_delta, f"l{i}.mix.", l["mixer"]
    fn = P.decayed_linear_attention if l["type"] == "parallel" else P.token_shift_recurrence
    return (lambda spec: spec.mixer.right), fn, f"l{i}.mix.right.", l["mixer"]["right"]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cfg,i", RECURRENT_CASES, ids=RECURRENT_IDS)
def test_linear_state_mixers_alone(dt, cfg, i):
    """Portions of 1, 2 and many tokens that hand the state (and the convolution's inputs, or the previous token's input) on
    through the slot; key sizes that fill a part of a lane's numbers, several lanes, and value sizes beyond a block's columns."""
    pick, plain, prefix, m = _recurrent_part(cfg, i)
    cpu, dev, spec = layer_tensors(cfg, i, dt)
    part, h, cache = loaded_mixer(dt, pick(spec), dev)
    x = (2 * torch.randn(100, cfg["width"], generator=torch.Generator().manual_seed(16))).to(dt)
    state = {}
    run_in_portions(part, h, cache, x, lambda xs: plain(xs, cpu, prefix, m, state, cfg["norm"]["eps"]), dt)


@pytest.mark.parametrize("cfg,i", [(SELINEX_B, 2), (SELINEX_B, 1), (SELINEX_B, 0)], ids=["delta", "decay", "shift"])
def test_a_state_written_once_is_read_hundreds_of_tokens_later(cfg, i):
    """Decays of (nearly) one and queries that ask for one early token's key: what that token wrote is read 400 tokens later,
    after portions and single tokens; a state that is lost, reset or read from another slot on the way shows."""
    dt = torch.float32
    pick, plain, prefix, m = _recurrent_part(cfg, i)
    cpu, dev, spec = layer_tensors(cfg, i, dt)
    slow = {"a2.b": 40.0, "w0": -20.0, "A_log": -20.0}   # sigmoid(40)^(1/tau), exp(-exp(-20)), exp(-exp(-20) * softplus(.)): all 1 - tiny
    for name, value in slow.items():
        if prefix + name in cpu:
            cpu[prefix + name] = torch.full_like(cpu[prefix + name], value)
            dev[prefix + name] = torch.full_like(dev[prefix + name], value)
    part, h, cache = loaded_mixer(dt, pick(spec), dev)
    T = 430
    x = 0.05 * torch.randn(T, cfg["width"], generator=torch.Generator().manual_seed(3))
    x[3] *= 60.0
    x[T - 2] = x[3]                                      # asks along the same directions as token 3 wrote
    state, eps = {}, cfg["norm"]["eps"]
    want = plain(x.double(), cpu, prefix, m, state, eps)
    got, lo = [], 0
    for n in (2, 1, 1, 130, 1, 2, 200, 61, 1, 1, 30):
        got.append(whole(part.forward(x[lo:lo + n].to(DEV), h.ctx([(1, n, [])]), cache)).cpu())
        lo += n
    assert lo == T
    close(torch.cat(got), want, dt, "portions", tol32=2e-4)
    state2 = {}
    fresh = plain(x[10:].double(), cpu, prefix, m, state2, eps)  # the same tokens without what token 3 wrote
    assert float((fresh[T - 12] - want[T - 2]).norm()) > 0.05 * float(want[T - 2].norm()), "the case is meant to depend on token 3"


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cfg,i", [(SELINEX_A, 1), (SELINEX_A, 2), (SELINEX_B, 0), (SELINEX_B, 1), (SELINEX_C, 0), (SELINEX_C, 2),
                                   (SELINEX_D, 0), (SELINEX_D, 1)], ids=["a1", "a2", "b0", "b1", "c0", "c2", "d0", "d1"])
def test_mixer_pair_alone(dt, cfg, i):
    """Both sides on the same input and their two ways of becoming one: weighted by unequal constants, and the mean of the two
    after each was divided by its root mean square and multiplied by a weight of its own."""
    cpu, dev, spec = layer_tensors(cfg, i, dt)
    part, h, cache = loaded_mixer(dt, spec.mixer, dev)
    l = cfg["layers"][i]
    x = (2 * torch.randn(100, cfg["width"], generator=torch.Generator().manual_seed(36))).to(dt)
    state = {}
    run_in_portions(part, h, cache, x, lambda xs: P.mixer(l["type"], xs, cpu, f"l{i}.mix.", l["mixer"], state, cfg["norm"]["eps"]), dt)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cfg,i", [(SELINEX_A, 0), (SELINEX_A, 2), (SELINEX_B, 1), (SELINEX_C, 1)], ids=["a0", "a2", "b1", "c1"])
def test_sandwich_block_alone(dt, cfg, i):
    """A whole layer on a float32 stream: norms with the weight 1 + w before and after each sublayer, the multiplier on what is
    added, and a layer that has no feed-forward."""
    cpu, dev, spec = layer_tensors(cfg, i, dt)
    env = Harness(dt).env
    block = build_part("block", spec, env)
    h, cache = mixer_harness(dt, 4, block.mixer)
    block = build_part("block", spec, h.env)
    block.load(dev)
    eps, mult, l = cfg["norm"]["eps"], cfg["residual_mult"], cfg["layers"][i]
    x = torch.randn(60, cfg["width"], generator=torch.Generator().manual_seed(46))
    state, lo = {}, 0
    for n in (17, 1, 2, 40):
        xs = x[lo:lo + n].double()
        y = P.mixer(l["type"], P.norm_one_plus(xs, cpu[f"l{i}.norm1"], eps), cpu, f"l{i}.mix.", l["mixer"], state, eps)
        want = xs + mult * P.norm_one_plus(y, cpu[f"l{i}.norm1b"], eps)
        if l.get("mlp"):
            hh = P.norm_one_plus(want, cpu[f"l{i}.norm2"], eps)
            f = l["mlp"]
            y = P.dense_ff(hh, cpu, f"l{i}.mlp.", f) if f["kind"] == "dense" else P.routed_ff(hh, cpu, f"l{i}.mlp.", f)
            want = want + mult * P.norm_one_plus(y, cpu[f"l{i}.norm2b"], eps)
        ctx = h.ctx([(1, n, [])])
        stream = x[lo:lo + n].to(DEV).contiguous()
        got = run_block(block, stream, ctx, cache)
        close(got.float().cpu(), want, dt, f"tokens {lo}..{lo + n}", tol16=6e-2)
        lo += n


# ---------------------------------------------------------------------------------------------- whole models
def replay(eng, trace):
    """The trace's steps through Engine.run_step, in this process -> {(request, position): logits row}."""
    ids, nxt, out = {}, 1, {}
    for k, s in enumerate(trace.steps):
        batch = []
        for e in s["entries"]:
            if e["id"] not in ids:
                ids[e["id"]], nxt = nxt, nxt + 1
            batch.append((ids[e["id"]], e["tokens"], e["want"]))
        lg = eng.run_step(batch, end=[ids[n] for n in s["end"]]).float().cpu().numpy()
        for n in s["end"]:
            ids.pop(n)
        for i, key in enumerate(trace.rows.get(k, [])):
            out[key] = lg[i].copy()
    return out


@pytest.fixture(scope="module", params=[(n, dt, sharp) for n in ("sa", "sb", "sc", "sd") for dt in DTYPES for sharp in (False, True)
                                        if not (sharp and n in ("sc", "sd"))],
                ids=lambda p: f"{p[0]}-{NAMES[p[1]]}{'-sharp' if p[2] else ''}")
def model(request, tmp_path_factory):
    name, dt, sharp = request.param
    cfg, page = SELINEX[name]
    d = write_model(str(tmp_path_factory.mktemp("selinex")), cfg, dt, sharp=sharp)
    pc, pw = P.read_model(d)
    lens = [5, 64, 33, 130, 97] if name != "sb" else [3, 47, 64, 200, 129]
    reqs = {f"r{i}": random_ids(n, cfg["vocab"], 50 + i) for i, n in enumerate(lens)}
    plain = {k: P.forward(pc, pw, v).numpy() for k, v in reqs.items()}
    if dt == torch.bfloat16:
        plain.update({k + ".rounded": rounded_forward(pc, pw, v) for k, v in reqs.items()})
    eng = llmengine.Engine(d, NAMES[dt], block_size=page)
    longest = max(round64(len(v)) for v in reqs.values())
    tokens = longest + 3 * 64  # room for the longest request and three short ones: pages are used again
    eng.configure_cache(num_blocks=tokens // page, block_size=page, num_slots=4)
    return dt, eng, reqs, plain, tokens, (pc, pw), cfg


@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_cuts_match_plain_and_one_another(model, cut):
    """whole: each prompt in one step; tail: its last 32 tokens one by one (prefill against decoding through the cache and the
    state); portions: sizes 7, 2, 13, 2, 5, 3, ... ; mixed: up to four live requests, portions beside single tokens, with so few
    pages and slots that both are used again."""
    dt, eng, reqs, plain, tokens, _, _ = model
    named = {f"{cut}.{k}": v for k, v in reqs.items()}
    trace = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}[cut](named) if cut != "mixed" else \
        trace_mixed(named, tokens, seed=5, sizes=MIXED_SIZES_LONG)
    rows = replay(eng, trace)
    assert eng.cm.num_requests == 0
    for k, ids in reqs.items():
        got = np.stack([rows[(f"{cut}.{k}", p)] for p in range(len(ids))])
        rows_close(got, plain[k], dt, f"{cut}, request {k}", plain.get(k + ".rounded"))
        if dt == torch.float32:  # where the first wrong position is, if any
            bad = np.nonzero(np.abs(got - plain[k]).max(1) > 1e-3 * max(1.0, np.abs(plain[k]).max()))[0]
            assert bad.size == 0, f"{cut}, request {k}: first wrong position {bad[0]} of {len(ids)}"


def test_the_stream_after_every_layer_run(model):
    """In float32 the residual stream behind every run of a layer (a looped layer counts each time) against the plain one."""
    dt, eng, reqs, _, _, (pc, pw), cfg = model
    if dt != torch.float32:
        pytest.skip("compared in float32")
    ids = reqs["r2"]
    after = []
    P.forward(pc, pw, ids, after_layers=after)
    got = []
    m = eng._ensure_model() if hasattr(eng, "_ensure_model") else eng.model
    m.after_run = lambda r, h: got.append(h[:len(ids)].float().cpu().clone())
    try:
        eng.run_step([(9, ids, [len(ids) - 1])], end=[9])
    finally:
        m.after_run = None
    assert len(got) == len(after) == len(P.layer_order(cfg))
    for r, (a, b) in enumerate(zip(got, after)):
        close(a, b, dt, f"run {r} (layer {P.layer_order(cfg)[r]})")


def test_keys_at_page_borders_window_edges_and_first_tokens(model):
    """A request that grows one token a step from its first token across page borders and past every window's length, beside a
    second one that starts later (so that its pages lie between the first one's, and its state in another slot)."""
    dt, eng, reqs, plain, _, _, _ = model
    a, b = reqs["r2"], reqs["r1"][:20]
    t = Trace()
    for p in range(len(a)):
        entries = [("a", a[p:p + 1], [0], p)]
        if 5 <= p < 5 + len(b):
            entries.append(("b", b[p - 5:p - 4], [0], p - 5))
        t.add(entries, end=[n for n, cond in (("a", p == len(a) - 1), ("b", p == 4 + len(b))) if cond])
    rows = replay(eng, t)
    rows_close(np.stack([rows[("a", p)] for p in range(len(a))]), plain["r2"], dt, "token by token", plain.get("r2.rounded"))
    rows_close(np.stack([rows[("b", p)] for p in range(len(b))]), plain["r1"][:20], dt, "the request beside it",
               plain["r1.rounded"][:20] if dt == torch.bfloat16 else None)


def test_a_slot_that_is_used_again_starts_at_zero(model):
    """Requests one after the other in an engine with a single live request at a time: each gets the one before's slot and
    pages, and must not see its state, its previous token or its convolution's inputs."""
    dt, eng, reqs, plain, _, _, _ = model
    for k in ("r3", "r1", "r3"):
        n = len(reqs[k])
        got = eng.run_step([(77, reqs[k], list(range(n)))], end=[77]).float().cpu().numpy()
        rows_close(got, plain[k], dt, k, plain.get(k + ".rounded"))


def test_long_decoding_and_generation(model):
    """Greedy generation through the engine's entry point and scheduler (decode steps replay CUDA graphs in bfloat16); in
    float32 the tokens are the plain implementation's."""
    dt, eng, reqs, plain, _, (pc, pw), cfg = model
    prompt = reqs["r2"][:11]
    out, reason = eng.generate(prompt, 90)
    assert reason == "length" and len(out) == 101 and out[:11] == prompt
    logits = P.forward(pc, pw, out).numpy()
    if dt == torch.float32:
        for p in range(10, 100):  # the chosen token is the plain logits' best, or ties with it within rounding
            assert logits[p, out[p + 1]] >= logits[p].max() - 1e-4 * max(1.0, np.abs(logits[p]).max()), p
    else:  # bfloat16: close to the plain logits' best; a router's choice that rounding flips may move single positions further
        off = [p for p in range(10, 100) if logits[p, out[p + 1]] < logits[p].max() - 0.1 * max(1.0, np.abs(logits[p]).max())]
        assert len(off) <= 9, f"{len(off)} of 90 generated tokens are far from the plain logits' best, first at {off[0]}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["sa", "sb"])
def test_replay_through_the_command(dtype, name, tmp_path):
    """bin/trace_run as a user runs it."""
    cfg, page = SELINEX[name]
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    d = write_model(str(tmp_path / "m"), cfg, dt)
    pc, pw = P.read_model(d)
    reqs = {f"q{i}": random_ids(n, cfg["vocab"], 80 + i) for i, n in enumerate([2, 70, 35, 150])}
    t = trace_mixed(reqs, 256 + 64, seed=3, sizes=MIXED_SIZES_LONG)
    rows = run_trace(d, dtype, t, str(tmp_path / "out"), 256 + 64, page, cfg["vocab"])
    for k, ids in reqs.items():
        rows_close(np.stack([rows[(k, p)] for p in range(len(ids))]), P.forward(pc, pw, ids).numpy(), dt, k,
                   rounded_forward(pc, pw, ids) if dtype == "bfloat16" else None)


def test_generation_from_the_command_line(tmp_path):
    from test_cli import run_cli
    d = write_model(str(tmp_path / "model"), SELINEX_C, torch.float32)
    r = run_cli("--model", d, "--prompt-ids", "5,17,3,90", "--max-new", "6", "--block-size", "8", "--num-blocks", "32")
    assert r.returncode == 0, r.stderr
    line = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")][0]
    pc, pw = P.read_model(d)
    assert line["token_ids"] == P.greedy(pc, pw, [5, 17, 3, 90], 6) and line["finish_reason"] == "length"
