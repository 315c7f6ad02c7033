"""Sogutar on the GPU against the plain implementation (tests/plain_sogutar.py): each mechanism alone (the layer norm with the
residual sum folded in, capped logits, the router with identity experts, a correction, a scale and the shared expert's gate, the
clamped experts, windowed attention with a norm over the whole projection and stretched rotation frequencies, attention on
another layer's keys, retention, the one-norm parallel block), then whole models through the engine's step function in true
32-bit and in bfloat16: whole prompts, prompts followed by token-by-token decoding, portions down to two tokens, batches of
unequal requests, pages and state slots that are given back and used again, attention made sharp so that a key that is lost or
let through a window's edge shows, decays so slow that a lost state shows hundreds of tokens later, long decoding, greedy
generation through the scheduler, and replay through bin/trace_run."""
import json
import math

import numpy as np
import pytest
import torch

import llmengine
import plain_sogutar as P
from gpu_helpers import DEV, Harness
from llmengine.config.sogutar import SogutarConfig
from llmengine.models.sogutar import describe_sogutar
from llmengine.ops import get_ops
from llmengine.parts import LayerCache, build_part
from llmengine.parts.registry import part_class
from tiny import MIXED_SIZES_LONG, Trace, random_ids, round64, run_trace, trace_mixed, trace_portions, trace_tail, trace_whole
from tiny_sogutar import SOGUTAR, SOGUTAR_A, SOGUTAR_B, SOGUTAR_C, att, dense, make_tensors, moe, ret, write_model

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
    difference against that of all values; the measure is the plain implementation with the same roundings (`rounded`): the
    median row and the worst row in ten stay within 3 times its (a router's choice between two experts that nearly tie can flip
    with the rounding, and a state then carries the other choice on)."""
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


def one_layer(layer, width=80, eps=1e-5, before=()):
    return {"architecture": "Sogutar", "vocab": 64, "width": width, "norm": {"eps": eps}, "max_positions": 2048, "layers": list(before) + [layer]}


def layer_tensors(cfg, i, dt, sharp=False, seed=5):
    """The tensors of layer i as the file would hold them -> (float64 for the plain side, on the device as the loader hands them
    over: matrices in the engine's precision, everything else float32, the block's description)."""
    t = {k: v for k, v in make_tensors(cfg, seed, dt, sharp).items() if k.startswith(f"l{i}.")}
    spec = describe_sogutar(SogutarConfig.from_dict(cfg)).layers[i]
    needs = {n.name: n for n in part_class("block", spec.kind).tensor_needs(spec)}
    assert set(needs) == set(t), "the test's tensors and the description's differ"
    dev = {k: v.to(DEV, dt if needs[k].precision == "compute" else torch.float32) for k, v in t.items()}
    return {k: v.double() for k, v in t.items()}, dev, spec


def cache_for(dt, page, part, pages=160):
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


def loaded(category, dt, spec, dev, page=4, pages=160):
    part = build_part(category, spec, Harness(dt).env)
    h, cache = cache_for(dt, page, part if category == "mixer" else part.mixer, pages)
    part = build_part(category, spec, h.env)
    part.load(dev)
    return part, h, cache


PORTIONS = ((0, 1), (1, 3), (3, 4), (4, 21), (21, 22), (22, 24), (24, 70), (70, 71), (71, 72), (72, 100))


def run_in_portions(part, h, cache, x, plain_step, dt, portions=PORTIONS, **tol):
    for lo, hi in portions:
        got = whole(part.forward(x[lo:hi].to(DEV), h.ctx([(1, hi - lo, [])]), cache)).cpu()
        close(got, plain_step(x[lo:hi].double()), dt, f"positions {lo}..{hi}", **tol)


# ---------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("n,dim,parts", [(5, 72, 0), (40, 128, 1), (3, 100, 3), (600, 1024, 1), (9, 4096, 2), (2, 37, 1), (7, 20000, 0)])
def test_layer_norm_alone(dt, n, dim, parts):
    """Rows with a mean far from zero (the variance must come from the deviations); the residual sum folded in, as one set of
    sums or several parts; rows picked by a list; widths that are no multiples of 4 and beyond a block's registers."""
    g = torch.Generator().manual_seed(n + dim)
    h = torch.randn(n, dim, generator=g) + 30.0
    w = 1.0 + 0.3 * torch.randn(dim, generator=g)
    delta = None if parts == 0 else torch.randn(parts, n, dim, generator=g) if parts > 1 else torch.randn(n, dim, generator=g)
    x = h.double() + (0 if delta is None else delta.double() if delta.dim() == 2 else delta.double().sum(0))
    want = P.layer_norm(x, w.double(), 1e-5)
    hd, out = h.to(DEV), torch.empty(n, dim, dtype=dt, device=DEV)
    get_ops().rmsnorm(hd, w.to(DEV), 1e-5, out, delta=None if delta is None else delta.to(DEV), center=True)
    close(out.float().cpu(), want, dt, "all rows", tol32=2e-5, tol16=1e-2)
    if delta is not None:
        np.testing.assert_allclose(hd.cpu().numpy(), x.float().numpy(), rtol=1e-6)  # the sum was written back
    rows = torch.tensor([n - 1, 0, n // 2], dtype=torch.int32)
    out2 = torch.empty(3, dim, dtype=dt, device=DEV)
    get_ops().rmsnorm(hd, w.to(DEV), 1e-5, out2, rows=rows.to(DEV), center=True)
    close(out2.float().cpu(), P.layer_norm(hd.cpu().double()[rows.long()], w.double(), 1e-5), dt, "picked rows", tol32=2e-5, tol16=1e-2)


def test_capped_logits_alone():
    x = torch.linspace(-90, 90, 1001).reshape(7, 143).contiguous()
    got = get_ops().softcap(x.to(DEV), 13.0).cpu()
    np.testing.assert_allclose(got.numpy(), (13.0 * torch.tanh(x.double() / 13.0)).numpy(), rtol=3e-6, atol=1e-6)


@pytest.mark.parametrize("E,identity,top,scale,n", [(5, 1, 2, 1.7, 40), (6, 2, 3, 2.5, 33), (2, 1, 3, 0.5, 9), (16, 0, 4, 1.0, 17), (4, 3, 2, 3.0, 64),
                                                    (1, 0, 1, 1.0, 5), (60, 4, 8, 1.0, 12)])
def test_router_alone(E, identity, top, scale, n):
    """Softmax over experts and identity experts together; a correction that changes choices but not weights; weights divided by
    their sum and multiplied by the scale; the shared expert's gate from one more row; identity experts that win."""
    g = torch.Generator().manual_seed(E * 7 + top)
    n_out = E + identity
    x, wr = torch.randn(n, 24, generator=g), torch.randn(n_out + 1, 24, generator=g) * 0.6
    corr = torch.randn(n_out, generator=g) * 0.3
    idx = torch.empty(n, top, dtype=torch.int32, device=DEV)
    share = torch.empty(n, top, dtype=torch.float32, device=DEV)
    gate = torch.empty(n, dtype=torch.float32, device=DEV)
    get_ops().route_grouped(x.to(DEV), wr.to(DEV), corr.to(DEV), top, 1, 1, 1e-20, idx, share, weight_scale=scale, gate_out=gate)
    w = {"router": wr[:n_out].double(), "correction": corr.double()}
    picks, weights = P.route(x.double(), w, "", {"top": top, "scale": scale})
    plain_choice_without = torch.topk(torch.softmax(x.double() @ wr[:n_out].double().T, -1), top).indices
    changed = won = 0
    for t in range(n):
        assert idx[t].tolist() == picks[t], f"token {t}"
        np.testing.assert_allclose(share[t].cpu().numpy(), weights[t].numpy(), rtol=2e-5)
        changed += int(sorted(picks[t]) != sorted(plain_choice_without[t].tolist()))
        won += int(any(e >= E for e in picks[t]))
    np.testing.assert_allclose(gate.cpu().numpy(), P.sigmoid(x.double() @ wr[n_out].double()).numpy(), rtol=2e-5)
    if n_out > top and n >= 30:
        assert changed > 0, "the case is meant to have choices that the correction changes"
    if identity and n >= 30:
        assert won > 0, "the case is meant to choose identity experts"


FF_CASES = [(SOGUTAR_A, 0, 19), (SOGUTAR_A, 1, 4), (SOGUTAR_A, 3, 70), (SOGUTAR_B, 0, 150), (SOGUTAR_B, 1, 9), (SOGUTAR_B, 1, 200), (SOGUTAR_B, 2, 33),
            (SOGUTAR_B, 4, 70), (SOGUTAR_C, 0, 1), (SOGUTAR_C, 0, 40), (SOGUTAR_C, 3, 7), (SOGUTAR_C, 3, 90)]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cfg,i,n", FF_CASES, ids=["a0", "a1", "a3", "b0", "b1", "b1-200", "b2", "b4", "c0-1", "c0", "c3", "c3-90"])
def test_feed_forward_alone(dt, cfg, i, n):
    """Dense: silu. Routed: gates and ups beyond the limit on both sides (the gate has no lower limit), identity experts among the
    chosen, every output chosen (c0), a shared expert with a limit of its own behind a gate a token."""
    cpu, dev, spec = layer_tensors(cfg, i, dt)
    h = Harness(dt)
    part = build_part("feed_forward", spec.feed_forward, h.env)
    part.load(dev)
    x = (1.5 * torch.randn(n, cfg["width"], generator=torch.Generator().manual_seed(8))).to(dt)
    got = whole(part.forward(x.to(DEV), h.ctx([(1, n, [])]))).cpu()
    f = cfg["layers"][i]["mlp"]
    if f["kind"] == "dense":
        return close(got, P.dense_ff(x.double(), cpu, f"l{i}.mlp."), dt)
    if n > 8:
        gate = x.double() @ cpu[f"l{i}.mlp.e0.gate"].T
        assert (gate > f["expert"]["limit"]).any() and (gate < -f["expert"]["limit"]).any(), "the case is meant to meet the limit"
    close(got, P.moe_ff(x.double(), cpu, f"l{i}.mlp.", f), dt)


def _attention_layer(heads, kv_heads, dim, vdim, window, rot, scaling=None):
    return one_layer({"type": "attention", "mixer": att(heads, kv_heads, dim, vdim, dim ** -0.5, window, rot, scaling), "mlp": None})


ATTENTION_CASES = [(SOGUTAR_A, 1), (SOGUTAR_B, 0), (SOGUTAR_B, 2), (SOGUTAR_C, 0), (SOGUTAR_C, 3),
                   (_attention_layer(6, 2, 64, 32, 16, (24, 1000.0), (4.0, 1.0, 4.0, 32)), 0), (_attention_layer(8, 1, 128, 128, None, None), 0),
                   (_attention_layer(2, 2, 32, 128, 7, (32, 5e5)), 0), (_attention_layer(12, 3, 128, 64, 21, (64, 100.0), (2.0, 0.5, 2.0, 16)), 0),
                   (_attention_layer(6, 2, 96, 48, 30, (24, 1e4)), 0)]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cfg,i", ATTENTION_CASES, ids=["a1", "b0", "b2", "c0", "c3", "64x32", "128x128", "32x128", "128x64", "96x48"])
@pytest.mark.parametrize("sharp", [False, True])
def test_attention_alone(dt, cfg, i, sharp):
    """A layer with keys of its own over a prompt portion, then over single tokens and further portions that read the first one's
    cache rows: one norm over all of q and one over all of k, windows shorter than a portion, of one page, and none; rotation of a
    part of a head with stretched frequencies, of all of it, and none; head sizes of every attention kernel."""
    cpu, dev, spec = layer_tensors(cfg, i, dt, sharp)
    part, h, cache = loaded("mixer", dt, spec.mixer, dev)
    m = cfg["layers"][i]["mixer"]
    x = (2 * torch.randn(100, cfg["width"], generator=torch.Generator().manual_seed(6))).to(dt)
    state = {}
    run_in_portions(part, h, cache, x, lambda xs: P.attention(xs, cpu, f"l{i}.mix.", m, cfg["norm"]["eps"], state), dt)


def test_rotation_frequencies():
    """The stretched frequencies against the three cases by hand: short wavelengths stay, long ones are divided, between them a blend."""
    from llmengine.parts.position import rope_inverse_frequencies
    from llmengine.parts.spec import PositionSpec
    rot = {"dims": 16, "base": 100.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 40}}
    spec = PositionSpec(kind="rope", head_dim=16, theta=100.0, max_positions=8, scaling_factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
                        original_max_positions=40, float64_frequencies=True)
    got, want = rope_inverse_frequencies(spec), P.frequencies(rot).numpy()
    np.testing.assert_allclose(got, want, rtol=1e-14)
    plain = np.array([100.0 ** (-2.0 * i / 16) for i in range(8)])
    wavelength = 2 * math.pi / plain
    assert (wavelength < 10).any() and (wavelength > 40).any() and ((wavelength > 10) & (wavelength < 40)).any()
    np.testing.assert_allclose(got[wavelength < 10], plain[wavelength < 10], rtol=1e-14)
    np.testing.assert_allclose(got[wavelength > 40], plain[wavelength > 40] / 4.0, rtol=1e-14)
    mid = (wavelength > 10) & (wavelength < 40)
    assert ((got[mid] < plain[mid]) & (got[mid] > plain[mid] / 4.0)).all()


def _probe_weights(cpu, dev, prefix, H, G, dk, dt, strength, with_keys=True):
    """Every query head asks along the model's first direction and every key answers along the second, with nothing else in
    either: a token whose input has the first direction set looks for the tokens whose input has the second one set. The norm
    over the projection then leaves one number a head, of size sqrt(dk) times its weight."""
    D = cpu[prefix + "q"].shape[1]
    q, k = torch.zeros(H * dk, D, dtype=torch.float64), torch.zeros(G * dk, D, dtype=torch.float64)
    q[dk - 1::dk, 0], k[dk - 1::dk, 1] = 1.0, 1.0     # the last number of a head: outside the rotated part
    names = [(prefix + "q", q), (prefix + "q.norm", torch.full((H * dk,), strength, dtype=torch.float64))]
    if with_keys:
        names += [(prefix + "k", k), (prefix + "k.norm", torch.ones(G * dk, dtype=torch.float64))]
    for name, w in names:
        cpu[name], dev[name] = w.to(dt).double(), w.to(DEV, dt if w.dim() == 2 else torch.float32)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("window,page", [(13, 4), (16, 16), (40, 16), (1, 4), (300, 16)])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("borrowed", [False, True])
def test_a_marked_key_just_inside_and_just_outside_the_window(dt, window, page, decoded, borrowed):
    """Hundreds of tokens of which one is marked; later tokens ask for it with a score that stands far out. The one that is
    `window - 1` behind it sees it and returns its value, the next one does not; the same when the asking tokens are decoded one
    by one, when the marked key lies on a page's last or first row, and when the asking layer reads ANOTHER layer's keys (whose
    own window is a different one) with a window of its own."""
    first = {"type": "attention", "mixer": att(4, 2, 16, 24, 0.25, 5 if borrowed else window, (8, 100.0)), "mlp": None}
    layers = [first] + ([{"type": "attention", "mixer": att(4, 2, 16, 24, 0.25, window, (8, 100.0), kv_from=0), "mlp": None}] if borrowed else [])
    cfg = one_layer(layers[-1], before=layers[:-1])
    cpu, dev, spec0 = layer_tensors(cfg, 0, dt)
    _probe_weights(cpu, dev, "l0.mix.", 4, 2, 16, dt, 60.0 / (0.25 * 16))
    T = 420
    owner, h, cache = loaded("mixer", dt, spec0.mixer, dev, page=page, pages=T // page + 4)
    assert owner.cache_needs()[0].window == (max(5, window) if borrowed else window)
    asker, m = owner, cfg["layers"][0]["mixer"]
    if borrowed:
        cpu1, dev1, spec1 = layer_tensors(cfg, 1, dt)
        _probe_weights(cpu1, dev1, "l1.mix.", 4, 2, 16, dt, 60.0 / (0.25 * 16), with_keys=False)
        asker = build_part("mixer", spec1.mixer, h.env)
        asker.load(dev1)
        assert not asker.cache_needs()
        cpu.update(cpu1)
        m = cfg["layers"][1]["mixer"]
    read = LayerCache(group=0, k=cache.k, v=cache.v, writes=False, window=cache.window)
    for marked in (page * 5 - 1, page * 5, 77):
        g = torch.Generator().manual_seed(marked)
        x = torch.randn(T, cfg["width"], generator=g)
        x[:, :2] = 0
        x[marked, 1] = 1.0                      # the key that is looked for
        x[marked, 2:] *= 3.0                    # and what it carries
        for a in (marked + window - 1, marked + window, marked + 150):
            if a < T and a != marked:
                x[a, 0] = 1.0
        x = x.to(dt)
        st0, st1 = {}, {}
        want = P.attention(x.double(), cpu, "l0.mix.", cfg["layers"][0]["mixer"], 1e-5, st0)
        if borrowed:
            want = P.attention(x.double(), cpu, "l1.mix.", m, 1e-5, st1, st0)
        cut = marked + 1 if decoded else T
        steps = [(0, cut)] + [(t, t + 1) for t in range(cut, min(T, marked + window + 2))]
        got = []
        for lo, hi in steps:
            ctx = h.ctx([(marked + 1, hi - lo, [])])
            y = owner.forward(x[lo:hi].to(DEV), ctx, cache)
            if borrowed:
                y = asker.forward(x[lo:hi].to(DEV), ctx, read)
            got.append(whole(y).cpu())
        got = torch.cat(got)
        close(got, want[:got.shape[0]], dt, f"marked key at {marked}")
        h.cm.release(marked + 1)
        if window > 1:  # the test tells the two apart: the value of the marked key is there, and one token later it is not
            v = (cpu["l0.mix.v"] @ x[marked].double()).view(2, 24)
            inside = marked + window - 1
            alone = torch.cat([v[a // 2] for a in range(4)]) @ cpu[("l1" if borrowed else "l0") + ".mix.o"].T
            assert float((want[inside] - alone).norm()) < 0.05 * float(alone.norm())
            if inside + 1 < T:
                assert float((want[inside + 1] - alone).norm()) > 0.5 * float(alone.norm())


RETENTION_CASES = [(SOGUTAR_A, 0), (SOGUTAR_A, 2), (SOGUTAR_B, 1), (SOGUTAR_B, 4), (SOGUTAR_C, 1),
                   (one_layer({"type": "retention", "mixer": ret(4, 128, 128, (0.9, 0.99, 0.999, 1.0), (128, 1e4)), "mlp": None}, width=96), 0),
                   (one_layer({"type": "retention", "mixer": ret(2, 100, 36, (0.0, 0.95), (50, 10.0)), "mlp": None}), 0)]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cfg,i", RETENTION_CASES, ids=["a0", "a2", "b1", "b4", "c1", "128x128", "100x36"])
def test_retention_alone(dt, cfg, i):
    """Portions of 1, 2 and many tokens that hand the state on through the slot; rotation of a part of a head, all of it and none;
    decays of 0 and 1; key sizes that fill a part of a lane's numbers and several lanes."""
    cpu, dev, spec = layer_tensors(cfg, i, dt)
    part, h, cache = loaded("mixer", dt, spec.mixer, dev)
    m = cfg["layers"][i]["mixer"]
    x = (2 * torch.randn(100, cfg["width"], generator=torch.Generator().manual_seed(16))).to(dt)
    state = {}
    run_in_portions(part, h, cache, x, lambda xs: P.retention(xs, cpu, f"l{i}.mix.", m, cfg["norm"]["eps"], state), dt)


def test_a_state_written_once_is_read_hundreds_of_tokens_later():
    """A decay of (nearly) one and a query that asks for one early token's key: what that token wrote is read 400 tokens later, after
    portions and single tokens; a state that is lost, reset or read from another slot on the way shows. No rotation, so that the
    early key and the late query meet."""
    dt = torch.float32
    cfg = one_layer({"type": "retention", "mixer": ret(2, 32, 48, (0.99999, 0.9999), None), "mlp": None})
    cpu, dev, spec = layer_tensors(cfg, 0, dt)
    part, h, cache = loaded("mixer", dt, spec.mixer, dev)
    m = cfg["layers"][0]["mixer"]
    T = 430
    x = 0.05 * torch.randn(T, cfg["width"], generator=torch.Generator().manual_seed(3))
    x[3] *= 60.0
    x[T - 2] = x[3]                                      # asks along the same directions as token 3 wrote
    state = {}
    want = P.retention(x.double(), cpu, "l0.mix.", m, 1e-5, state)
    got, lo = [], 0
    for n in (2, 1, 1, 130, 1, 2, 200, 61, 1, 1, 30):
        got.append(whole(part.forward(x[lo:lo + n].to(DEV), h.ctx([(1, n, [])]), cache)).cpu())
        lo += n
    assert lo == T
    close(torch.cat(got), want, dt, "portions", tol32=2e-4)
    fresh = P.retention(x[10:].double(), cpu, "l0.mix.", m, 1e-5, {})  # the same tokens without what token 3 wrote
    assert float((fresh[T - 12] - want[T - 2]).norm()) > 0.05 * float(want[T - 2].norm()), "the case is meant to depend on token 3"


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cfg,i", [(SOGUTAR_A, 0), (SOGUTAR_A, 1), (SOGUTAR_A, 2), (SOGUTAR_B, 1), (SOGUTAR_B, 2), (SOGUTAR_C, 3)],
                         ids=["a0", "a1", "a2", "b1", "b2", "c3"])
def test_parallel_block_with_one_norm_alone(dt, cfg, i):
    """A whole layer on a float32 stream: one layer norm whose rows the mixer and the feed-forward both read, their results added
    to the stream together; a layer without a feed-forward."""
    from llmengine.parts.base import Residual
    cpu, dev, spec = layer_tensors(cfg, i, dt)
    block, h, cache = loaded("block", dt, spec, dev)
    eps, l = cfg["norm"]["eps"], cfg["layers"][i]
    x = torch.randn(60, cfg["width"], generator=torch.Generator().manual_seed(46)) + 0.5
    state, lo = {}, 0
    for n in (17, 1, 2, 40):
        xs = x[lo:lo + n].double()
        hh = P.layer_norm(xs, cpu[f"l{i}.norm1"], eps)
        mix = P.attention if l["type"] == "attention" else P.retention
        want = xs + mix(hh, cpu, f"l{i}.mix.", l["mixer"], eps, state)
        f = l.get("mlp")
        if f:
            want = want + (P.dense_ff(hh, cpu, f"l{i}.mlp.") if f["kind"] == "dense" else P.moe_ff(hh, cpu, f"l{i}.mlp.", f))
        res = block.forward(Residual(x[lo:lo + n].to(DEV).contiguous()), h.ctx([(1, n, [])]), cache)
        if res.pending is not None:
            get_ops().residual_add(res.h, res.pending)
        close(res.h.float().cpu(), want, dt, f"tokens {lo}..{lo + n}", tol16=6e-2)
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


@pytest.fixture(scope="module", params=[(n, dt, sharp) for n in ("ga", "gb", "gc") for dt in DTYPES for sharp in (False, True)
                                        if not (sharp and n == "gc")],
                ids=lambda p: f"{p[0]}-{NAMES[p[1]]}{'-sharp' if p[2] else ''}")
def model(request, tmp_path_factory):
    name, dt, sharp = request.param
    cfg, page = SOGUTAR[name]
    d = write_model(str(tmp_path_factory.mktemp("sogutar")), cfg, dt, sharp=sharp)
    pc, pw = P.read_model(d)
    lens = [5, 64, 33, 130, 97] if name != "gb" else [3, 47, 64, 200, 129]
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


def test_the_stream_after_every_layer(model):
    """In float32 the residual stream behind every layer against the plain one."""
    dt, eng, reqs, _, _, (pc, pw), cfg = model
    if dt != torch.float32:
        pytest.skip("compared in float32")
    ids = reqs["r2"]
    after = []
    P.forward(pc, pw, ids, after_layers=after)
    got = []
    m = eng._ensure_model()
    m.after_run = lambda r, h: got.append(h[:len(ids)].float().cpu().clone())
    try:
        eng.run_step([(9, ids, [len(ids) - 1])], end=[9])
    finally:
        m.after_run = None
    assert len(got) == len(after) == len(cfg["layers"])
    for r, (a, b) in enumerate(zip(got, after)):
        close(a, b, dt, f"layer {r}")


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


def test_a_batch_of_unequal_requests_against_each_alone(model):
    """Four requests of unequal length in ONE step, then each alone: the same rows (float32: to rounding)."""
    dt, eng, reqs, plain, _, _, _ = model
    names = ["r0", "r2", "r1", "r4"]
    lg = eng.run_step([(20 + i, reqs[k], list(range(len(reqs[k])))) for i, k in enumerate(names)], end=[20, 21, 22, 23]).float().cpu().numpy().copy()
    lo = 0
    for k in names:
        n = len(reqs[k])
        alone = eng.run_step([(30, reqs[k], list(range(n)))], end=[30]).float().cpu().numpy()
        rows_close(lg[lo:lo + n], plain[k], dt, f"{k} in the batch", plain.get(k + ".rounded"))
        close(lg[lo:lo + n], alone, dt, f"{k}: batch against alone", tol32=2e-5, tol16=3e-2)
        lo += n


def test_a_slot_that_is_used_again_starts_at_zero(model):
    """Requests one after the other in an engine with a single live request at a time: each gets the one before's slot and
    pages, and must not see its state or its keys."""
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


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("dim,vdim,window", [(64, 64, 136), (64, 64, None), (128, 128, 700), (32, 64, 200), (48, 48, 136)])
def test_single_tokens_behind_long_contexts(dt, dim, vdim, window, tmp_path):
    """Three requests of unequal length (up to 1,500 tokens) whose last tokens come one a step, side by side: single tokens whose
    key range is cut into pieces that run side by side and are merged, with a window that ends inside a piece, begins behind
    whole pieces, or is absent; an attention layer on borrowed keys and a retention layer behind it."""
    layers = [{"type": "attention", "mixer": att(4, 2, dim, vdim, dim ** -0.5, window, (dim // 2, 1e4), (4.0, 1.0, 4.0, 256)), "mlp": dense(64)},
              {"type": "retention", "mixer": ret(2, 32, 48, (0.99, 0.999), (16, 100.0)), "mlp": None},
              {"type": "attention", "mixer": att(4, 2, dim, vdim, 0.1, 90 if window else 300, (dim // 2, 1e4), (4.0, 1.0, 4.0, 256), kv_from=0), "mlp": None}]
    cfg = {"architecture": "Sogutar", "vocab": 120, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 20.0, "max_positions": 2048, "layers": layers}
    d = write_model(str(tmp_path / "m"), cfg, dt, sharp=True)
    pc, pw = P.read_model(d)
    reqs = {"a": random_ids(1500, 120, 1), "b": random_ids(700, 120, 2), "c": random_ids(200, 120, 3)}
    tail = 24
    eng = llmengine.Engine(d, NAMES[dt], block_size=16)
    eng.configure_cache(num_blocks=(1536 + 704 + 256) // 16, block_size=16, num_slots=4)
    ids = {"a": 1, "b": 2, "c": 3}
    for k, v in reqs.items():
        eng.run_step([(ids[k], v[:-tail], [])], end=[])
    rows = {k: [] for k in reqs}
    for t in range(tail):
        batch = [(ids[k], [v[len(v) - tail + t]], [0]) for k, v in reqs.items()]
        lg = eng.run_step(batch, end=list(ids.values()) if t == tail - 1 else []).float().cpu().numpy()
        for i, k in enumerate(reqs):
            rows[k].append(lg[i].copy())
    for k, v in reqs.items():
        want = P.forward(pc, pw, v).numpy()[-tail:]
        rounded = rounded_forward(pc, pw, v)[-tail:] if dt == torch.bfloat16 else None
        rows_close(np.stack(rows[k]), want, dt, f"request {k}", rounded)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["ga", "gb"])
def test_replay_through_the_command(dtype, name, tmp_path):
    """bin/trace_run as a user runs it."""
    cfg, page = SOGUTAR[name]
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
    d = write_model(str(tmp_path / "model"), SOGUTAR_C, torch.float32)
    r = run_cli("--model", d, "--prompt-ids", "5,17,3,90", "--max-new", "6", "--block-size", "8", "--num-blocks", "32")
    assert r.returncode == 0, r.stderr
    line = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")][0]
    pc, pw = P.read_model(d)
    assert line["token_ids"] == P.greedy(pc, pw, [5, 17, 3, 90], 6) and line["finish_reason"] == "length"
