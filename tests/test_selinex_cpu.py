"""Selinex without a GPU: configuration and its errors, the description in parts (tensor names, the layer order of a loop, what a
file may carry unread, sizes that only tensor shapes give), the random-weights mode, the plain implementation against itself (whole
prompts against portions and single tokens; every mechanism's rule on cases made by hand), and the engine's host side on the test
double of the kernels."""
import copy
import json
import math

import numpy as np
import pytest
import torch

import llmengine
import plain_selinex as P
from llmengine.config import ConfigError
from llmengine.config.registry import config_from_dir, get_architecture
from llmengine.config.selinex import SelinexConfig
from llmengine.models.selinex import describe_selinex
from llmengine.weights.random_init import model_tensor_needs
from cpu_ops import CpuOps
from tiny import random_ids
from tiny_selinex import RANKS, SELINEX, SELINEX_A, SELINEX_B, SELINEX_C, SELINEX_D, make_tensors, write_model


def with_ranks(cfg, name):
    """The configuration with the ranks that a model folder's tensor shapes would add."""
    c = copy.deepcopy(cfg)
    for i, r in RANKS[name].items():
        c["layers"][i]["mixer"]["right"]["rank"] = r
    return c


@pytest.mark.parametrize("name", sorted(SELINEX))
def test_configuration_round_trip_and_tensor_names(name):
    cfg = with_ranks(SELINEX[name][0], name)
    c = SelinexConfig.from_dict(cfg)
    assert SelinexConfig.from_dict(c.to_dict()) == c
    assert get_architecture("Selinex").parse_config(cfg, None) == c
    spec = describe_selinex(c)
    needs = model_tensor_needs(spec)
    made = make_tensors(SELINEX[name][0], 1, torch.float32)
    assert set(needs) <= set(made)
    for k in set(made) - set(needs):
        assert k in spec.ignore, k
    for k, n in needs.items():
        assert tuple(made[k].shape) == tuple(n.shape), k
    assert [b.kind for b in spec.layers] == ["sandwich"] * len(cfg["layers"])
    assert [r.layer for r in spec.order] == P.layer_order(cfg)


def test_description_reads_every_option():
    spec = describe_selinex(SelinexConfig.from_dict(with_ranks(SELINEX_A, "sa")))
    assert [b.mixer.kind for b in spec.layers] == ["gated_delta", "mixer_pair", "mixer_pair", "gated_delta"]
    assert [r.layer for r in spec.order] == [0, 1, 2, 1, 2, 1, 2, 3]
    d0, d3 = spec.layers[0].mixer, spec.layers[3].mixer
    assert (d0.heads, d0.kv_heads, d0.dim, d0.vdim, d0.taps) == (4, 2, 12, 10, 3) and d3.taps == 1 and d0.unit_eps == 1e-6
    p1, p2 = spec.layers[1].mixer, spec.layers[2].mixer
    assert (p1.combine, p1.left_scale, p1.right_scale) == ("weighted", 1.3, 0.7) and p2.combine == "normed_mean"
    assert (p2.left_norm, p2.right_norm) == ("l2.mix.left.out", "l2.mix.right.out")
    a1, a2 = p1.left, p2.left
    assert (a1.num_heads, a1.num_kv_heads, a1.head_dim, a1.value_dim, a1.window, a1.scale) == (6, 2, 24, 10, 13, 0.21)
    assert a1.gate_weight == "l1.mix.left.g" and a1.gate_per_head and a2.gate_weight is None
    assert a1.position.dims == 0 and (a2.position.dims, a2.position.base, a2.window) == (8, 777.0, 9)
    r1, r2 = p1.right, p2.right
    assert (r1.kind, r1.heads, r1.dim, r1.vdim, r1.tau, r1.rank) == ("decayed_linear_attention", 3, 20, 14, 7.0, 5)
    assert (r2.kind, r2.heads, r2.dim, r2.rank) == ("token_shift_mix", 5, 14, 3)
    f0, f1, f3 = spec.layers[0].feed_forward, spec.layers[1].feed_forward, spec.layers[3].feed_forward
    assert (f0.experts, f0.top, f0.groups, f0.keep_groups, f0.group_top, f0.score, f0.normalize) == (6, 2, 3, 2, 2, "sigmoid", False)
    assert (f1.activation, f1.limit, f1.slope, f1.intermediate) == ("clamped_swish", 0.8, 1.702, 44)
    assert (f3.groups, f3.keep_groups, f3.top) == (1, 1, 1)
    assert spec.layers[2].feed_forward is None and spec.layers[2].norm2 is None and "l2.norm2" in spec.ignore
    assert all(b.residual_mult == 0.6 for b in spec.layers) and spec.head.weight == "embed" == spec.embedding.weight
    assert all(b.norm1.kind == "rmsnorm_unit_offset" and b.norm1_out.kind == "rmsnorm_unit_offset" for b in spec.layers)


@pytest.mark.parametrize("cfg,order", [(SELINEX_B, [0, 1, 2]), (SELINEX_C, [0, 1, 2, 0, 1, 2]), (SELINEX_D, [0, 1])])
def test_layer_order_of_a_loop(cfg, order):
    spec = describe_selinex(SelinexConfig.from_dict(cfg))
    assert [r.layer for r in spec.order] == order == P.layer_order(cfg)
    c = copy.deepcopy(SELINEX_A)
    c["loop"] = {"start": 3, "stop": 4, "times": 1}  # a loop that runs once changes nothing
    assert [r.layer for r in describe_selinex(SelinexConfig.from_dict(c)).order] == [0, 1, 2, 3]


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][2]["mixer"]["left"]["rot"].update(dims=14), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][1]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][3]["mlp"].update(kind="sparse"), "unknown kind"),
    (lambda c: c["layers"][0]["mixer"].pop("conv"), "conv"),
    (lambda c: c["loop"].update(stop=5), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_errors(change, word):
    cfg = copy.deepcopy(SELINEX_A)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        SelinexConfig.from_dict(cfg)
    assert word in str(e.value)


@pytest.mark.parametrize("name", sorted(SELINEX))
def test_ranks_come_from_the_tensor_shapes(name, tmp_path):
    """config.json names no rank of a low-rank decay map: a model folder's configuration takes it from the checkpoint's header."""
    cfg = SELINEX[name][0]
    d = write_model(str(tmp_path / "m"), cfg, torch.bfloat16)
    arch, parsed = config_from_dir(d)
    assert arch.name == "Selinex"
    for i, r in RANKS[name].items():
        assert parsed.layers[i].mixer.right.rank == r
    assert parsed == SelinexConfig.from_dict(with_ranks(cfg, name))


def test_random_weights_mode_writes_the_design(tmp_path):
    d = llmengine.write_random_model(str(tmp_path / "m"), with_ranks(SELINEX_C, "sc"), seed=3, dtype=torch.bfloat16)
    arch, cfg = config_from_dir(d)
    assert arch.name == "Selinex" and cfg == SelinexConfig.from_dict(with_ranks(SELINEX_C, "sc"))
    pc, pw = P.read_model(d)
    assert set(pw) == set(model_tensor_needs(describe_selinex(cfg)))
    assert pw["l0.mix.right.a1"].shape == (2, 48) and pw["l2.mix.right.w2"].shape == (18, 7) and pw["l2.mix.right.u"].shape == (3, 6)
    assert pw["l1.mix.q.conv"].shape == (20, 2) and pw["l0.mix.left.g"].shape == (5, 48)
    assert torch.isfinite(P.forward(pc, pw, [1, 2, 3, 4])).all()


# ---------------------------------------------------------------------------------------------- the plain implementation
@pytest.mark.parametrize("name", sorted(SELINEX))
def test_plain_portions_and_single_tokens_match_the_whole_prompt(name, tmp_path):
    cfg = SELINEX[name][0]
    d = write_model(str(tmp_path / "m"), cfg, torch.float32, sharp=True)
    pc, pw = P.read_model(d)
    ids = [(7 * i * i + 3 * i + 1) % cfg["vocab"] for i in range(75)]
    want = P.forward(pc, pw, ids)
    for cuts in ([1, 2, 30, 31, 33, 60, 75], list(range(1, 76))):
        seq, got, lo = P.Sequence(pc), [], 0
        for hi in cuts:
            got.append(P.forward(pc, pw, ids[lo:hi], seq))
            lo = hi
        assert float((torch.cat(got) - want).abs().max()) < 1e-9


def test_plain_router_rules():
    def logit(p):
        return torch.log(torch.tensor(p, dtype=torch.float64)) - torch.log1p(-torch.tensor(p, dtype=torch.float64))

    s = [0.05, 0.90, 0.10, 0.05, 0.50, 0.46, 0.12, 0.08]
    z, zero = logit(s), torch.zeros(8, dtype=torch.float64)
    # no groups: the largest scores; the weights are the scores themselves, not divided by their sum
    chosen, w = P.choose_experts(z, zero, 2, 0, 0)
    assert chosen.tolist() == [1, 4] and np.allclose(w.numpy(), [0.90, 0.50])
    # four groups of two, one stays: a group counts by the sum of its two largest, so (0.50, 0.46) beats (0.05, 0.90) although that one holds the largest score
    chosen, w = P.choose_experts(z, zero, 2, 4, 1)
    assert chosen.tolist() == [4, 5] and np.allclose(w.numpy(), [0.50, 0.46])
    # two groups of four: (0.90 + 0.10) against (0.50 + 0.46); only the group's two largest count
    chosen, w = P.choose_experts(z, zero, 3, 2, 1)
    assert chosen.tolist() == [1, 2, 0]  # 0.05 twice: the lower index first
    # the correction moves the choice and not the weights; choice scores below zero still win inside a kept group, and the
    # experts of a dropped group count as minus infinity although every kept score is negative
    corr = torch.tensor([-2.0, -2.9, -2.0, -2.0, -3.0, -3.0, -3.0, -3.0], dtype=torch.float64)
    chosen, w = P.choose_experts(z, corr, 3, 2, 1)
    assert chosen.tolist() == [2, 0, 3] and np.allclose(w.numpy(), [0.10, 0.05, 0.05])


def test_plain_window_and_gate_rules():
    """One head whose last query matches the first key only: a key `size - 1` back is seen, a key `size` back is not; the gate
    multiplies the head's result."""
    f = torch.float64
    w = {"q": torch.tensor([[40.0, 0, 0]], dtype=f), "k": torch.tensor([[0, 1.0, 0]], dtype=f), "v": torch.tensor([[0, 0, 1.0]], dtype=f),
         "o": torch.tensor([[1.0], [0], [0]], dtype=f), "g": torch.zeros(1, 3, dtype=f)}
    h = torch.tensor([[0, 1.0, 7], [0, 0, 1], [0, 0, 2], [1, 0, 3]], dtype=f)  # (asks, is asked for, carries)

    def last(size, gated=True):
        m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "scale": 1.0, "mask": {"size": size}}
        return float(P.window_attention(h, w, "", m, {}, gated=gated)[3, 0])

    assert abs(last(3) - 0.5 * (1 + 2 + 3) / 3) < 1e-12       # the first token is three back: outside; the gate is sigmoid(0)
    assert abs(last(4) - 0.5 * 7) < 1e-9                      # inside: its score of 40 takes all the weight
    assert abs(last(4, gated=False) - 7) < 1e-9
    assert abs(last(1) - 0.5 * 3) < 1e-12                     # a window of one key: the token itself


def test_plain_recurrences_by_hand():
    """Two tokens through each recurrence, by hand."""
    one = torch.ones(1, 1, dtype=torch.float64)
    # decay per key channel: S1 = k1 v1; S2 = a2 S1 + k2 v2; o2 = S2 q2 / sqrt(dk)
    w = {"q": one * 2, "k": one * 3, "v": one * 5, "g": one, "o": one, "norm": torch.ones(1, dtype=torch.float64),
         "a1": one, "a2": one, "a2.b": torch.zeros(1, dtype=torch.float64)}
    st = {}
    P.decayed_linear_attention(torch.tensor([[1.0], [2.0]], dtype=torch.float64), w, "", {"heads": 1, "dim": 1, "vdim": 1, "tau": 2.0}, st, 0.0)
    a2 = (1 / (1 + math.exp(-2.0))) ** 0.5
    assert abs(float(st["S"]) - (a2 * 15 + 60)) < 1e-12
    # token shift with a bonus: o2 = (S1 + u k2 v2) r2 with S1 = k1 v1 (the first token's previous input is zero)
    w = {"mu." + s: torch.full((1,), 0.25, dtype=torch.float64) for s in "rkvgw"}
    w.update({"r": one, "k": one, "v": one, "g": one, "o": one, "w1": one, "w2": one, "w0": torch.zeros(1, dtype=torch.float64),
              "u": one * 0.5, "norm": torch.ones(1, dtype=torch.float64)})
    st = {}
    P.token_shift_recurrence(torch.tensor([[4.0], [8.0]], dtype=torch.float64), w, "", {"heads": 1, "dim": 1}, st, 0.0)
    x1, x2 = 4 + (0 - 4) * 0.25, 8 + (4 - 8) * 0.25
    decay2 = math.exp(-math.exp(math.tanh(x2)))
    assert abs(float(st["S"]) - (decay2 * x1 * x1 + x2 * x2)) < 1e-12 and float(st["prev"]) == 8.0
    # delta rule: with beta = 1 and no decay the state answers k with v exactly
    w = {"q": torch.eye(2, dtype=torch.float64), "k": torch.eye(2, dtype=torch.float64), "v": torch.eye(2, dtype=torch.float64),
         "g": torch.eye(2, dtype=torch.float64), "o": torch.eye(2, dtype=torch.float64), "norm": torch.ones(2, dtype=torch.float64),
         "b": torch.full((1, 2), 50.0, dtype=torch.float64), "a": torch.zeros(1, 2, dtype=torch.float64),
         "A_log": torch.full((1,), -40.0, dtype=torch.float64), "dt_bias": torch.zeros(1, dtype=torch.float64)}
    for s in "qkv":
        w[s + ".conv"] = torch.ones(2, 1, dtype=torch.float64)
    st = {}
    h = torch.tensor([[3.0, 0.1], [0.2, 2.0]], dtype=torch.float64)
    P.gated_delta(h, w, "", {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "conv": 1}, st, 0.0)
    k2 = P.silu(h[1]); k2 = k2 / torch.sqrt((k2 * k2).sum() + 1e-6)
    assert torch.allclose(st["S"][0].t() @ k2, P.silu(h[1]), atol=1e-6)


# ---------------------------------------------------------------------------------------------- the engine's host side
@pytest.fixture(scope="module", params=["sa", "sc", "sd"])
def cpu_engine(request, tmp_path_factory):
    """The engine on the test double of the kernels: batch building, block tables, state slots of every run of a looped layer,
    the wiring of the parts."""
    cfg, page = SELINEX[request.param]
    d = write_model(str(tmp_path_factory.mktemp("selinex_" + request.param)), cfg, torch.float32, sharp=True)
    eng = llmengine.Engine(d, "fp32", device="cpu", ops=CpuOps(), block_size=page, num_blocks=40)
    eng.configure_cache(num_blocks=40, block_size=page, num_slots=3)
    return eng, P.read_model(d), cfg


def test_engine_on_the_test_double_matches_plain(cpu_engine):
    eng, (pc, pw), cfg = cpu_engine
    a, b = random_ids(37, cfg["vocab"], 1), random_ids(11, cfg["vocab"], 2)
    want = {k: P.forward(pc, pw, ids).numpy() for k, ids in (("a", a), ("b", b))}
    got = eng.run_step([(1, a, list(range(len(a))))], end=[1]).numpy()
    assert np.abs(got - want["a"]).max() < 2e-4
    rows = {}
    steps = [([(2, a[:9], [8]), (3, b[:10], [9])], []), ([(2, a[9:11], [0, 1]), (3, b[10:], [0])], [3]),
             ([(2, a[11:36], [24]), (4, b[:3], [2])], []), ([(2, a[36:], [0]), (4, b[3:], [7])], [2, 4])]
    at = {2: 0, 3: 0, 4: 0}
    for batch, end in steps:
        lg = eng.run_step(batch, end=end).numpy().copy()
        i = 0
        for rid, toks, w in batch:
            for k in w:
                rows[(rid, at[rid] + k)] = lg[i]
                i += 1
            at[rid] += len(toks)
    for (rid, pos), row in rows.items():
        ref = want["a"] if rid == 2 else want["b"]
        assert np.abs(row - ref[pos]).max() < 2e-4, (rid, pos)
    assert eng.cm.num_requests == 0


def test_stream_after_every_layer_run_on_the_test_double(cpu_engine):
    """Model.after_run sees the stream behind every run of a layer; a looped layer counts each time."""
    eng, (pc, pw), cfg = cpu_engine
    ids = random_ids(23, cfg["vocab"], 4)
    want, got = [], []
    P.forward(pc, pw, ids, after_layers=want)
    model = eng._ensure_model()
    model.after_run = lambda r, h: got.append((r, h.clone()))
    try:
        eng.run_step([(8, ids, [len(ids) - 1])], end=[8])
    finally:
        model.after_run = None
    assert [r for r, _ in got] == list(range(len(P.layer_order(cfg)))) and len(want) == len(got)
    for (r, a), b in zip(got, want):
        assert float((a.double() - b).abs().max()) < 2e-4 * max(1.0, float(b.abs().max())), r


def test_generation_through_the_scheduler_matches_plain(cpu_engine):
    eng, (pc, pw), cfg = cpu_engine
    prompt = random_ids(9, cfg["vocab"], 3)
    out, reason = eng.generate(prompt, 7)
    assert reason == "length" and out == P.greedy(pc, pw, prompt, 7)


def test_command_line_random_weights_mode(tmp_path):
    from test_cli import run_cli
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(SELINEX_B))
    out = tmp_path / "model"
    r = run_cli("--random-weights", str(out), "--config", str(cfg), "--seed", "4", "--dtype", "bf16")
    assert r.returncode == 0, r.stderr
    arch, parsed = config_from_dir(str(out))
    assert arch.name == "Selinex" and len(parsed.layers) == 3
    names = set(P.read_safetensors(str(out / "model.safetensors")))
    assert names >= {"embed", "final.norm", "l0.mix.right.mu.w", "l0.mix.left.out", "l1.mix.right.a2.b", "l1.mlp.correction", "l2.mix.A_log",
                     "l2.mlp.e15.down", "l0.norm2b"}
