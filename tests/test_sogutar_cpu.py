"""Sogutar without a GPU: configuration and its errors, the description in parts (tensor names, which run reads whose cache, how
many keys a cache keeps for its borrowers, sizes that tensor shapes give), the random-weights mode, the plain implementation
against itself (whole prompts against portions and single tokens; every mechanism's rule on cases made by hand), and the engine's
host side on the test double of the kernels."""
import copy
import json
import math

import numpy as np
import pytest
import torch

import llmengine
import plain_sogutar as P
from llmengine.config import ConfigError
from llmengine.config.registry import config_from_dir, get_architecture
from llmengine.config.sogutar import SogutarConfig, sizes_from_tensors
from llmengine.models.sogutar import describe_sogutar, kept_window
from llmengine.weights.random_init import model_tensor_needs
from cpu_ops import CpuOps
from tiny import random_ids
from tiny_sogutar import SOGUTAR, SOGUTAR_A, SOGUTAR_B, SOGUTAR_C, make_tensors, write_model


@pytest.mark.parametrize("name", sorted(SOGUTAR))
def test_configuration_round_trip_and_tensor_names(name):
    cfg = SOGUTAR[name][0]
    c = SogutarConfig.from_dict(cfg)
    assert SogutarConfig.from_dict(c.to_dict()) == c
    assert get_architecture("Sogutar").parse_config(cfg, None) == c
    spec = describe_sogutar(c)
    needs = model_tensor_needs(spec)
    made = make_tensors(cfg, 1, torch.float32)
    assert set(needs) == set(made)
    for k, n in needs.items():
        assert tuple(made[k].shape) == tuple(n.shape), k
    assert [b.kind for b in spec.layers] == ["parallel"] * len(cfg["layers"])
    assert [r.layer for r in spec.order] == list(range(len(cfg["layers"])))
    assert [r.cache_from for r in spec.order] == [l["mixer"].get("kv_from") for l in cfg["layers"]]


def test_description_reads_every_option():
    spec = describe_sogutar(SogutarConfig.from_dict(SOGUTAR_A))
    assert [b.mixer.kind for b in spec.layers] == ["retention", "gated_attention", "retention", "gated_attention"]
    assert all(b.norm2 is None and b.norm1.kind == "layernorm" for b in spec.layers) and spec.layers[2].feed_forward is None
    assert spec.embedding.kind == "lookup_normed" and spec.embedding.norm.weight == "embed.norm" and spec.head.weight == "embed"
    assert spec.head.softcap == 9.0 and describe_sogutar(SogutarConfig.from_dict(SOGUTAR_B)).head.softcap == 0.0
    r0, a1, r2, a3 = (b.mixer for b in spec.layers)
    assert (r0.heads, r0.dim, r0.vdim, r0.decay) == (3, 20, 14, (0.9, 0.99, 0.999)) and r0.k_scale == 20 ** -0.5
    assert (r0.position.head_dim, r0.position.theta, r0.position.original_max_positions) == (12, 5000.0, 0)
    assert r2.position.kind == "rope_ramp" and r2.position.dims == 0   # nothing is rotated
    assert (a1.num_heads, a1.num_kv_heads, a1.head_dim, a1.value_dim, a1.scale, a1.window) == (6, 2, 24, 10, 0.21, 13)
    assert a1.norm_scope == "projection" and a1.own_kv and a1.k_norm == "l1.mix.k.norm" and a1.q_norm == "l1.mix.q.norm"
    p = a1.position
    assert (p.head_dim, p.theta, p.scaling_factor, p.low_freq_factor, p.high_freq_factor, p.original_max_positions) == (8, 777.0, 3.0, 1.0, 3.0, 40)
    assert p.float64_frequencies
    assert not a3.own_kv and a3.k_norm is None and a3.window == 21 and a3.position == a1.position
    assert a1.cache_window == 21 and a3.cache_window is None    # the owner keeps what its widest reader asks for
    f0, f3 = spec.layers[0].feed_forward, spec.layers[3].feed_forward
    assert (f0.experts, f0.identity, f0.top, f0.weight_scale, f0.limit, f0.slope, f0.activation) == (5, 1, 2, 1.7, 0.8, 1.702, "clamped_swish")
    assert (f0.score, f0.normalize, f0.norm_eps, f0.correction, f0.shared_gate) == ("softmax", True, 1e-20, "l0.mlp.correction", "l0.mlp.shared.sg")
    assert (f0.shared.intermediate, f0.shared.limit, f0.shared.activation) == (28, 1.1, "clamped_swish")
    assert f3.shared is None and f3.shared_gate is None and f3.identity == 0
    assert spec.layers[1].feed_forward.activation == "silu"


def test_a_cache_keeps_what_its_widest_reader_asks_for():
    c = SogutarConfig.from_dict(SOGUTAR_C)   # layer 0 (window 8) is read by layer 2 (window 1) and layer 4 (no window)
    assert kept_window(c, 0) == 0
    b = SogutarConfig.from_dict(SOGUTAR_B)   # layer 0 (window 48) is read by layer 3 (window 17)
    assert kept_window(b, 0) == 48 and kept_window(b, 2) == 40
    from llmengine.engine.model import Model
    from llmengine.parts.base import BuildEnv
    m = Model(describe_sogutar(b), BuildEnv(torch.device("cpu"), torch.float32, CpuOps(), 16))
    assert sorted(m.windows) == [40, 48] and m.run_group[3] is None and m.run_needs[3] == ()


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][1]["mixer"].update(heads=5), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5, 0.5]), "a number a head"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5, 0.5, 1.5]), "[0, 1]"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "no earlier attention layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "no earlier attention layer"),
    (lambda c: c["layers"][3]["mixer"].update(dim=32), "differ"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].update(high=1.0), "high > low"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "experts"),
    (lambda c: c["layers"][0]["mlp"]["expert"].update(limit=0.0), "limit"),
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "unknown kind"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
])
def test_configuration_errors(change, message):
    cfg = copy.deepcopy(SOGUTAR_A)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        SogutarConfig.from_dict(cfg)
    assert message in str(e.value)


def test_a_layer_cannot_borrow_from_a_borrower():
    cfg = copy.deepcopy(SOGUTAR_C)
    cfg["layers"][4]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError) as e:
        SogutarConfig.from_dict(cfg)
    assert "no keys and values of its own" in str(e.value)


def test_sizes_that_only_tensor_shapes_give(tmp_path):
    """A file without vocab, width, a head's sizes and the feed-forwards' inner sizes: the checkpoint's header gives them."""
    d = write_model(str(tmp_path / "m"), SOGUTAR_A, torch.float32)
    cfg = copy.deepcopy(SOGUTAR_A)
    del cfg["vocab"], cfg["width"]
    for l in cfg["layers"]:
        if l["mixer"].get("kv_from") is None:
            del l["mixer"]["dim"], l["mixer"]["vdim"]
        f = l["mlp"]
        if f and f["kind"] == "dense":
            del f["ff"]
        elif f:
            del f["expert"]["ff"]
            if "shared" in f:
                del f["shared"]["ff"]
    del cfg["layers"][1]["mixer"]["kv_heads"]
    with open(tmp_path / "m" / "config.json", "w") as f:
        json.dump(cfg, f)
    arch, parsed = config_from_dir(str(tmp_path / "m"))
    assert parsed == SogutarConfig.from_dict(SOGUTAR_A)
    assert sizes_from_tensors(SOGUTAR_A, lambda name: (1, 1))["layers"] == SOGUTAR_A["layers"]   # what the file says stays


def test_random_weights_mode(tmp_path):
    d = llmengine.write_random_model(str(tmp_path / "m"), SOGUTAR_B, seed=3, dtype=torch.bfloat16)
    arch, parsed = config_from_dir(d)
    assert arch.name == "Sogutar" and len(parsed.layers) == 5
    names = set(P.read_safetensors(str(tmp_path / "m" / "model.safetensors")))
    assert names >= {"embed", "embed.norm", "final.norm", "l0.mix.k.norm", "l1.mix.g", "l1.mlp.correction", "l1.mlp.e5.down", "l1.mlp.shared.sg", "l3.mix.q.norm"}
    assert "l3.mix.k" not in names and "l1.mlp.e6.gate" not in names and "l0.norm2" not in names


# ---------------------------------------------------------------------------------------------- the plain rules by hand
def test_plain_layer_norm_by_hand():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 0.5, -1.0], dtype=torch.float64)
    d = x - 3.0
    want = d / math.sqrt((4 + 1 + 0 + 9) / 4 + 0.1) * w
    assert torch.allclose(P.layer_norm(x, w, 0.1), want)


def test_plain_rotation_by_hand():
    rot = {"dims": 4, "base": 100.0}
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]], dtype=torch.float64)
    y = P.rotate(x, 3, rot)
    f = [1.0, 100.0 ** -0.5]
    for i in range(2):
        a = 3 * f[i]
        assert math.isclose(float(y[0, i]), float(x[0, i]) * math.cos(a) - float(x[0, i + 2]) * math.sin(a))
        assert math.isclose(float(y[0, i + 2]), float(x[0, i + 2]) * math.cos(a) + float(x[0, i]) * math.sin(a))
    assert y[0, 4:].tolist() == [5.0, 6.0] and P.rotate(x, 0, rot).tolist() == x.tolist()


def test_plain_router_by_hand():
    """Three experts and one identity expert; the correction moves the choice from expert 0 to the identity expert, the weights
    are the softmax's own numbers divided by their sum, times the scale."""
    w = {"router": torch.eye(4, dtype=torch.float64), "correction": torch.tensor([-1.0, 0.0, 0.0, 0.5], dtype=torch.float64)}
    h = torch.tensor([[2.0, 1.0, 0.0, 0.5]], dtype=torch.float64)
    picks, weights = P.route(h, w, "", {"top": 2, "scale": 3.0})
    s = torch.softmax(h[0], 0)
    assert picks[0] == [3, 1]
    assert torch.allclose(weights[0], torch.stack([s[3], s[1]]) / (s[3] + s[1]) * 3.0)


def test_plain_experts_by_hand():
    w = {"gate": torch.tensor([[1.0], [1.0]], dtype=torch.float64), "up": torch.tensor([[1.0], [-1.0]], dtype=torch.float64),
         "down": torch.eye(2, dtype=torch.float64)}
    y = P.clamped_expert(torch.tensor([[5.0]], dtype=torch.float64), w, "", 2.0)   # gate 5 -> 2; up 5 -> 2 and -5 -> -2
    g = 2.0 / (1.0 + math.exp(-1.702 * 2.0))
    assert torch.allclose(y, torch.tensor([[g * 3.0, g * -1.0]], dtype=torch.float64))
    y = P.clamped_expert(torch.tensor([[-5.0]], dtype=torch.float64), w, "", 2.0)  # the gate has no lower limit
    g = -5.0 / (1.0 + math.exp(1.702 * 5.0))
    assert torch.allclose(y, torch.tensor([[g * -1.0, g * 3.0]], dtype=torch.float64))


def test_plain_identity_expert_and_shared_gate_by_hand():
    D = 3
    w = {"router": torch.tensor([[0.0, 0.0, 0.0], [9.0, 0.0, 0.0]], dtype=torch.float64), "correction": torch.zeros(2, dtype=torch.float64),
         "e0.gate": torch.zeros(2, D, dtype=torch.float64), "e0.up": torch.zeros(2, D, dtype=torch.float64), "e0.down": torch.zeros(D, 2, dtype=torch.float64),
         "shared.gate": torch.ones(1, D, dtype=torch.float64), "shared.up": torch.zeros(1, D, dtype=torch.float64),
         "shared.down": torch.ones(D, 1, dtype=torch.float64), "shared.sg": torch.tensor([[0.0, 1.0, 0.0]], dtype=torch.float64)}
    f = {"expert": {"ff": 2, "limit": 1.0}, "router": {"experts": 1, "identity": 1, "top": 1, "scale": 2.0}, "shared": {"ff": 1, "limit": 0.5}}
    h = torch.tensor([[1.0, 2.0, 3.0]], dtype=torch.float64)
    y = P.moe_ff(h, w, "", f)
    g = 0.5 / (1.0 + math.exp(-1.702 * 0.5))            # the shared expert: gate 6 -> 0.5, up 0 -> times (0 + 1)
    want = 2.0 * h + (1.0 / (1.0 + math.exp(-2.0))) * g  # the identity expert with weight 1 * scale, plus sigmoid(h . sg) * shared
    assert torch.allclose(y, want)


def test_plain_retention_by_hand():
    """One head of two key channels and one value, no rotation: after two tokens S = decay k1 v1 + k2 v2 and o = S^T q."""
    w = {"q": torch.eye(2, dtype=torch.float64), "k": torch.eye(2, dtype=torch.float64), "v": torch.tensor([[1.0, 1.0]], dtype=torch.float64),
         "g": torch.tensor([[1.0, 0.0]], dtype=torch.float64), "o": torch.tensor([[1.0], [0.0]], dtype=torch.float64)}
    h = torch.tensor([[1.0, 0.0], [0.0, 2.0]], dtype=torch.float64)
    st = {}
    P.retention(h, w, "", {"heads": 1, "dim": 2, "vdim": 1, "decay": [0.5]}, 0.0, st)
    k1, k2 = h[0] * 2 ** -0.5, h[1] * 2 ** -0.5
    assert torch.allclose(st["S"][0][:, 0], 0.5 * k1 * 1.0 + k2 * 2.0)


def test_plain_window_and_borrowed_keys_by_hand():
    """A window of 2 sees itself and one token back; a layer that borrows reads the owner's keys with its own window."""
    cfg = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 1.0, "mask": {"size": 2}}
    w = {"q": torch.zeros(2, 2, dtype=torch.float64), "q.norm": torch.ones(2, dtype=torch.float64), "k": torch.eye(2, dtype=torch.float64),
         "k.norm": torch.ones(2, dtype=torch.float64), "v": torch.eye(2, dtype=torch.float64), "o": torch.eye(2, dtype=torch.float64)}
    h = torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0], [2.0, 0.0]], dtype=torch.float64)
    st = {}
    y = P.attention(h, w, "", cfg, 1e-9, st)      # queries are zero: a plain mean over the visible values
    assert torch.allclose(y[0], h[0]) and torch.allclose(y[2], (h[1] + h[2]) / 2) and torch.allclose(y[3], (h[2] + h[3]) / 2)
    wide = dict(cfg, mask={"size": 3}, kv_from=0)
    y = P.attention(h, {k: v for k, v in w.items() if k in ("q", "q.norm", "o")}, "", wide, 1e-9, {}, st)
    assert torch.allclose(y[3], (h[1] + h[2] + h[3]) / 3)


@pytest.mark.parametrize("name", sorted(SOGUTAR))
def test_plain_whole_against_portions_and_single_tokens(name):
    cfg = SOGUTAR[name][0]
    w = {k: v.double() for k, v in make_tensors(cfg, 2, torch.float32).items()}
    ids = random_ids(45, cfg["vocab"], 7)
    want = P.forward(cfg, w, ids)
    m = P.Plain(cfg, w)
    got = torch.cat([m.run(ids[a:b]) for a, b in ((0, 1), (1, 3), (3, 20), (20, 21), (21, 45))])
    assert float((got - want).abs().max()) < 1e-9


# ---------------------------------------------------------------------------------------------- the engine's host side
@pytest.fixture(scope="module", params=["ga", "gc"])
def cpu_engine(request, tmp_path_factory):
    """The engine on the test double of the kernels: batch building, block tables (a window's pages given back while a borrower
    still reads), state slots, the wiring of the parts."""
    cfg, page = SOGUTAR[request.param]
    d = write_model(str(tmp_path_factory.mktemp("sogutar_" + request.param)), cfg, torch.float32, sharp=True)
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


def test_stream_after_every_layer_on_the_test_double(cpu_engine):
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
    assert [r for r, _ in got] == list(range(len(cfg["layers"]))) and len(want) == len(got)
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
    cfg.write_text(json.dumps(SOGUTAR_B))
    out = tmp_path / "model"
    r = run_cli("--random-weights", str(out), "--config", str(cfg), "--seed", "4", "--dtype", "bf16")
    assert r.returncode == 0, r.stderr
    arch, parsed = config_from_dir(str(out))
    assert arch.name == "Sogutar" and len(parsed.layers) == 5
