"""The Selinex decoder ("architecture": "Selinex") as a description in parts.

Tensors: `embed` [vocab, width] (also the output head), `final.norm`; per layer i `l<i>.norm1`, `l<i>.norm1b` and, with a
feed-forward, `l<i>.norm2`, `l<i>.norm2b`; a pair of mixers' `l<i>.mix.left.{q, k, v, o}` (attention; `g` where the heads'
results are gated) beside `l<i>.mix.right.{q, k, v, g, o, norm, a1, a2, a2.b}` (decay per key channel) or
`l<i>.mix.right.{mu.r, mu.k, mu.v, mu.g, mu.w, r, k, v, g, w1, w2, w0, u, norm, o}` with `l<i>.mix.left.out`, `l<i>.mix.right.out`
(token shift); a delta mixer's `l<i>.mix.{q, k, v, q.conv, k.conv, v.conv, b, a, A_log, dt_bias, g, norm, o}`; a dense
feed-forward's `l<i>.mlp.{gate, up, down}` or a routed one's `l<i>.mlp.{router, correction, e<k>.gate, e<k>.up, e<k>.down}`.

A layer is a sandwich block: h += m * norm1b(mixer(norm1(h))); h += m * norm2b(ff(norm2(h))), every norm with the weight
1 + w. A loop in the configuration repeats a range of layers with the same weights; every repetition is a run of its own in
the layer order, so it owns its cache and state.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.selinex import DenseFF, MoEFF, SelinexConfig, sizes_from_tensors
from ..parts.spec import (BlockSpec, DecayedLinearAttentionSpec, EmbeddingSpec, GatedAttentionSpec, GatedDeltaSpec, GatedMLPSpec,
                          GroupRoutedMLPSpec, HeadSpec, LayerRun, MixerPairSpec, ModelSpec, NormSpec, ScaledRotarySpec, TokenShiftMixSpec)

SWISH_SLOPE = 1.702  # the dense feed-forward's gate is g * sigmoid(1.702 g)
UNIT_EPS = 1e-6      # under the root when the delta rule's queries and keys are made unit vectors


def layer_order(cfg: SelinexConfig):
    L = len(cfg.layers)
    if cfg.loop is None:
        return tuple(LayerRun(i) for i in range(L))
    lp = cfg.loop
    order = [LayerRun(i) for i in range(lp.start)]
    for _ in range(lp.times):
        order += [LayerRun(i) for i in range(lp.start, lp.stop)]
    return tuple(order + [LayerRun(i) for i in range(lp.stop, L)])


def _attention(cfg: SelinexConfig, a, p: str, gated: bool) -> GatedAttentionSpec:
    position = ScaledRotarySpec(kind="rope_ramp", dims=a.rot_dims, base=a.rot_base, max_positions=cfg.max_positions)
    return GatedAttentionSpec(kind="gated_attention", hidden=cfg.width, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim,
                              value_dim=a.vdim, scale=a.scale, eps=cfg.eps, position=position, q_weight=p + "q", k_weight=p + "k",
                              v_weight=p + "v", o_weight=p + "o", gate_weight=p + "g" if gated else None, gate_per_head=gated,
                              window=a.window)


def describe_selinex(cfg: SelinexConfig) -> ModelSpec:
    layers, ignore = [], []

    def norm(name):
        return NormSpec("rmsnorm_unit_offset", cfg.width, cfg.eps, name)

    for i, l in enumerate(cfg.layers):
        p, m = f"l{i}.", l.mixer
        q = p + "mix."
        if l.type == "delta":
            mixer = GatedDeltaSpec(kind="gated_delta", hidden=cfg.width, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                                   taps=m.taps, eps=cfg.eps, q_weight=q + "q", k_weight=q + "k", v_weight=q + "v", q_conv=q + "q.conv",
                                   k_conv=q + "k.conv", v_conv=q + "v.conv", b_weight=q + "b", a_weight=q + "a", a_log=q + "A_log",
                                   dt_bias=q + "dt_bias", g_weight=q + "g", norm_weight=q + "norm", o_weight=q + "o", unit_eps=UNIT_EPS)
        elif l.type == "parallel":
            r, rp = m.right, q + "right."
            right = DecayedLinearAttentionSpec(kind="decayed_linear_attention", hidden=cfg.width, heads=r.heads, dim=r.dim, vdim=r.vdim,
                                               rank=r.rank, tau=r.tau, eps=cfg.eps, q_weight=rp + "q", k_weight=rp + "k", v_weight=rp + "v",
                                               g_weight=rp + "g", o_weight=rp + "o", norm_weight=rp + "norm", a1_weight=rp + "a1",
                                               a2_weight=rp + "a2", a2_bias=rp + "a2.b")
            mixer = MixerPairSpec(kind="mixer_pair", hidden=cfg.width, left=_attention(cfg, m.left, q + "left.", True), right=right,
                                  combine="weighted", left_scale=m.left_scale, right_scale=m.right_scale)
        else:
            r, rp = m.right, q + "right."
            right = TokenShiftMixSpec(kind="token_shift_mix", hidden=cfg.width, heads=r.heads, dim=r.dim, rank=r.rank, eps=cfg.eps,
                                      mu=tuple(rp + "mu." + s for s in "rkvgw"), r_weight=rp + "r", k_weight=rp + "k", v_weight=rp + "v",
                                      g_weight=rp + "g", o_weight=rp + "o", w1_weight=rp + "w1", w2_weight=rp + "w2", w0=rp + "w0",
                                      bonus=rp + "u", norm_weight=rp + "norm")
            mixer = MixerPairSpec(kind="mixer_pair", hidden=cfg.width, left=_attention(cfg, m.left, q + "left.", False), right=right,
                                  combine="normed_mean", left_norm=q + "left.out", right_norm=q + "right.out", eps=cfg.eps)
        ff = norm2 = norm2_out = None
        f = l.mlp
        if f is None:
            ignore += [p + "norm2", p + "norm2b"]  # a layer without a feed-forward has no use for them
        else:
            norm2, norm2_out = norm(p + "norm2"), norm(p + "norm2b")
            if isinstance(f, DenseFF):
                ff = GatedMLPSpec(kind="gated_mlp", hidden=cfg.width, intermediate=f.ff, gate_weight=p + "mlp.gate", up_weight=p + "mlp.up",
                                  down_weight=p + "mlp.down", activation="clamped_swish", limit=f.limit, slope=SWISH_SLOPE)
            else:
                assert isinstance(f, MoEFF)
                ff = GroupRoutedMLPSpec(kind="group_routed_mlp", hidden=cfg.width, intermediate=f.ff, experts=f.experts, top=f.top,
                                        router_weight=p + "mlp.router", correction=p + "mlp.correction",
                                        gate_weights=tuple(f"{p}mlp.e{k}.gate" for k in range(f.experts)),
                                        up_weights=tuple(f"{p}mlp.e{k}.up" for k in range(f.experts)),
                                        down_weights=tuple(f"{p}mlp.e{k}.down" for k in range(f.experts)),
                                        groups=f.groups, keep_groups=f.keep, activation="silu", score="sigmoid", group_top=2, normalize=False)
        layers.append(BlockSpec(kind="sandwich", norm1=norm(p + "norm1"), mixer=mixer, norm2=norm2, feed_forward=ff,
                                norm1_out=norm(p + "norm1b"), norm2_out=norm2_out, residual_mult=cfg.residual_mult))
    return ModelSpec(
        architecture=cfg.architecture,
        embedding=EmbeddingSpec("embed", cfg.vocab, cfg.width),
        layers=tuple(layers),
        order=layer_order(cfg),
        final_norm=norm("final.norm"),
        head=HeadSpec("embed", cfg.vocab, cfg.width),
        max_positions=cfg.max_positions,
        eos_token_ids=cfg.eos_token_ids,
        ignore=tuple(ignore),
    )


SELINEX = Architecture(name="Selinex", parse_config=SelinexConfig.from_dict, describe=describe_selinex,
                       config_to_json=lambda cfg: cfg.to_dict(), sizes_from_tensors=sizes_from_tensors)
register_architecture(SELINEX, replace=True)
