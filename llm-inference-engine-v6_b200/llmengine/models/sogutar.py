"""The Sogutar decoder ("architecture": "Sogutar") as a description in parts.

Tensors: `embed` [vocab, width] (also the output head), `embed.norm`, `final.norm`; per layer i `l<i>.norm1`; an attention
mixer's `l<i>.mix.{q, k, v, q.norm, k.norm, o}` (a layer that reads another layer's keys and values has only `q`, `q.norm`, `o`);
a retention mixer's `l<i>.mix.{q, k, v, g, o}`; a dense feed-forward's `l<i>.mlp.{gate, up, down}` or a routed one's
`l<i>.mlp.{router, correction, e<k>.gate, e<k>.up, e<k>.down, shared.gate, shared.up, shared.down, shared.sg}`.

The stream starts as the layer norm of the embedding row. A layer is a parallel block with ONE layer norm:
h += mixer(norm1(h)) + ff(norm1(h)). Logits come from the embedding table and are capped smoothly: c * tanh(logits / c).
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.sogutar import DenseFF, MoEFF, Rotation, SogutarConfig, sizes_from_tensors
from ..parts.spec import (BlockSpec, EmbeddingSpec, GatedAttentionSpec, GatedMLPSpec, GroupRoutedMLPSpec, HeadSpec, LayerRun, ModelSpec,
                          NormSpec, PositionSpec, RetentionSpec, ScaledRotarySpec)

SWISH_SLOPE = 1.702   # an expert's gate is g * sigmoid(1.702 g)
ROUTER_NORM_EPS = 1e-20  # added to the sum of the chosen scores before they are divided by it


def _position(cfg: SogutarConfig, rot: Rotation):
    """Rotation tables over the first rot.dims numbers of a head, frequencies base^(-2i/dims), stretched as the scaling says."""
    if rot is None or rot.dims == 0:
        return ScaledRotarySpec(kind="rope_ramp", dims=0, base=10000.0, max_positions=cfg.max_positions)  # nothing is rotated
    sc = rot.scaling
    if sc is None:
        return PositionSpec(kind="rope", head_dim=rot.dims, theta=rot.base, max_positions=cfg.max_positions, float64_frequencies=True)
    return PositionSpec(kind="rope", head_dim=rot.dims, theta=rot.base, max_positions=cfg.max_positions, scaling_factor=sc.factor,
                        low_freq_factor=sc.low, high_freq_factor=sc.high, original_max_positions=sc.original, float64_frequencies=True)


def kept_window(cfg: SogutarConfig, owner: int) -> int:
    """How many of the last keys layer `owner`'s cache must keep: the widest window among the layer itself and the layers that read
    its keys and values (0, everything, as soon as one of them has no window)."""
    windows = [cfg.layers[owner].mixer.window] + [l.mixer.window for l in cfg.layers if l.type == "attention" and l.mixer.kv_from == owner]
    return 0 if 0 in windows else max(windows)


def describe_sogutar(cfg: SogutarConfig) -> ModelSpec:
    layers, order = [], []

    def norm(name):
        return NormSpec("layernorm", cfg.width, cfg.eps, name)

    for i, l in enumerate(cfg.layers):
        p, m = f"l{i}.", l.mixer
        q = p + "mix."
        if l.type == "attention":
            own = m.kv_from is None
            mixer = GatedAttentionSpec(kind="gated_attention", hidden=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
                                       value_dim=m.vdim, scale=m.scale, eps=cfg.eps, position=_position(cfg, m.rot), q_weight=q + "q",
                                       k_weight=q + "k", v_weight=q + "v", o_weight=q + "o", q_norm=q + "q.norm",
                                       k_norm=q + "k.norm" if own else None, window=m.window, norm_scope="projection", own_kv=own,
                                       cache_window=kept_window(cfg, i) if own else None)
            order.append(LayerRun(i, cache_from=m.kv_from))  # every layer runs once, so a layer's index is its run's
        else:
            mixer = RetentionSpec(kind="retention", hidden=cfg.width, heads=m.heads, dim=m.dim, vdim=m.vdim, decay=tuple(m.decay),
                                  k_scale=m.dim ** -0.5, eps=cfg.eps, position=_position(cfg, m.rot), q_weight=q + "q", k_weight=q + "k",
                                  v_weight=q + "v", g_weight=q + "g", o_weight=q + "o")
            order.append(LayerRun(i))
        f, ff = l.mlp, None
        if isinstance(f, DenseFF):
            ff = GatedMLPSpec(kind="gated_mlp", hidden=cfg.width, intermediate=f.ff, gate_weight=p + "mlp.gate", up_weight=p + "mlp.up",
                              down_weight=p + "mlp.down", activation="silu")
        elif isinstance(f, MoEFF):
            shared = None
            if f.shared is not None:
                shared = GatedMLPSpec(kind="gated_mlp", hidden=cfg.width, intermediate=f.shared.ff, gate_weight=p + "mlp.shared.gate",
                                      up_weight=p + "mlp.shared.up", down_weight=p + "mlp.shared.down", activation="clamped_swish",
                                      limit=f.shared.limit, slope=SWISH_SLOPE)
            ff = GroupRoutedMLPSpec(kind="group_routed_mlp", hidden=cfg.width, intermediate=f.ff, experts=f.experts, top=f.top,
                                    router_weight=p + "mlp.router", correction=p + "mlp.correction",
                                    gate_weights=tuple(f"{p}mlp.e{k}.gate" for k in range(f.experts)),
                                    up_weights=tuple(f"{p}mlp.e{k}.up" for k in range(f.experts)),
                                    down_weights=tuple(f"{p}mlp.e{k}.down" for k in range(f.experts)),
                                    norm_eps=ROUTER_NORM_EPS, activation="clamped_swish", limit=f.limit, slope=SWISH_SLOPE, shared=shared,
                                    score="softmax", normalize=True, weight_scale=f.scale, identity=f.identity,
                                    shared_gate=p + "mlp.shared.sg" if shared is not None else None)
        layers.append(BlockSpec(kind="parallel", norm1=norm(p + "norm1"), mixer=mixer, norm2=None, feed_forward=ff))
    return ModelSpec(
        architecture=cfg.architecture,
        embedding=EmbeddingSpec("embed", cfg.vocab, cfg.width, kind="lookup_normed", norm=norm("embed.norm")),
        layers=tuple(layers),
        order=tuple(order),
        final_norm=norm("final.norm"),
        head=HeadSpec("embed", cfg.vocab, cfg.width, softcap=cfg.logit_softcap),
        max_positions=cfg.max_positions,
        eos_token_ids=cfg.eos_token_ids,
    )


SOGUTAR = Architecture(name="Sogutar", parse_config=SogutarConfig.from_dict, describe=describe_sogutar,
                       config_to_json=lambda cfg: cfg.to_dict(), sizes_from_tensors=sizes_from_tensors)
register_architecture(SOGUTAR, replace=True)
