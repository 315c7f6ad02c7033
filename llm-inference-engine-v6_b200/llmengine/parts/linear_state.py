"""Recurrent mixers whose memory is a matrix per head, S [dk, dv] in float32, kept in the request's state slot and updated token
after token by a rank-one write k v^T (ops.linear_state). Four of them, which differ in what decays the matrix, what is
written, and what the projections read:

    Retention                q, k, v, g = W h;  q and k rotated at the token's position, k times a constant;  one decay a head
                             that is a constant of the model:  S <- decay_h S + k v^T;  o = S^T q;  no weight on the heads' norm
    DecayedLinearAttention   q, k, v, g = W h;  a = sigmoid(W_a2 (W_a1 h) + b)^(1/tau) per key channel
                             S <- diag(a) S + k v^T;  o = S^T (q dk^-1/2)
    TokenShiftMix            every projection reads its own blend h + (h_prev - h) * mu of the token's input with the previous
                             token's (kept in the slot); decay = exp(-exp(W_w2 tanh(W_w1 x_w) + w0)) per key channel
                             o = (S + diag(bonus) k v^T)^T r;  S <- diag(decay) S + k v^T
    GatedDelta               q, k, v behind a short causal convolution and silu (its last inputs kept in the slot), q and k unit
                             vectors per head; g, beta per head;  S <- g S;  w = beta (v - S^T k);  S <- S + k w^T;  o = S^T q

All of them finish alike: every head's o divided by its root mean square, times a weight, times silu of a gate projection, then
the output projection. Decays, gates, unit norms, the state and o are float32 in both engine precisions; the projections'
float32 sums are read as they come (K-split parts are added where they are read).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .attention import add_into_stream_or_partials, project_sums
from .base import LayerCache, Mixer, NormalizedRows, StateNeed
from .registry import build_part, part_class, register_part
from .spec import DecayedLinearAttentionSpec, GatedDeltaSpec, RetentionSpec, TensorNeed, TokenShiftMixSpec


def _state_shape(env, heads: int, dk: int, dv: int):
    return tuple(env.ops.linear_state_shape(heads, dk, dv))


class DecayedLinearAttention(Mixer):
    def __init__(self, spec: DecayedLinearAttentionSpec, env):
        super().__init__(spec, env)
        if min(spec.heads, spec.dim, spec.vdim, spec.rank) <= 0 or not spec.tau > 0:
            raise ValueError("decayed linear attention: sizes and tau must be positive")
        self.w_in = self.w_a1 = self.w_a2_t = self.a2_bias = self.norm_w = self.w_o = None

    @staticmethod
    def tensor_needs(spec: DecayedLinearAttentionSpec) -> List[TensorNeed]:
        H, dk, dv, D, R = spec.heads, spec.dim, spec.vdim, spec.hidden, spec.rank
        return [TensorNeed(spec.q_weight, (H * dk, D)), TensorNeed(spec.k_weight, (H * dk, D)), TensorNeed(spec.v_weight, (H * dv, D)),
                TensorNeed(spec.g_weight, (H * dv, D)), TensorNeed(spec.o_weight, (D, H * dv)),
                TensorNeed(spec.norm_weight, (dv,), "float32", init="around_one"), TensorNeed(spec.a1_weight, (R, D)),
                TensorNeed(spec.a2_weight, (H * dk, R)), TensorNeed(spec.a2_bias, (H * dk,), "float32")]

    def cache_needs(self):
        s = self.spec
        return (StateNeed("decayed_linear.state", _state_shape(self.env, s.heads, s.dim, s.vdim)),)

    def load(self, tensors) -> None:
        s = self.spec
        self.w_in = torch.cat([tensors[s.q_weight], tensors[s.k_weight], tensors[s.v_weight], tensors[s.g_weight]], dim=0).contiguous()
        self.w_a1 = tensors[s.a1_weight]
        self.w_a2_t = tensors[s.a2_weight].t().contiguous()  # [rank, channels]: neighbouring channels read neighbouring words
        self.a2_bias, self.norm_w, self.w_o = tensors[s.a2_bias], tensors[s.norm_weight], tensors[s.o_weight]

    def forward(self, x, ctx, cache: LayerCache) -> Optional[torch.Tensor]:
        s, ops, n, dt = self.spec, self.env.ops, ctx.n_tokens, self.env.dtype
        if isinstance(x, NormalizedRows):
            x = x.dense(ctx)
        H, dk, dv = s.heads, s.dim, s.vdim
        sums = project_sums(ops, ctx, x, self.w_in, "decayed_linear.in")
        low = ctx.ws.get("decayed_linear.low", (n, s.rank), torch.float32)
        ops.gemm(x[:n], self.w_a1, low, ctx.ws)
        decay = ctx.ws.get("decayed_linear.decay", (n, H * dk), torch.float32)
        ops.lowrank_map(low, s.rank, self.w_a2_t, self.a2_bias, decay, n, None, "sigmoid_root", s.tau)
        o = ctx.ws.get("decayed_linear.o", (n, H * dv), torch.float32)
        ops.linear_state("decay_write_read", sums, 0, sums, H * dk, sums, 2 * H * dk, decay, 0, None, cache.states["decayed_linear.state"],
                         ctx, o, H, H, dk, dv, q_scale=dk ** -0.5)
        y = ctx.ws.get("decayed_linear.y", (n, H * dv), dt)
        ops.head_norm_gate(o, self.norm_w, sums, 2 * H * dk + H * dv, s.eps, y, n, H, dv)
        return add_into_stream_or_partials(ops, y, self.w_o, ctx, False, "decayed_linear.delta")


class Retention(Mixer):
    """Linear attention with a fixed decay per head (RetentionSpec). The projections' float32 sums are rotated in float32
    (ops.rotate_sums, which also applies the keys' constant), the state walks the tokens under the rule "decay_write_read" with
    one constant row of decays, and head_norm_gate divides by the heads' root mean squares and applies silu(Wg h)."""

    def __init__(self, spec: RetentionSpec, env):
        super().__init__(spec, env)
        if min(spec.heads, spec.dim, spec.vdim) <= 0 or len(spec.decay) != spec.heads:
            raise ValueError("retention: sizes must be positive, and there is one decay a head")
        self.position = build_part("position", spec.position, env)
        tables = self.position.rotation_tables()
        if tables is None:
            raise ValueError("retention needs a position encoding with rotation tables")
        self.cos, self.sin = tables
        if self.cos is not None and 2 * self.cos.shape[1] > spec.dim:
            raise ValueError(f"retention: {2 * self.cos.shape[1]} rotated dimensions do not fit a head of {spec.dim}")
        self.w_in = self.w_o = self.decay = self.ones = None

    @staticmethod
    def tensor_needs(spec: RetentionSpec) -> List[TensorNeed]:
        H, dk, dv, D = spec.heads, spec.dim, spec.vdim, spec.hidden
        return [TensorNeed(spec.q_weight, (H * dk, D)), TensorNeed(spec.k_weight, (H * dk, D)), TensorNeed(spec.v_weight, (H * dv, D)),
                TensorNeed(spec.g_weight, (H * dv, D)), TensorNeed(spec.o_weight, (D, H * dv))] + \
            list(part_class("position", spec.position.kind).tensor_needs(spec.position))

    def subparts(self):
        return (self.position,)

    def cache_needs(self):
        s = self.spec
        return (StateNeed("retention.state", _state_shape(self.env, s.heads, s.dim, s.vdim)),)

    def load(self, tensors) -> None:
        s, dev = self.spec, self.env.device
        self.w_in = torch.cat([tensors[s.q_weight], tensors[s.k_weight], tensors[s.v_weight], tensors[s.g_weight]], dim=0).contiguous()
        self.w_o = tensors[s.o_weight]
        # the decays as the kernel reads them: a number a (head, key channel), one row for all tokens; float32 from the configuration's doubles
        self.decay = torch.tensor(s.decay, dtype=torch.float64).to(torch.float32).repeat_interleave(s.dim).reshape(1, s.heads * s.dim).contiguous().to(dev)
        self.ones = torch.ones(s.vdim, dtype=torch.float32, device=dev)
        self.position.load(tensors)

    def forward(self, x, ctx, cache: LayerCache) -> Optional[torch.Tensor]:
        s, ops, n, dt = self.spec, self.env.ops, ctx.n_tokens, self.env.dtype
        if isinstance(x, NormalizedRows):
            x = x.dense(ctx)
        H, dk, dv = s.heads, s.dim, s.vdim
        sums = project_sums(ops, ctx, x, self.w_in, "retention.in")  # [q | k | v | g], float32, never rounded
        qk = ctx.ws.get("retention.qk", (n, 2 * H * dk), torch.float32)
        ops.rotate_sums(sums, 0, 2 * H, dk, self.cos, self.sin, ctx.positions, qk, n, scaled_from=H, scale=float(s.k_scale))
        o = ctx.ws.get("retention.o", (n, H * dv), torch.float32)
        ops.linear_state("decay_write_read", qk, 0, qk, H * dk, sums, 2 * H * dk, self.decay, 0, None, cache.states["retention.state"], ctx, o,
                         H, H, dk, dv, decay_const=True)
        y = ctx.ws.get("retention.y", (n, H * dv), dt)
        ops.head_norm_gate(o, self.ones, sums, 2 * H * dk + H * dv, s.eps, y, n, H, dv)
        return add_into_stream_or_partials(ops, y, self.w_o, ctx, False, "retention.delta")


class TokenShiftMix(Mixer):
    BLENDS = 5  # r, k, v, g, w

    def __init__(self, spec: TokenShiftMixSpec, env):
        super().__init__(spec, env)
        if min(spec.heads, spec.dim, spec.rank) <= 0 or len(spec.mu) != self.BLENDS:
            raise ValueError("token-shift mixer: sizes must be positive, and there are five blends (r, k, v, g, w)")
        self.mu = self.w_r = self.w_k = self.w_v = self.w_g = self.w_w1 = self.w_w2_t = self.w0 = self.bonus = self.norm_w = self.w_o = None

    @staticmethod
    def tensor_needs(spec: TokenShiftMixSpec) -> List[TensorNeed]:
        H, dk, D, R = spec.heads, spec.dim, spec.hidden, spec.rank
        out = [TensorNeed(name, (D,), "float32") for name in spec.mu]
        out += [TensorNeed(name, (H * dk, D)) for name in (spec.r_weight, spec.k_weight, spec.v_weight, spec.g_weight)]
        return out + [TensorNeed(spec.o_weight, (D, H * dk)), TensorNeed(spec.w1_weight, (R, D)), TensorNeed(spec.w2_weight, (H * dk, R)),
                      TensorNeed(spec.w0, (H * dk,), "float32"), TensorNeed(spec.bonus, (H, dk), "float32"),
                      TensorNeed(spec.norm_weight, (H * dk,), "float32", init="around_one")]

    def cache_needs(self):
        s = self.spec
        return (StateNeed("token_shift.state", _state_shape(self.env, s.heads, s.dim, s.dim)), StateNeed("token_shift.previous", (s.hidden,)))

    def load(self, tensors) -> None:
        s = self.spec
        self.mu = torch.stack([tensors[name] for name in s.mu]).contiguous()
        self.w_r, self.w_k, self.w_v, self.w_g = tensors[s.r_weight], tensors[s.k_weight], tensors[s.v_weight], tensors[s.g_weight]
        self.w_w1 = tensors[s.w1_weight]
        self.w_w2_t = tensors[s.w2_weight].t().contiguous()
        self.w0, self.bonus, self.norm_w, self.w_o = tensors[s.w0], tensors[s.bonus].contiguous(), tensors[s.norm_weight], tensors[s.o_weight]

    def forward(self, x, ctx, cache: LayerCache) -> Optional[torch.Tensor]:
        s, ops, n, dt = self.spec, self.env.ops, ctx.n_tokens, self.env.dtype
        if isinstance(x, NormalizedRows):
            x = x.dense(ctx)
        H, dk = s.heads, s.dim
        blends = ctx.ws.get("token_shift.blends", (self.BLENDS, n, s.hidden), dt)
        ops.token_shift(x[:n], self.mu, cache.states["token_shift.previous"], ctx, blends)
        r = project_sums(ops, ctx, blends[0], self.w_r, "token_shift.r")
        k = project_sums(ops, ctx, blends[1], self.w_k, "token_shift.k")
        v = project_sums(ops, ctx, blends[2], self.w_v, "token_shift.v")
        g = project_sums(ops, ctx, blends[3], self.w_g, "token_shift.g")
        low = ctx.ws.get("token_shift.low", (n, s.rank), torch.float32)
        ops.gemm(blends[4], self.w_w1, low, ctx.ws)
        decay = ctx.ws.get("token_shift.decay", (n, H * dk), torch.float32)
        ops.lowrank_map(low, s.rank, self.w_w2_t, self.w0, decay, n, "tanh", "exp_neg_exp")
        o = ctx.ws.get("token_shift.o", (n, H * dk), torch.float32)
        ops.linear_state("bonus_read_decay_write", r, 0, k, 0, v, 0, decay, 0, self.bonus, cache.states["token_shift.state"], ctx, o,
                         H, H, dk, dk)
        y = ctx.ws.get("token_shift.y", (n, H * dk), dt)
        ops.head_norm_gate(o, self.norm_w, g, 0, s.eps, y, n, H, dk)
        return add_into_stream_or_partials(ops, y, self.w_o, ctx, False, "token_shift.delta")


class GatedDelta(Mixer):
    def __init__(self, spec: GatedDeltaSpec, env):
        super().__init__(spec, env)
        if min(spec.heads, spec.kv_heads, spec.dim, spec.vdim, spec.taps) <= 0 or spec.heads % spec.kv_heads:
            raise ValueError("gated delta rule: sizes must be positive and heads a multiple of kv_heads")
        self.w_in = self.w_conv = self.a_log = self.dt_bias = self.norm_w = self.w_o = None

    @staticmethod
    def tensor_needs(spec: GatedDeltaSpec) -> List[TensorNeed]:
        H, G, dk, dv, D, K = spec.heads, spec.kv_heads, spec.dim, spec.vdim, spec.hidden, spec.taps
        return [TensorNeed(spec.q_weight, (G * dk, D)), TensorNeed(spec.k_weight, (G * dk, D)), TensorNeed(spec.v_weight, (H * dv, D)),
                TensorNeed(spec.q_conv, (G * dk, K), "float32"), TensorNeed(spec.k_conv, (G * dk, K), "float32"),
                TensorNeed(spec.v_conv, (H * dv, K), "float32"), TensorNeed(spec.b_weight, (H, D)), TensorNeed(spec.a_weight, (H, D)),
                TensorNeed(spec.a_log, (H,), "float32"), TensorNeed(spec.dt_bias, (H,), "float32"), TensorNeed(spec.g_weight, (H * dv, D)),
                TensorNeed(spec.norm_weight, (dv,), "float32", init="around_one"), TensorNeed(spec.o_weight, (D, H * dv))]

    def cache_needs(self):
        s = self.spec
        channels = 2 * s.kv_heads * s.dim + s.heads * s.vdim
        return (StateNeed("delta.state", _state_shape(self.env, s.heads, s.dim, s.vdim)), StateNeed("delta.conv", (s.taps - 1, channels)))

    def load(self, tensors) -> None:
        s = self.spec
        # one product for everything that reads the mixer's input: [q | k | v | g | a | b]
        self.w_in = torch.cat([tensors[n] for n in (s.q_weight, s.k_weight, s.v_weight, s.g_weight, s.a_weight, s.b_weight)], dim=0).contiguous()
        self.w_conv = torch.cat([tensors[s.q_conv], tensors[s.k_conv], tensors[s.v_conv]], dim=0).contiguous()  # float32 [channels, taps]
        self.a_log, self.dt_bias, self.norm_w, self.w_o = tensors[s.a_log], tensors[s.dt_bias], tensors[s.norm_weight], tensors[s.o_weight]

    def forward(self, x, ctx, cache: LayerCache) -> Optional[torch.Tensor]:
        s, ops, n, dt = self.spec, self.env.ops, ctx.n_tokens, self.env.dtype
        if isinstance(x, NormalizedRows):
            x = x.dense(ctx)
        H, G, dk, dv = s.heads, s.kv_heads, s.dim, s.vdim
        C = 2 * G * dk + H * dv
        g_off, a_off, b_off = C, C + H * dv, C + H * dv + H
        sums = project_sums(ops, ctx, x, self.w_in, "delta.in")
        qkv = ctx.ws.get("delta.conv_out", (n, C), torch.float32)  # float32: what follows (unit norms, the recurrence) is
        ops.conv_silu(sums, 0, C, self.w_conv, None, cache.states["delta.conv"], ctx, qkv)
        gates = ctx.ws.get("delta.gates", (n, 2 * H), torch.float32)
        ops.delta_gates(sums, a_off, sums, b_off, self.a_log, self.dt_bias, gates, n)
        o = ctx.ws.get("delta.o", (n, H * dv), torch.float32)
        ops.linear_state("delta", qkv, 0, qkv, G * dk, qkv, 2 * G * dk, gates, 0, None, cache.states["delta.state"], ctx, o, H, G, dk, dv,
                         q_scale=dk ** -0.5, unit_eps=s.unit_eps)
        y = ctx.ws.get("delta.y", (n, H * dv), dt)
        ops.head_norm_gate(o, self.norm_w, sums, g_off, s.eps, y, n, H, dv)
        return add_into_stream_or_partials(ops, y, self.w_o, ctx, False, "delta.delta")


register_part("mixer", "retention", Retention)
register_part("mixer", "decayed_linear_attention", DecayedLinearAttention)
register_part("mixer", "token_shift_mix", TokenShiftMix)
register_part("mixer", "gated_delta", GatedDelta)
