"""Routed feed-forward (mixture of experts): every token goes through `top` of `experts` small feed-forward
layers, chosen by a linear router, and the results are added with the router's weights.

    z = Wr x + b  (float32);  chosen = the `top` largest z;  g = softmax(z[chosen])
    out = sum_e g_e * Wdown_e act(Wup_e x),  act = the exact (erf) gelu, no biases

The step's (token, choice) pairs are sorted by expert on the device into tiles of rows of one expert; the
per-expert products run over those tiles (all experts in one launch) and write each pair's row at the
pair's own index, so the weighted sum is a fixed-order sum over a token's `top` rows. All shapes depend on
the number of tokens alone: nothing is read back, and a decode step can be recorded as a CUDA graph.
"""
from __future__ import annotations

from typing import List

import torch

from .base import FeedForward, NormalizedRows
from .registry import build_part, part_class, register_part
from .spec import GroupRoutedMLPSpec, RoutedMLPSpec, TensorNeed


class RoutedMLP(FeedForward):
    def __init__(self, spec: RoutedMLPSpec, env):
        super().__init__(spec, env)
        if spec.activation != "gelu":
            raise ValueError(f"routed feed-forward: activation '{spec.activation}' is not implemented (gelu is)")
        if not (1 <= spec.top <= spec.experts):
            raise ValueError(f"routed feed-forward: cannot choose {spec.top} of {spec.experts} experts")
        if len(spec.up_weights) != spec.experts or len(spec.down_weights) != spec.experts:
            raise ValueError("routed feed-forward: one up and one down matrix per expert")
        self.router = self.bias = self.w_up = self.w_down = None

    @staticmethod
    def tensor_needs(spec: RoutedMLPSpec) -> List[TensorNeed]:
        out = [TensorNeed(spec.router_weight, (spec.experts, spec.hidden))]
        if spec.router_bias:
            out.append(TensorNeed(spec.router_bias, (spec.experts,), "float32", init="zeros"))
        for up, down in zip(spec.up_weights, spec.down_weights):
            out += [TensorNeed(up, (spec.intermediate, spec.hidden)), TensorNeed(down, (spec.hidden, spec.intermediate))]
        return out

    def kernel_notes(self):
        s = self.spec
        if self.env.dtype == torch.bfloat16 and (s.hidden % 8 or s.intermediate % 8):
            return [f"routed feed-forward: sizes {s.hidden} and {s.intermediate} are not both multiples of 8: the per-expert "
                    "products run on CUDA cores"]
        return []

    def load(self, tensors) -> None:
        s = self.spec
        self.router = tensors[s.router_weight]
        self.bias = tensors[s.router_bias] if s.router_bias else None
        self.w_up = torch.stack([tensors[n] for n in s.up_weights]).contiguous()      # [E, ff, hidden]
        self.w_down = torch.stack([tensors[n] for n in s.down_weights]).contiguous()  # [E, hidden, ff]

    def forward(self, x, ctx) -> torch.Tensor:
        s, ops, n, dt = self.spec, self.env.ops, ctx.n_tokens, self.env.dtype
        if isinstance(x, NormalizedRows):
            x = x.dense(ctx)
        x = x[:n]
        idx = ctx.ws.get("routed.idx", (n, s.top), torch.int32)
        share = ctx.ws.get("routed.share", (n, s.top), torch.float32)
        ops.route(x, self.router, self.bias, s.top, idx, share)
        tile = ops.routed_tile_rows(n, dt, (s.hidden, s.intermediate), n * s.top / s.experts)
        tile_expert, tile_rows = ops.routed_group(idx, s.experts, tile, ctx.ws, "routed")
        act = ctx.ws.get("routed.act", (n * s.top, s.intermediate), dt)
        ops.routed_product(x, s.top, self.w_up, tile_expert, tile_rows, act, "gelu")
        y = ctx.ws.get("routed.y", (n * s.top, s.hidden), torch.float32)
        ops.routed_product(act, 1, self.w_down, tile_expert, tile_rows, y, "share", share=share.view(-1))
        out = ctx.ws.get("routed.delta", (n, s.hidden), torch.float32)
        return ops.routed_combine(y, out, s.top)


class GroupRoutedMLP(FeedForward):
    """Gated experts chosen by scores over all experts, with a correction that only the choice sees and a limit on groups
    of experts (GroupRoutedMLPSpec), plus an optional expert that every token goes through:

        s = softmax(Wr x) or sigmoid(Wr x)  (float32);  choice = s + correction;  only the best `keep_groups` of `groups` groups stay
        (by their largest choice score, or by the sum of their two largest)
        chosen = the `top` largest choice scores;  g_e = s_e / (sum of the chosen s + norm_eps) * weight_scale
        out = sum_e g_e * Wdown_e (act(Wgate_e x, Wup_e x))  +  [sigmoid(w_sg . x) *] shared(x)

    act is silu(gate) * up, or the clamped form (min(gate, L), clamp(up, -L, L), gate * sigmoid(slope * gate) * (up + 1)). With
    `identity` > 0 the router has that many more outputs behind the experts' whose "expert" returns x itself: they take part in
    scores and choice like the others, get no tiles in the per-expert products, and are added where the chosen rows are summed.

    An expert's gate and up rows are stored in turn ([E, 2 ff, hidden]: row 2 f the gate, row 2 f + 1 its up row), so that the
    per-expert product has both in one thread's hands and applies silu(gate) * up in its epilogue. Where the caller says that
    it takes pairs (ctx.takes_delta_pairs: a block that adds two sets of sums in one kernel), the routed sum and the shared
    expert's partial sums are returned side by side; otherwise they are added here."""

    def __init__(self, spec: GroupRoutedMLPSpec, env):
        super().__init__(spec, env)
        if spec.activation not in ("silu", "clamped_swish") or (spec.activation == "clamped_swish" and not spec.limit > 0):
            raise ValueError(f"routed gated feed-forward: activation '{spec.activation}' is not implemented (silu and clamped_swish with a positive limit are)")
        self.act = (spec.activation, float(spec.limit), float(spec.slope)) if spec.activation == "clamped_swish" else spec.activation
        if spec.identity < 0 or (spec.shared_gate and spec.shared is None):
            raise ValueError("routed feed-forward: identity experts cannot be negative, and a gate on the shared expert needs one")
        self.outputs = spec.experts + spec.identity  # what the router scores and chooses among
        if not (1 <= spec.top <= self.outputs):
            raise ValueError(f"routed feed-forward: cannot choose {spec.top} of {self.outputs} experts")
        if spec.groups < 1 or self.outputs % spec.groups or not (1 <= spec.keep_groups <= spec.groups):
            raise ValueError(f"routed feed-forward: {self.outputs} experts do not form {spec.groups} equal groups of which {spec.keep_groups} stay")
        if spec.score not in ("softmax", "sigmoid") or spec.group_top not in (1, 2):
            raise ValueError("routed feed-forward: score is 'softmax' or 'sigmoid', a group's score sums its 1 or 2 largest")
        if spec.keep_groups * (self.outputs // spec.groups) < spec.top:
            raise ValueError("routed feed-forward: the groups that stay hold fewer experts than a token uses")
        if not (len(spec.gate_weights) == len(spec.up_weights) == len(spec.down_weights) == spec.experts):
            raise ValueError("routed feed-forward: one gate, one up and one down matrix per expert")
        self.shared = build_part("feed_forward", spec.shared, env) if spec.shared is not None else None
        self.router = self.correction = self.w_gate_up = self.w_down = None

    @staticmethod
    def tensor_needs(spec: GroupRoutedMLPSpec) -> List[TensorNeed]:
        outputs = spec.experts + spec.identity
        out = [TensorNeed(spec.router_weight, (outputs, spec.hidden))]
        if spec.correction:
            out.append(TensorNeed(spec.correction, (outputs,), "float32", init="zeros"))
        if spec.shared_gate:
            out.append(TensorNeed(spec.shared_gate, (1, spec.hidden)))
        for g, u, d in zip(spec.gate_weights, spec.up_weights, spec.down_weights):
            out += [TensorNeed(g, (spec.intermediate, spec.hidden)), TensorNeed(u, (spec.intermediate, spec.hidden)),
                    TensorNeed(d, (spec.hidden, spec.intermediate))]
        if spec.shared is not None:
            out += part_class("feed_forward", spec.shared.kind).tensor_needs(spec.shared)
        return out

    def subparts(self):
        return (self.shared,) if self.shared is not None else ()

    def kernel_notes(self):
        s = self.spec
        if self.env.dtype == torch.bfloat16 and (s.hidden % 8 or s.intermediate % 8):
            return [f"routed feed-forward: sizes {s.hidden} and {s.intermediate} are not both multiples of 8: the per-expert "
                    "products run on CUDA cores"]
        return []

    def load(self, tensors) -> None:
        s = self.spec
        self.router = tensors[s.router_weight]
        if s.shared_gate:  # the shared expert's gate is one more row behind the router's: the routing kernel forms both in float32
            self.router = torch.cat([self.router, tensors[s.shared_gate].reshape(1, s.hidden)], dim=0).contiguous()
        self.correction = tensors[s.correction] if s.correction else None
        gu = [torch.stack([tensors[g], tensors[u]], dim=1).reshape(2 * s.intermediate, s.hidden) for g, u in zip(s.gate_weights, s.up_weights)]
        self.w_gate_up = torch.stack(gu).contiguous()                                  # [E, 2 ff, hidden], gate and up rows in turn
        self.w_down = torch.stack([tensors[n] for n in s.down_weights]).contiguous()  # [E, hidden, ff]
        if self.shared is not None:
            self.shared.load(tensors)

    def forward(self, x, ctx) -> torch.Tensor:
        s, ops, n, dt = self.spec, self.env.ops, ctx.n_tokens, self.env.dtype
        if isinstance(x, NormalizedRows):
            x = x.dense(ctx)
        x = x[:n]
        idx = ctx.ws.get("routed.idx", (n, s.top), torch.int32)
        share = ctx.ws.get("routed.share", (n, s.top), torch.float32)
        extra = {}
        if (s.score, s.group_top, s.normalize) != ("softmax", 1, True):
            extra.update(score=s.score, group_top=s.group_top, normalize=s.normalize)
        gate = None
        if s.weight_scale != 1.0:
            extra["weight_scale"] = float(s.weight_scale)
        if s.shared_gate:
            gate = extra["gate_out"] = ctx.ws.get("routed.shared_gate", (n,), torch.float32)
        ops.route_grouped(x, self.router, self.correction, s.top, s.groups, s.keep_groups, s.norm_eps, idx, share, **extra)
        tile = ops.routed_tile_rows(n, dt, (s.hidden, s.intermediate), n * s.top / s.experts)
        if s.identity:
            tile_expert, tile_rows = ops.routed_group(idx, self.outputs, tile, ctx.ws, "routed", real_experts=s.experts)
        else:
            tile_expert, tile_rows = ops.routed_group(idx, s.experts, tile, ctx.ws, "routed")
        act = ctx.ws.get("routed.act", (n * s.top, s.intermediate), dt)
        if s.activation == "silu":
            ops.routed_product(x, s.top, self.w_gate_up, tile_expert, tile_rows, act, "silu_pairs")
        else:
            ops.routed_product(x, s.top, self.w_gate_up, tile_expert, tile_rows, act, "gated_pairs", act=self.act)
        y = ctx.ws.get("routed.y", (n * s.top, s.hidden), torch.float32)
        ops.routed_product(act, 1, self.w_down, tile_expert, tile_rows, y, "share", share=share.view(-1))
        identity = (idx, share, s.experts, x) if s.identity else None
        out = ctx.ws.get("routed.delta", (n, s.hidden), torch.float32)
        if self.shared is None:
            return ops.routed_combine(y, out, s.top, identity=identity) if identity else ops.routed_combine(y, out, s.top)
        # the shared expert's last product, as it comes (it works for no stream here: its sums are added to the routed sum)
        keep = ctx.residual
        ctx.residual = None
        b = self.shared.forward(x, ctx)
        ctx.residual = keep
        if gate is not None or identity is not None:
            # one kernel adds the chosen rows, the identity experts' shares of x and the shared expert's sums times its gate
            return ops.routed_combine(y, out, s.top, identity=identity, extra=b, extra_gate=gate)
        ops.routed_combine(y, out, s.top)
        if getattr(ctx, "takes_delta_pairs", False):
            return out, b  # the caller adds the two sets of sums itself, in this order
        return ops.stream_add(out, b, n_rows=n)


register_part("feed_forward", "routed_mlp", RoutedMLP)
register_part("feed_forward", "group_routed_mlp", GroupRoutedMLP)
