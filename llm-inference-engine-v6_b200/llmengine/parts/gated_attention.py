"""Gated attention: causal grouped-query softmax attention over the paged cache with keys and values of different sizes
and a set of options that a model description switches on one by one (GatedAttentionSpec).

With h the mixer's input, per token at position p:
    q = Wq h, k = Wk h, v = Wv h, g = Wg h                      (one product against [Wq; Wk; Wv; Wg], float32 sums)
    q_a <- rot_p(rmsnorm(q_a) * wq),  k_b <- rot_p(rmsnorm(k_b) * wk)   per head, one norm weight for all heads
    v <- (1 - m) v + m v_first                                  (value mixing; the mixed v is what the cache holds)
    score_a(i, j) = (q_a(i) . k_b(j)) * scale,  b = a // (H / G),  j <= i in the same chunk (and inside the window)
    p_a(i, j) = exp(score) / (sum_j exp(score) + exp(sink_a))   the sink only enlarges the denominator
    out = Wo ((heads' results side by side) * sigmoid(g))       g: a gate a number of the result, or (gate_per_head) one a head
With norm_scope "projection" the two norms are over all of q and all of k at once (weights of the projections' sizes). A layer
without keys and values of its own (own_kv False) forms queries only and reads the cache of the run its LayerRun names.
Norms, rotation, scores, softmax and the gate are float32 in both engine precisions. v_first are the values that the
first layer with value mixing computed for the same tokens in the same step: that layer leaves them in the step
context (`ctx.shared`), the later ones read them there.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .attention import add_into_stream_or_partials
from .base import KVNeed, LayerCache, Mixer, NormalizedRows
from .registry import build_part, part_class, register_part
from .spec import GatedAttentionSpec, TensorNeed

V_FIRST = "gated_attention.v_first"  # key of ctx.shared


class GatedAttention(Mixer):
    def __init__(self, spec: GatedAttentionSpec, env):
        super().__init__(spec, env)
        for name in ("num_heads", "num_kv_heads", "head_dim", "value_dim"):
            if getattr(spec, name) <= 0:
                raise ValueError(f"gated attention: {name} must be >= 1")
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"gated attention: {spec.num_heads} heads cannot share {spec.num_kv_heads} key/value heads")
        if spec.window < 0 or spec.chunk < 0:
            raise ValueError("gated attention: window and chunk must be >= 0")
        if spec.norm_scope not in ("head", "projection"):
            raise ValueError("gated attention: norm_scope is 'head' or 'projection'")
        if not spec.own_kv and (spec.value_mix is not None or spec.k_norm):
            raise ValueError("gated attention: a layer that borrows keys and values has no key norm and mixes no values")
        if spec.value_mix not in (None, "first", "mix") or (spec.value_mix == "mix" and not spec.value_mix_weight):
            raise ValueError("gated attention: value_mix is None, 'first' or 'mix' (with the name of its weight)")
        self.position = build_part("position", spec.position, env)
        tables = self.position.rotation_tables()
        if tables is None:
            raise ValueError("gated attention needs a position encoding with rotation tables")
        self.cos, self.sin = tables
        if self.cos is not None and 2 * self.cos.shape[1] > spec.head_dim:
            raise ValueError(f"gated attention: {2 * self.cos.shape[1]} rotated dimensions do not fit a head of {spec.head_dim}")
        self.w_in = self.w_o = self.q_norm = self.k_norm = self.sink = self.mix = None

    @staticmethod
    def tensor_needs(spec: GatedAttentionSpec) -> List[TensorNeed]:
        H, G, dk, dv = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.value_dim
        out = [TensorNeed(spec.q_weight, (H * dk, spec.hidden)), TensorNeed(spec.o_weight, (spec.hidden, H * dv))]
        if spec.own_kv:
            out += [TensorNeed(spec.k_weight, (G * dk, spec.hidden)), TensorNeed(spec.v_weight, (G * dv, spec.hidden))]
        if spec.gate_weight:
            out.append(TensorNeed(spec.gate_weight, (H if spec.gate_per_head else H * dv, spec.hidden)))
        wide = spec.norm_scope == "projection"
        for name, heads in ((spec.q_norm, H), (spec.k_norm, G)):
            if name:
                out.append(TensorNeed(name, (heads * dk if wide else dk,), "float32", init="around_one"))
        if spec.sink:
            out.append(TensorNeed(spec.sink, (H,), "float32"))
        if spec.value_mix_weight:  # read by "mix" layers; a "first" layer's file may carry one that nobody uses
            out.append(TensorNeed(spec.value_mix_weight, (), "float32"))
        return out + list(part_class("position", spec.position.kind).tensor_needs(spec.position))

    def subparts(self):
        return (self.position,)

    def cache_needs(self):
        s = self.spec
        if not s.own_kv:
            return ()
        return (KVNeed(s.num_kv_heads, s.head_dim, s.window if s.cache_window is None else s.cache_window, value_dim=s.value_dim),)

    def kernel_notes(self):
        s, ops = self.spec, self.env.ops
        if self.env.dtype == torch.bfloat16 and hasattr(ops, "gated_attention_kernel"):
            kernel = ops.gated_attention_kernel(s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim)
            if kernel != "tensor cores":
                return [f"gated attention with heads of {s.head_dim} / {s.value_dim} numbers: runs on {kernel}"]
        return []

    def load(self, tensors) -> None:
        s = self.spec
        rows = [tensors[s.q_weight]] + ([tensors[s.k_weight], tensors[s.v_weight]] if s.own_kv else [])
        if s.gate_weight:
            rows.append(tensors[s.gate_weight])
        self.w_in = torch.cat(rows, dim=0).contiguous()  # one product for everything that reads the mixer's input
        self.w_o = tensors[s.o_weight]
        self.q_norm = tensors[s.q_norm] if s.q_norm else None
        self.k_norm = tensors[s.k_norm] if s.k_norm else None
        self.sink = tensors[s.sink] if s.sink else None
        self.mix = tensors[s.value_mix_weight].reshape(1) if s.value_mix == "mix" else None
        self.position.load(tensors)

    def forward(self, x, ctx, cache: LayerCache) -> Optional[torch.Tensor]:
        s, ops, n, dt = self.spec, self.env.ops, ctx.n_tokens, self.env.dtype
        if isinstance(x, NormalizedRows):
            x = x.dense(ctx)
        H, G, dk, dv = s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim
        if cache.k is None or (not s.own_kv and cache.writes):
            raise RuntimeError("gated attention: this layer has no keys and values of its own, and its run names no cache to read")
        if n <= 64:
            parts = ops.gemm_partials(x[:n], self.w_in, ctx.ws, "gated_attention.in_parts")
        else:
            parts = ctx.ws.get("gated_attention.in_parts", (1, n, self.w_in.shape[0]), torch.float32)
            ops.gemm(x[:n], self.w_in, parts[0])
        role, v_first = 0, None
        if s.value_mix is not None:
            shared = ctx.shared
            if s.value_mix == "first":
                role = 1
                v_first = shared[V_FIRST] = ctx.ws.get(V_FIRST, (n, G * dv), torch.float32)
            else:
                role, v_first = 2, shared.get(V_FIRST)
                if v_first is None or v_first.shape[1] != G * dv:
                    raise RuntimeError("gated attention: a layer mixes values in, but no earlier layer of the step left values of its shape")
        q = ctx.ws.get("gated_attention.q", (n, H * dk), dt)
        writes = cache.writes and cache.k is not None and s.own_kv
        wide = {"norm_wide": True} if s.norm_scope == "projection" else {}
        ops.qkv_prep(parts, H, G if s.own_kv else 0, dk, dv, self.q_norm, self.k_norm, s.eps, self.cos, self.sin, ctx, ctx.block_tables[cache.group], q,
                     cache.k if writes else None, cache.v if writes else None, role, self.mix, v_first, **wide)
        att = ctx.ws.get("gated_attention.out", (n, H * dv), dt)
        g_off = H * dk + (G * dk + G * dv if s.own_kv else 0)
        ops.gated_attention(q, cache.k, cache.v, ctx, ctx.block_tables[cache.group], att, H, G, dk, dv, s.scale, s.window, s.chunk,
                            self.sink, parts if s.gate_weight else None, g_off, **({"gate_per_head": True} if s.gate_per_head else {}))
        return add_into_stream_or_partials(ops, att, self.w_o, ctx, False, "gated_attention.delta")


register_part("mixer", "gated_attention", GatedAttention)
