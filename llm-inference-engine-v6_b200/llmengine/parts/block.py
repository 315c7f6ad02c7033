"""Arrangement of parts in a layer. "pre_norm": h += mixer(norm1(h)); h += feed_forward(norm2(h))
(src/engine.cpp:307-413). The residual sums are fused into the norm that follows them.
"parallel": h += mixer(norm1(h)) + feed_forward(norm2(h)), both norms of the same h (or, without a norm2, ONE norm whose
rows both sub-layers read); then an optional input from the tokens themselves, h += token_input(h).
"post_norm": the sub-layers read h itself and the norms sit on their outputs, each followed by an optional per-column
layer scale: h += scale1 * norm1(mixer(h)); h += scale2 * norm2(feed_forward(h)).
"sandwich": a norm before and one after each sub-layer, and one multiplier on everything that is added:
h += m * norm1_out(mixer(norm1(h))); h += m * norm2_out(feed_forward(norm2(h)))."""
from __future__ import annotations

from typing import List

import torch

from .base import Block, LayerCache, Norm, Residual
from .registry import build_part, part_class, register_part
from .spec import BlockSpec, TensorNeed


class PreNormBlock(Block):
    def __init__(self, spec: BlockSpec, env):
        super().__init__(spec, env)
        self.norm1 = build_part("norm", spec.norm1, env)
        self.mixer = build_part("mixer", spec.mixer, env)
        self.norm2 = build_part("norm", spec.norm2, env)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, env)

    @staticmethod
    def tensor_needs(spec: BlockSpec) -> List[TensorNeed]:
        out: List[TensorNeed] = []
        for cat, sub in (("norm", spec.norm1), ("mixer", spec.mixer), ("norm", spec.norm2),
                         ("feed_forward", spec.feed_forward)):
            out += part_class(cat, sub.kind).tensor_needs(sub)
        return out

    def subparts(self):
        return (self.norm1, self.mixer, self.norm2, self.feed_forward)

    def cache_needs(self):
        return self.mixer.cache_needs()

    def load(self, tensors) -> None:
        for p in (self.norm1, self.mixer, self.norm2, self.feed_forward):
            p.load(tensors)

    def first_norm(self):
        return self.norm1

    def forward(self, res: Residual, ctx, cache: LayerCache) -> Residual:
        ctx.residual = res  # a part whose last product can add into the stream itself returns None
        x = self._norm(self.norm1, self.mixer, res, ctx)
        ctx.next_norm = self.norm2  # who reads the stream after the mixer has written it
        res.pending = self.mixer.forward(x, ctx, cache)
        x = self._norm(self.norm2, self.feed_forward, res, ctx)
        ctx.next_norm = getattr(ctx, "norm_after_block", None)
        res.pending = self.feed_forward.forward(x, ctx)
        ctx.residual = ctx.next_norm = None
        return res

    @staticmethod
    def _norm(norm, consumer, res: Residual, ctx):
        if norm.can_defer and consumer.wants_lazy_norm(ctx):
            return norm.forward(res, ctx, lazy=True)
        return norm.forward(res, ctx)


class ParallelBlock(Block):
    """Mixer and feed-forward read the same stream through a norm each; their results are added together.
    What is pending on the stream is added by the first norm; the two deltas are added by one kernel, which
    also leaves the stream in the engine dtype when a token input wants it as an operand; the token input's
    delta is left pending for the next reader."""

    def __init__(self, spec: BlockSpec, env):
        super().__init__(spec, env)
        self.norm1 = build_part("norm", spec.norm1, env)
        self.mixer = build_part("mixer", spec.mixer, env)
        self.feed_forward = self.norm2 = self.token_input = None
        if spec.feed_forward is not None:
            if spec.norm2 is not None:  # None: the feed-forward reads the first norm's rows
                self.norm2 = build_part("norm", spec.norm2, env)
            self.feed_forward = build_part("feed_forward", spec.feed_forward, env)
        if spec.token_input is not None:
            self.token_input = build_part("token_input", spec.token_input, env)

    @staticmethod
    def tensor_needs(spec: BlockSpec) -> List[TensorNeed]:
        out: List[TensorNeed] = []
        subs = [("norm", spec.norm1), ("mixer", spec.mixer)]
        if spec.feed_forward is not None:
            subs += ([("norm", spec.norm2)] if spec.norm2 is not None else []) + [("feed_forward", spec.feed_forward)]
        if spec.token_input is not None:
            subs.append(("token_input", spec.token_input))
        for cat, sub in subs:
            out += part_class(cat, sub.kind).tensor_needs(sub)
        return out

    def subparts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward, self.token_input) if p is not None)

    def cache_needs(self):
        return self.mixer.cache_needs()

    def load(self, tensors) -> None:
        for p in self.subparts():
            p.load(tensors)

    def first_norm(self):
        return self.norm1

    def forward(self, res: Residual, ctx, cache: LayerCache) -> Residual:
        ops, n = self.env.ops, ctx.n_tokens
        ctx.residual = ctx.next_norm = None  # the parts' last products return their sums; nobody adds into the stream
        x1 = self.norm1.forward(res, ctx)    # adds what is pending
        # the second norm's rows go to a buffer of their own: the mixer runs first and both read the same stream
        x2 = None
        if self.feed_forward is not None:
            if self.norm2 is None:
                x2 = x1  # one norm for both: the mixer leaves its input as it is
            else:
                x2 = ctx.ws.get("block.norm2_out", (n, res.h.shape[1]), self.env.dtype)
                self.norm2.run(res.h, ctx, None, n, out=x2)
        a = self.mixer.forward(x1, ctx, cache)
        b = self.feed_forward.forward(x2, ctx) if self.feed_forward is not None else None
        if self.token_input is None:
            if b is None:
                res.pending = a
            else:
                ops.stream_add(res.h, a, b, n_rows=n)
            res.sumsq = res.prescaled = res.prescaled_weight = res.operand = None
            return res
        xs = ctx.ws.get("block.stream_copy", (n, res.h.shape[1]), self.env.dtype)
        ops.stream_add(res.h, a, b, copy=xs, n_rows=n)
        res.sumsq = res.prescaled = res.prescaled_weight = res.operand = None
        res.pending = self.token_input.forward(xs, ctx)
        return res


class PostNormBlock(Block):
    """h += scale1 * norm1(mixer(h)); h += scale2 * norm2(feed_forward(h)): the sub-layers read the stream itself (in the
    engine precision, as the operand of their first product), the norms (of the form weight * y / rms(y)) sit on their
    results. One kernel a sub-layer takes the result's partial sums, normalises, scales, adds into the float32 stream and
    leaves the stream in the engine precision for the next reader."""

    def __init__(self, spec: BlockSpec, env):
        super().__init__(spec, env)
        self.norm1 = build_part("norm", spec.norm1, env)
        self.mixer = build_part("mixer", spec.mixer, env)
        self.feed_forward = self.norm2 = None
        if spec.feed_forward is not None:
            self.norm2 = build_part("norm", spec.norm2, env)
            self.feed_forward = build_part("feed_forward", spec.feed_forward, env)
        for norm in (self.norm1, self.norm2):
            if norm is not None and type(norm).prescale_weight is Norm.prescale_weight:  # not a norm that can be applied as weight * y * s(row)
                raise ValueError("a post-norm block needs norms of the form weight * y / rms(y)")
        self.scale1 = self.scale2 = None

    @staticmethod
    def tensor_needs(spec: BlockSpec) -> List[TensorNeed]:
        out: List[TensorNeed] = []
        subs = [("norm", spec.norm1), ("mixer", spec.mixer)]
        if spec.feed_forward is not None:
            subs += [("norm", spec.norm2), ("feed_forward", spec.feed_forward)]
        for cat, sub in subs:
            out += part_class(cat, sub.kind).tensor_needs(sub)
        if spec.scale1:
            out.append(TensorNeed(spec.scale1, (spec.norm1.dim,), "float32", init="around_one"))
        if spec.scale2 and spec.feed_forward is not None:
            out.append(TensorNeed(spec.scale2, (spec.norm2.dim,), "float32", init="around_one"))
        return out

    def subparts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None)

    def cache_needs(self):
        return self.mixer.cache_needs()

    def load(self, tensors) -> None:
        for p in self.subparts():
            p.load(tensors)
        self.scale1 = tensors[self.spec.scale1] if self.spec.scale1 else None
        self.scale2 = tensors[self.spec.scale2] if (self.spec.scale2 and self.feed_forward is not None) else None

    def forward(self, res: Residual, ctx, cache: LayerCache) -> Residual:
        ops, n, dt = self.env.ops, ctx.n_tokens, self.env.dtype
        ctx.residual = ctx.next_norm = None  # the parts' last products return their sums; nobody adds into the stream
        same = dt == torch.float32  # the 32-bit engine reads the stream as it is
        xs = res.h if same else ctx.ws.get("block.stream_copy", (n, res.h.shape[1]), dt)
        if res.pending is not None or not (same or (res.operand is not None and res.operand.data_ptr() == xs.data_ptr())):
            # what an earlier block left pending is added, and the stream in the engine precision is made, unless the block
            # before this one was of this kind and has left it (its last kernel writes it)
            ops.stream_add(res.h, res.pending, None, copy=None if same else xs, n_rows=n)
            res.pending = None
        res.sumsq = res.prescaled = res.prescaled_weight = None
        a = self.mixer.forward(xs, ctx, cache)
        ops.norm_add(res.h, a, None, self.norm1.prescale_weight(), self.scale1, self.norm1.spec.eps, copy=None if same else xs, n_rows=n)
        if self.feed_forward is not None:
            ctx.takes_delta_pairs = True  # a feed-forward made of two branches may hand both sets of sums over: one kernel adds them
            b = self.feed_forward.forward(xs, ctx)
            ctx.takes_delta_pairs = False
            b, b2 = b if isinstance(b, tuple) else (b, None)
            ops.norm_add(res.h, b, b2, self.norm2.prescale_weight(), self.scale2, self.norm2.spec.eps, copy=None if same else xs, n_rows=n)
        res.operand = None if same else xs  # valid until somebody else writes the stream
        return res


class SandwichBlock(Block):
    """h += m * norm1_out(mixer(norm1(h))); h += m * norm2_out(feed_forward(norm2(h))). The norms before the sub-layers are the
    framework's norm kernel on the float32 stream; the norms on the results (of the form weight * y / rms(y)) run in the kernel
    that takes a sub-layer's float32 sums, normalises, multiplies by m and adds into the stream, the row in registers."""

    def __init__(self, spec: BlockSpec, env):
        super().__init__(spec, env)
        if spec.norm1_out is None or (spec.feed_forward is not None and (spec.norm2 is None or spec.norm2_out is None)):
            raise ValueError("a sandwich block needs a norm before and after each of its sub-layers")
        self.norm1 = build_part("norm", spec.norm1, env)
        self.mixer = build_part("mixer", spec.mixer, env)
        self.norm1_out = build_part("norm", spec.norm1_out, env)
        self.feed_forward = self.norm2 = self.norm2_out = None
        if spec.feed_forward is not None:
            self.norm2 = build_part("norm", spec.norm2, env)
            self.feed_forward = build_part("feed_forward", spec.feed_forward, env)
            self.norm2_out = build_part("norm", spec.norm2_out, env)
        for norm in (self.norm1_out, self.norm2_out):
            if norm is not None and type(norm).prescale_weight is Norm.prescale_weight:
                raise ValueError("a sandwich block needs norms of the form weight * y / rms(y) on its sub-layers' results")
        self.mult = None

    def _subs(self):
        spec = self.spec
        subs = [("norm", spec.norm1), ("mixer", spec.mixer), ("norm", spec.norm1_out)]
        if spec.feed_forward is not None:
            subs += [("norm", spec.norm2), ("feed_forward", spec.feed_forward), ("norm", spec.norm2_out)]
        return subs

    @staticmethod
    def tensor_needs(spec: BlockSpec) -> List[TensorNeed]:
        out: List[TensorNeed] = []
        subs = [("norm", spec.norm1), ("mixer", spec.mixer), ("norm", spec.norm1_out)]
        if spec.feed_forward is not None:
            subs += [("norm", spec.norm2), ("feed_forward", spec.feed_forward), ("norm", spec.norm2_out)]
        for cat, sub in subs:
            out += part_class(cat, sub.kind).tensor_needs(sub)
        return out

    def subparts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.norm1_out, self.norm2, self.feed_forward, self.norm2_out) if p is not None)

    def cache_needs(self):
        return self.mixer.cache_needs()

    def load(self, tensors) -> None:
        for p in self.subparts():
            p.load(tensors)
        m = float(self.spec.residual_mult)
        self.mult = None if m == 1.0 else torch.full((self.spec.norm1.dim,), m, dtype=torch.float32, device=self.env.device)

    def first_norm(self):
        return self.norm1

    def forward(self, res: Residual, ctx, cache: LayerCache) -> Residual:
        ops, n = self.env.ops, ctx.n_tokens
        ctx.residual = ctx.next_norm = None  # the parts' last products return their sums; the norms on them add into the stream
        x = self.norm1.forward(res, ctx)     # adds what an earlier block left pending
        a = self.mixer.forward(x, ctx, cache)
        ops.norm_add(res.h, a, None, self.norm1_out.prescale_weight(), self.mult, self.norm1_out.spec.eps, n_rows=n)
        res.sumsq = res.prescaled = res.prescaled_weight = res.operand = None
        if self.feed_forward is not None:
            x = self.norm2.forward(res, ctx)
            b = self.feed_forward.forward(x, ctx)
            ops.norm_add(res.h, b, None, self.norm2_out.prescale_weight(), self.mult, self.norm2_out.spec.eps, n_rows=n)
        return res


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "sandwich", SandwichBlock)
register_part("block", "post_norm", PostNormBlock)
register_part("block", "parallel", ParallelBlock)
