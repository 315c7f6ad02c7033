"""Two mixers side by side: both read the same input, each keeps its own cache or state (their needs are put together: one may
keep keys and values, both may keep state under names of their own), and their results become one (MixerPairSpec):
"weighted": left_scale * left + right_scale * right; "normed_mean": the mean of the two, each first divided by its root mean
square over the model width and multiplied by a weight of its own. One kernel adds the two sets of float32 sums."""
from __future__ import annotations

from typing import List, Optional

import torch

from .base import KVNeed, LayerCache, Mixer, NormalizedRows
from .registry import build_part, part_class, register_part
from .spec import MixerPairSpec, TensorNeed


class MixerPair(Mixer):
    def __init__(self, spec: MixerPairSpec, env):
        super().__init__(spec, env)
        if spec.combine not in ("weighted", "normed_mean"):
            raise ValueError(f"mixer pair: combine '{spec.combine}' is not implemented (weighted and normed_mean are)")
        if spec.combine == "normed_mean" and not (spec.left_norm and spec.right_norm):
            raise ValueError("mixer pair: normed_mean needs the names of both weights")
        self.left = build_part("mixer", spec.left, env)
        self.right = build_part("mixer", spec.right, env)
        needs = list(self.left.cache_needs()) + list(self.right.cache_needs())
        names = [n.name for n in needs if not isinstance(n, KVNeed)]
        if len(names) != len(set(names)) or sum(isinstance(n, KVNeed) for n in needs) > 1:
            raise ValueError("mixer pair: the two mixers' states need names of their own, and at most one of them keeps keys and values")
        self._needs = tuple(needs)
        self.left_norm = self.right_norm = None

    @staticmethod
    def tensor_needs(spec: MixerPairSpec) -> List[TensorNeed]:
        out = list(part_class("mixer", spec.left.kind).tensor_needs(spec.left)) + list(part_class("mixer", spec.right.kind).tensor_needs(spec.right))
        if spec.combine == "normed_mean":
            out += [TensorNeed(spec.left_norm, (spec.hidden,), "float32", init="around_one"),
                    TensorNeed(spec.right_norm, (spec.hidden,), "float32", init="around_one")]
        return out

    def subparts(self):
        return (self.left, self.right)

    def cache_needs(self):
        return self._needs

    def load(self, tensors) -> None:
        self.left.load(tensors)
        self.right.load(tensors)
        if self.spec.combine == "normed_mean":
            self.left_norm, self.right_norm = tensors[self.spec.left_norm], tensors[self.spec.right_norm]

    def forward(self, x, ctx, cache: LayerCache) -> Optional[torch.Tensor]:
        s, ops, n = self.spec, self.env.ops, ctx.n_tokens
        if isinstance(x, NormalizedRows):
            x = x.dense(ctx)
        keep = ctx.residual
        ctx.residual = None  # neither side adds into the stream: their sums are put together first
        a = self.left.forward(x, ctx, cache)
        b = self.right.forward(x, ctx, cache)
        ctx.residual = keep
        out = ctx.ws.get("mixer_pair.delta", (n, s.hidden), torch.float32)
        if s.combine == "weighted":
            return ops.pair_combine(a, b, None, None, s.left_scale, s.right_scale, 0.0, out, n)
        return ops.pair_combine(a, b, self.left_norm, self.right_norm, 0.5, 0.5, s.eps, out, n)


register_part("mixer", "mixer_pair", MixerPair)
