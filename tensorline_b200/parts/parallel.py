"""A mixer made of two mixers side by side: both read the same input, each output is RMS-normalised over the
model width with a weight of its own (a plain weight, statistics in float32), and the result is a fixed multiple
of their sum (one half: the mean).

    y = scale * (left(h) / rms(left(h)) * w_left + right(h) / rms(right(h)) * w_right)

With `normed` False the outputs are not normalised and there are no such weights: the result is
left_scale * left(h) + right_scale * right(h), handed on as a `WeightedPair` that the residual sum multiplies and adds in float32.

The two may keep different things between steps (pages of keys and values, a state slot): the mixer's cache need
is {"left": ..., "right": ...} and it is handed {"left": view, "right": view}.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import MIXERS, Part, PartSpec, Runtime, TensorSpec, register_mixer
from .linear import WeightedPair, resolve


@register_mixer("parallel_pair")
class ParallelPair(Part):
    def __init__(self, rt: Runtime, hidden: int, left: PartSpec, right: PartSpec, norm_eps: float, scale: float = 0.5,
                 names: dict | None = None, normed: bool = True, left_scale: float = 1.0, right_scale: float = 1.0):
        super().__init__(rt)
        self.hidden, self.eps, self.scale = hidden, norm_eps, float(scale)
        self.normed, self.left_scale, self.right_scale = bool(normed), float(left_scale), float(right_scale)
        self.left, self.right = MIXERS.build(left, rt), MIXERS.build(right, rt)
        self.names = {"left": "left", "right": "right", "left_norm": "left.out", "right_norm": "right.out", **(names or {})}
        self.w_left = self.w_right = None

    @property
    def graph_capturable(self) -> bool:
        return self.left.graph_capturable and self.right.graph_capturable

    def cache_need(self):
        needs = {"left": self.left.cache_need(), "right": self.right.cache_need()}
        return {k: v for k, v in needs.items() if v is not None} or None

    def expected_tensors(self, prefix):
        n = self.names
        out = dict(self.left.expected_tensors(f"{prefix}.{n['left']}"))
        out.update(self.right.expected_tensors(f"{prefix}.{n['right']}"))
        if self.normed:
            out[f"{prefix}.{n['left_norm']}"] = TensorSpec((self.hidden,), init="ones")
            out[f"{prefix}.{n['right_norm']}"] = TensorSpec((self.hidden,), init="ones")
        return out

    def bind(self, weights, prefix):
        n = self.names
        self.left.bind(weights, f"{prefix}.{n['left']}")
        self.right.bind(weights, f"{prefix}.{n['right']}")
        if self.normed:
            self.w_left = weights[f"{prefix}.{n['left_norm']}"].contiguous()
            self.w_right = weights[f"{prefix}.{n['right_norm']}"].to(self.w_left.dtype).contiguous()

    def forward(self, h, ctx, cache):
        cache = cache or {}
        a = resolve(self.left.forward(h, ctx, cache.get("left")))
        b = resolve(self.right.forward(h, ctx, cache.get("right")))
        if not self.normed:
            return WeightedPair(a, self.left_scale, b, self.right_scale)
        y = torch.empty_like(a)
        ops.sum_normed(a, b, self.w_left, self.w_right, y, self.eps, self.scale)
        return y
