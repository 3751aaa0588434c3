"""The arrangement of a layer: pre-norm residual block (tensorline/paged.py:245-276).

    h = norm1(x += pending);  a = mixer(h);  h = norm2(x += a);  pending = feed_forward(h)

The sum of a sub-block's output into the residual stream happens inside the next norm
(tensorline/paged.py:247, :275); what the feed-forward returns is handed to the next layer's
first norm (or the model's last) as `pending`.
"""
from __future__ import annotations

from .base import FEED_FORWARDS, MIXERS, NORMS, Part, PartSpec, Runtime, register_block
from .linear import PairSum, PostNormed, Scaled, StreamUpdate, resolve


@register_block("pre_norm")
class PreNormBlock(Part):
    def __init__(self, rt: Runtime, mixer: PartSpec, feed_forward: PartSpec | None, norm1: PartSpec, norm2: PartSpec | None,
                 names: dict | None = None, residual_scale: float = 1.0):
        """`feed_forward` None: the layer is norm and mixer only.  `residual_scale`: each sub-block's output counts
        that many times in the residual sum, x += scale * y."""
        super().__init__(rt)
        self.norm1 = NORMS.build(norm1, rt)
        self.mixer = MIXERS.build(mixer, rt)
        # a layer without a feed-forward has no use for a second norm; a stored one is accepted and left alone
        self.norm2 = NORMS.build(norm2, rt) if norm2 is not None else None
        self.ff = FEED_FORWARDS.build(feed_forward, rt) if feed_forward is not None else None
        self.residual_scale = float(residual_scale)
        # names of the sub-parts inside the layer's tensor prefix
        self.names = {"norm1": "input_layernorm", "mixer": "self_attn", "norm2": "post_attention_layernorm",
                      "feed_forward": "mlp", **(names or {})}

    def _children(self, prefix):
        n = self.names
        parts = ((self.norm1, f"{prefix}.{n['norm1']}"), (self.mixer, f"{prefix}.{n['mixer']}"),
                 (self.norm2, f"{prefix}.{n['norm2']}"), (self.ff, f"{prefix}.{n['feed_forward']}"))
        return tuple((part, p) for part, p in parts if part is not None)

    def expected_tensors(self, prefix):
        import dataclasses
        out = {}
        for part, p in self._children(prefix):
            specs = part.expected_tensors(p)
            if part is self.norm2 and self.ff is None:
                specs = {k: dataclasses.replace(v, optional=True) for k, v in specs.items()}
            out.update(specs)
        return out

    def bind(self, weights, prefix):
        for part, p in self._children(prefix):
            if part is self.norm2 and self.ff is None:
                continue
            part.bind(weights, p)

    def cache_need(self):
        return self.mixer.cache_need()

    @property
    def graph_capturable(self) -> bool:
        return all(part.graph_capturable for part in (self.norm1, self.mixer, self.norm2 if self.ff is not None else None, self.ff)
                   if part is not None)

    def forward(self, x, pending, ctx, cache):
        # a norm that supports it hands a part that says it can take one (`accepts_normed_input`) the recipe of its
        # result instead of the result (see parts/linear.py)
        h = self._norm(self.norm1, x, pending, self.mixer)
        a = self._addend(self.mixer.forward(h, ctx, cache))
        if self.ff is None:
            return a
        h = self._norm(self.norm2, x, a, self.ff)
        return self._addend(self.ff.forward(h, ctx))

    def _addend(self, y):
        return y if self.residual_scale == 1.0 else Scaled(y, self.residual_scale)

    @staticmethod
    def _norm(norm, x, pending, consumer):
        if getattr(consumer, "accepts_normed_input", False) and getattr(norm, "can_defer", False):
            return norm.add_norm(x, pending, defer=True)
        return norm.add_norm(x, pending)


@register_block("parallel_residual")
class ParallelResidualBlock(PreNormBlock):
    """A block whose mixer and feed-forward read the same stream, each through a norm of its own, and whose outputs join
    it together:

        x += mixer(norm1(x)) + feed_forward(norm2(x))

    The two norms share their statistics and are one kernel, which also adds the pair of outputs of the block in front
    (a `PairSum`) into the stream, in float32."""

    def forward(self, x, pending, ctx, cache):
        h1, h2 = self.norm1.add_norm_pair(x, pending, self.norm2 if self.ff is not None else None)
        a = resolve(self.mixer.forward(h1, ctx, cache))
        if self.ff is None:
            return a
        return PairSum(a, self.ff.forward(h2, ctx))


@register_block("sandwich_norm")
class SandwichNormBlock(PreNormBlock):
    """A pre-norm block whose sub-blocks are normalised once more on their way into the residual stream:

        x += norm1b(mixer(norm1(x)));   x += norm2b(feed_forward(norm2(x)))

    A sub-block's output travels as a `PostNormed` addend: its own norm, the residual sum and the next norm are one kernel
    in float32.  The second norms are the layer's `norm1b` / `norm2b` tensors (plain weights, the first norms' eps)."""

    def __init__(self, rt: Runtime, mixer: PartSpec, feed_forward: PartSpec | None, norm1: PartSpec, norm2: PartSpec | None,
                 post_norm1: PartSpec, post_norm2: PartSpec | None, names: dict | None = None):
        super().__init__(rt, mixer, feed_forward, norm1, norm2,
                         {"post_norm1": "norm1b", "post_norm2": "norm2b", **(names or {})})
        self.post1 = NORMS.build(post_norm1, rt)
        self.post2 = NORMS.build(post_norm2, rt) if post_norm2 is not None else None

    def _children(self, prefix):
        n = self.names
        parts = ((self.post1, f"{prefix}.{n['post_norm1']}"), (self.post2, f"{prefix}.{n['post_norm2']}"))
        return super()._children(prefix) + tuple((part, p) for part, p in parts if part is not None)

    def expected_tensors(self, prefix):
        import dataclasses
        out = super().expected_tensors(prefix)
        if self.ff is None and self.post2 is not None:
            for k, v in self.post2.expected_tensors(f"{prefix}.{self.names['post_norm2']}").items():
                out[k] = dataclasses.replace(v, optional=True)
        return out

    def bind(self, weights, prefix):
        for part, p in self._children(prefix):
            if self.ff is None and (part is self.norm2 or part is self.post2):
                continue
            part.bind(weights, p)

    @property
    def graph_capturable(self) -> bool:
        return super().graph_capturable

    def forward(self, x, pending, ctx, cache):
        h = self.norm1.add_norm(x, pending)
        a = PostNormed(self.mixer.forward(h, ctx, cache), self.post1.weight, self.post1.eps)
        if self.ff is None:
            return a
        h = self.norm2.add_norm(x, a)
        return PostNormed(self.ff.forward(h, ctx), self.post2.weight, self.post2.eps)


@register_block("hyper_connections")
class HyperConnectionBlock(PreNormBlock):
    """A pre-norm block over `streams` copies x_1 .. x_S of the residual stream (x float32 [T, S * hidden]).  For sublayer
    q (1: the mixer, 2: the feed-forward) with the layer's tensors `hc<q>.in` [S], `hc<q>.out` [S] and `hc<q>.mix` [S, S]:

        u = sum_s in[s] x_s;   y = sublayer(norm_q(u));   x_r <- sum_s mix[s, r] x_s + out[r] y     for every r at once

    The rebuild of the copies travels as a `StreamUpdate` to the next norm (this block's second, the next block's first or
    the model's), which applies it, reads the copies with its own `in` and normalises, all in one float32 kernel."""

    def __init__(self, rt: Runtime, mixer: PartSpec, feed_forward: PartSpec | None, norm1: PartSpec, norm2: PartSpec | None,
                 streams: int, names: dict | None = None):
        super().__init__(rt, mixer, feed_forward, norm1, norm2, {"hc1": "hc1", "hc2": "hc2", **(names or {})})
        if not 1 <= streams <= 16:
            raise ValueError(f"{streams} stream copies: the kernel takes 1 to 16")
        self.S = int(streams)
        self.hc = {}

    def _hc_names(self, prefix, q):
        base = f"{prefix}.{self.names[f'hc{q}']}"
        return {"in": f"{base}.in", "out": f"{base}.out", "mix": f"{base}.mix"}

    def expected_tensors(self, prefix):
        from .base import TensorSpec
        out = super().expected_tensors(prefix)
        for q in (1, 2) if self.ff is not None else (1,):
            n = self._hc_names(prefix, q)
            out[n["in"]] = TensorSpec((self.S,), init="ones")
            out[n["out"]] = TensorSpec((self.S,), init="ones")
            out[n["mix"]] = TensorSpec((self.S, self.S))
        return out

    def bind(self, weights, prefix):
        super().bind(weights, prefix)
        for q in (1, 2) if self.ff is not None else (1,):
            n = self._hc_names(prefix, q)
            self.hc[q] = {k: weights[n[k]].float().contiguous() for k in ("in", "out", "mix")}      # they enter float32 sums

    def forward(self, x, pending, ctx, cache):
        h = self.norm1.read_streams(x, pending, self.hc[1]["in"])
        update = StreamUpdate(self.mixer.forward(h, ctx, cache), self.hc[1]["mix"], self.hc[1]["out"])
        if self.ff is None:
            return update
        h = self.norm2.read_streams(x, update, self.hc[2]["in"])
        return StreamUpdate(self.ff.forward(h, ctx), self.hc[2]["mix"], self.hc[2]["out"])
