"""RMSNorm with the residual add folded in (tensorline/fused.py:19-32, :58-69)."""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, Runtime, TensorSpec, register_norm, tensor_name
from .linear import FUSE_NORMS, NormedInput, PairSum, PendingProduct, PostNormed, Scaled, SplitSum, StreamUpdate, WeightedPair, resolve


@register_norm("rms_norm")
class RMSNorm(Part):
    graph_capturable = True
    can_defer = True                    # add_norm(..., defer=True) may return a `NormedInput`

    def __init__(self, rt: Runtime, dim: int, eps: float, tensor: str = "weight", one_plus: bool = False,
                 cast_first: bool = True):
        """`tensor`: the weight's name under the norm's prefix ("": the prefix itself).  `one_plus`: the stored weight
        lies around zero and the norm multiplies by 1 + w.  `cast_first` False: x * rstd * w in float32 and one
        rounding at the end, instead of a rounding to the activation type before the weight."""
        super().__init__(rt)
        self.dim, self.eps = dim, eps
        self.tensor, self.one_plus, self.cast_first = tensor, one_plus, cast_first
        self.can_defer = cast_first and not one_plus         # the products that normalise on the fly round first
        self.weight = None

    def expected_tensors(self, prefix):
        return {tensor_name(prefix, self.tensor): TensorSpec((self.dim,), init="normal" if self.one_plus else "ones")}

    def bind(self, weights, prefix):
        w = weights[tensor_name(prefix, self.tensor)]
        self.weight = (1.0 + w.float()).contiguous() if self.one_plus else w.contiguous()      # else in its stored type

    def norm_stream(self, x):
        """The float32 stream itself normalised, x <- norm(x), nothing rounded (a norm right behind the embedding)."""
        out = torch.empty_like(x)
        ops.add_rmsnorm(x, None, self.weight, out, self.eps, cast_first=False)
        return out

    def add_norm_pair(self, x, pending, other: "RMSNorm | None", rows=None):
        """x += pending (a tensor, a `PairSum` or None), then this norm and `other`'s of the same rows of x with one set
        of statistics: (h, h_other); float32 up to the weights, the results rounded once.  `other` None: (h, None)."""
        if self.cast_first or self.one_plus or (other is not None and (other.cast_first or other.one_plus or other.eps != self.eps
                                                                      or other.weight.dtype != self.weight.dtype)):
            raise NotImplementedError("two norms of one stream share a kernel only as plain float32 norms with one eps")
        a = b = None
        if isinstance(pending, PairSum):
            a, b = pending.a, pending.b
        elif pending is not None:
            a = resolve(pending)
        n = x.shape[0] if rows is None else rows.numel()
        h = torch.empty((n, self.dim), dtype=self.rt.act_dtype, device=x.device)
        h2 = torch.empty_like(h) if other is not None else None
        ops.add_rmsnorm_pair(x, a, b, self.weight, None if other is None else other.weight, h, h2, self.eps, rows=rows)
        return h, h2

    def read_streams(self, x, pending, read, rows=None):
        """x float32 [T, S * dim]: S copies of the residual stream side by side.  `pending` (a `StreamUpdate` or None) is
        applied to them; then u = sum_r read[r] x_r (`read` float32 [S]; None: the plain sum) is normalised: one kernel,
        float32 up to the rounding of the result.  With `rows` only those rows are produced and x is left alone."""
        if self.cast_first or self.one_plus:
            raise NotImplementedError("several stream copies are read by plain float32 norms")
        S = x.shape[1] // self.dim
        n = x.shape[0] if rows is None else rows.numel()
        h = torch.empty((n, self.dim), dtype=self.rt.act_dtype, device=x.device)
        kw = {}
        if pending is not None:
            v = pending.value
            if isinstance(v, WeightedPair):
                kw = {"a": v.a, "alpha": v.alpha, "b": v.b, "beta": v.beta}
            else:
                kw = {"a": v}
            kw.update(mix=pending.mix, out=pending.out)
        ops.stream_step(x, S, read=read, w=self.weight, eps=self.eps, h=h, rows=rows, **kw)
        return h

    def add_norm(self, x, pending, rows=None, defer=False):
        """`defer`: the caller's next step is a product that takes a `NormedInput`."""
        n = x.shape[0] if rows is None else rows.numel()
        if isinstance(pending, StreamUpdate) or x.shape[1] != self.dim:       # several copies: their sum is what this norm reads
            return self.read_streams(x, pending, None, rows=rows)
        if isinstance(pending, WeightedPair):
            pending = resolve(pending)
        if isinstance(pending, PairSum):
            if self.cast_first or self.one_plus:
                x.add_(pending.a.float() + pending.b.float())
                pending = None
            else:
                return self.add_norm_pair(x, pending, None, rows=rows)[0]
        if isinstance(pending, PostNormed):              # x += value / rms(value) * its weight (+ a row), then this norm
            if self.cast_first or self.one_plus or pending.eps != self.eps or \
                    (pending.weight is not None and pending.weight.dtype != self.weight.dtype):
                if rows is not None:
                    raise NotImplementedError("a normalised addend before a norm of picked rows needs this norm's float form")
                pending.add_into(x)
                pending = None
            else:
                h = torch.empty((n, self.dim), dtype=self.rt.act_dtype, device=x.device)
                ops.post_norm_add_norm(x, pending.value, pending.weight if pending.value is not None else None, self.weight, h,
                                       self.eps, extra=pending.extra, rows=rows)
                return h
        if isinstance(pending, Scaled):                  # x += alpha * value
            h = torch.empty((n, self.dim), dtype=self.rt.act_dtype, device=x.device)
            ops.add_rmsnorm(x, pending.value, self.weight, h, self.eps, rows=rows, alpha=pending.alpha, cast_first=self.cast_first)
            return h
        if not self.cast_first:
            pending = resolve(pending)
            h = torch.empty((n, self.dim), dtype=self.rt.act_dtype, device=x.device)
            ops.add_rmsnorm(x, pending, self.weight, h, self.eps, rows=rows, cast_first=False)
            return h
        if isinstance(pending, PendingProduct):
            ssq = pending.add_into(x)                    # the product adds its result into x itself, where its plan allows
            if ssq is None:
                pending = pending.run()
            else:                                        # x holds the sum (also with `rows`: nobody reads x after the last norm)
                if defer and FUSE_NORMS and self.dim % 8 == 0 and self.weight.dtype in (torch.float32, torch.bfloat16):
                    return NormedInput(x, ssq, self.weight, self.eps, rows, self.rt.act_dtype)
                h = torch.empty((n, self.dim), dtype=self.rt.act_dtype, device=x.device)
                ops.add_rmsnorm(x, None, self.weight, h, self.eps, rows=rows)
                return h
        h = torch.empty((n, self.dim), dtype=self.rt.act_dtype, device=x.device)
        if isinstance(pending, SplitSum):                # a split-K product: its pieces are summed inside the kernel
            if pending.dtype == h.dtype and self.dim % 4 == 0 and self.dim <= 32768:
                ops.add_rmsnorm(x, None, self.weight, h, self.eps, rows=rows, pieces=pending.pieces)
                return h
            pending = pending.sum()
        ops.add_rmsnorm(x, pending, self.weight, h, self.eps, rows=rows)
        return h
