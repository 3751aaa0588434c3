"""Token embedding (tensorline/paged.py:240) and the output head (tensorline/paged.py:287)."""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, Runtime, TensorSpec, register_embedding, register_head, tensor_name
from .linear import matmul


@register_embedding("token_table")
class Embedding(Part):
    graph_capturable = True

    def __init__(self, rt: Runtime, vocab: int, dim: int, tensor: str = "weight", scale: float = 1.0, copies: int = 1):
        """`scale`: every row is multiplied by it on its way into the stream (in float32; a tied head reads the table itself).
        `copies`: the stream starts as that many equal copies side by side, [T, copies * dim]."""
        super().__init__(rt)
        self.vocab, self.dim, self.tensor, self.scale, self.copies = vocab, dim, tensor, float(scale), int(copies)
        self.weight = None

    def expected_tensors(self, prefix):
        return {tensor_name(prefix, self.tensor): TensorSpec((self.vocab, self.dim))}

    def bind(self, weights, prefix):
        self.weight = self._compute_copy(weights[tensor_name(prefix, self.tensor)])

    def forward(self, ids):
        """The residual stream starts here, in float32."""
        x = torch.empty((ids.numel(), self.copies * self.dim), dtype=torch.float32, device=ids.device)
        if self.copies == 1:
            ops.embed(x, self.weight, ids, scale=self.scale)
        else:
            ops.embed_streams(x, self.weight, ids, scale=self.scale, copies=self.copies)
        return x


@register_embedding("token_pairs")
class PairEmbedding(Embedding):
    """The token's row times `scale` plus a row of a second table chosen by a hash of (previous token, token):

        row = (previous * mul_prev + token * mul_cur) mod buckets;   a request's first token takes row `buckets`

    The table (`pairs_tensor`, a name beside the embedding's own) has buckets + 1 rows.  The previous token of the first
    row of a portion is the request's last token of the step before: one int32 per request slot, written behind every
    step by a kernel of its own, so the part reads the step from device tensors only."""

    def __init__(self, rt: Runtime, vocab: int, dim: int, buckets: int, mul_prev: int, mul_cur: int, tensor: str = "weight",
                 scale: float = 1.0, copies: int = 1, pairs_tensor: str = "pairs"):
        super().__init__(rt, vocab, dim, tensor, scale, copies)
        self.buckets, self.mul_prev, self.mul_cur, self.pairs_tensor = int(buckets), int(mul_prev), int(mul_cur), pairs_tensor
        self.pairs = None

    def cache_need(self):
        from ..cache import SlotState
        return SlotState((1,), "int32")

    def expected_tensors(self, prefix):
        out = super().expected_tensors(prefix)
        out[self.pairs_tensor] = TensorSpec((self.buckets + 1, self.dim))
        return out

    def bind(self, weights, prefix):
        super().bind(weights, prefix)
        self.pairs = self._compute_copy(weights[self.pairs_tensor]).to(self.weight.dtype)

    def forward(self, ids, ctx=None, cache=None):
        if ctx is None or cache is None:
            raise ops.KernelError("the pair embedding needs the step's context and its state of one token a request slot")
        x = torch.empty((ids.numel(), self.copies * self.dim), dtype=torch.float32, device=ids.device)
        last = cache.state.view(-1)
        ops.embed_streams(x, self.weight, ids, scale=self.scale, copies=self.copies, pairs=self.pairs, mul_prev=self.mul_prev,
                          mul_cur=self.mul_cur, pos=ctx.pos, req_slot=ctx.req_slot, last_token=last)
        ops.remember_last(ids, ctx.q_start, ctx.slots, last, ctx.B)
        return x


@register_head("linear")
class LMHead(Part):
    """logits = h W^T in float32, no bias.  Tied: W is the embedding table; a stored
    `lm_head.weight` is then ignored."""
    graph_capturable = True
    accepts_normed_input = True         # `h` may be a `NormedInput`: the product normalises it on the fly

    def __init__(self, rt: Runtime, vocab: int, dim: int, tied: bool, tensor: str = "weight", softcap: float | None = None):
        """`softcap`: the logits become softcap * tanh(logits / softcap)."""
        super().__init__(rt)
        self.vocab, self.dim, self.tied, self.tensor = vocab, dim, tied, tensor
        self.softcap = None if softcap is None else float(softcap)
        self.weight = None

    def expected_tensors(self, prefix):
        return {tensor_name(prefix, self.tensor): TensorSpec((self.vocab, self.dim), optional=self.tied)}

    def bind(self, weights, prefix, embedding: Embedding | None = None):
        if self.tied:
            self.weight = embedding.weight
        else:
            self.weight = self._compute_copy(weights[tensor_name(prefix, self.tensor)])

    def forward(self, h):
        logits = matmul(h, self.weight, out_dtype=torch.float32)
        if self.softcap is not None:
            logits = logits.contiguous()
            ops.softcap(logits, self.softcap)
        return logits
