"""Choice of the attention kernel for a step.

float32: the exact-order kernel for everything.  bfloat16: the tensor-core kernels, one for
steps that hold prompt portions and one (split over the keys) for steps of single decoded
tokens; both read the same pages.  `ctx.force_exact_attention` routes a bfloat16 step through
the exact-order kernel too (tests compare the two).
"""
from __future__ import annotations

import torch

from .. import ops


def attend(mixer, qkv, o, ctx, cache, table, rope=None, gate=None) -> None:
    """`gate` (float32 [T, query heads]): head h's output of token t is multiplied by sigmoid(gate[t, h]); the exact-order
    kernel does it where it writes a row, the tensor-core kernels are followed by a kernel that does."""
    nq, nkv, d = mixer.nq, mixer.nkv, mixer.d
    sink = getattr(mixer, "sink", None)
    keep_first = getattr(mixer, "keep_first", 0) if mixer.window else 0
    chunk, slopes = getattr(mixer, "chunk", None), getattr(mixer, "slopes", None)
    from .. import ops_attention
    if qkv.dtype == torch.float32 or ctx.force_exact_attention or d > 256 or \
            (keep_first and not ops_attention.TAKES_KEEP_FIRST) or \
            ((chunk or slopes is not None) and not ops_attention.TAKES_CHUNKS):   # heads wider than the tensor-core kernels take
        ops.attn_tokenwise(qkv, qkv.shape[1], o, cache.k, cache.v, table, ctx.page_size, ctx.pos, ctx.req_slot,
                           nq, nkv, d, mixer.window, mixer.scale, sink=sink, keep_first=keep_first, gate=gate, chunk=chunk,
                           slopes=slopes)
        return
    ops_attention.attend_bf16(qkv, o, ctx, cache.k, cache.v, table, nq, nkv, d, mixer.window, mixer.scale, rope=rope, sink=sink,
                              keep_first=keep_first, chunk=chunk, slopes=slopes)
    if gate is not None:
        ops.head_gate(o, gate, nq, d)
