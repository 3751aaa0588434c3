"""Grouped-query attention over the paged cache: the mixer of this architecture.

Order of work for the T tokens of a step (tensorline/paged.py:248-275):
  qkv = h Wqkv^T                      one product against the stacked q|k|v matrix
  bias, rotary encoding, K/V write    one kernel (tensorline/fused.py:34-51, paged.py:252-253);
                                      every token's k, v are in the pages before any query runs
  attention over the pages            query at position p reads keys lo..p of its own request
                                      (paged.py:237, paged_attn.py:43), scale d^-1/2 (paged.py:119)
  y = o Wo^T                          no bias
The number of heads, of KV heads, the head size, the biases, the window, the position encoding
(with its pairing of dimensions) and an optional RMS norm of every q and k head before the rotation
(`qk_norm_eps`; weights `q_norm.weight`, `k_norm.weight` of the head size) are parameters; the
fused kernel takes all of them as arguments.  A run entry that reads another entry's cache
(`cache.owner` false) computes its own queries and writes no keys or values.

Further parameters: `sink` (a learned number per query head, tensor `sink`: every softmax denominator of the
head also holds exp(sink), a term without key or value that is not scaled), `v_head_dim` (values of another size
than queries and keys) and `names` (the tensors' names under the mixer's prefix).  The kernels and the pages work
on one head size: with `v_head_dim` != `head_dim`, or a size the bfloat16 kernels do not take, the smaller of
q/k and v is padded with zero rows in the stacked projection (and zero columns in the output projection), which
changes no score and no output.

`keep_first` (with a window): the first `keep_first` positions of the request stay visible to every later query beside
its window, at their true positions.  `sink_value`: the sink is this fixed number for every head instead of a tensor
(0.0: the denominator holds one more term 1).  `head_gate` (tensor `head_gate`, [query heads, hidden]): head h's output
is multiplied by sigmoid(W_g x)_h, one number per token and head computed in float32 from the mixer's input, before the
output projection.

`chunk` (instead of a window): the sequence is cut into chunks of that many positions counted from position 0, and a query
reads the keys of its own chunk only; the pages of chunks that lie behind are given back.  `distance_slopes` (one number a
query head): the score of key j seen from position p loses slope * (p - j), in float32 beside the scaled product.
`qk_norm_weight` False: the q/k norm has no weights (every head is divided by its root mean square and nothing else); the
norm then also works over a head that is padded, taking its mean over the head's own size.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import PagedKV
from .base import POSITION_ENCODINGS, Part, PartSpec, Rotary, Runtime, TensorSpec, register_mixer
from .linear import SplitSum, matmul, resolve

_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
          "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias",
          "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "sink": "sink", "head_gate": "gate"}


def _pad_heads(t: torch.Tensor, heads: int, size: int, to: int) -> torch.Tensor:
    """[heads * size, ...] -> [heads * to, ...] with zeros behind every head's rows."""
    if size == to:
        return t
    rest = t.shape[1:]
    out = torch.zeros((heads, to) + tuple(rest), dtype=t.dtype, device=t.device)
    out[:, :size] = t.reshape((heads, size) + tuple(rest))
    return out.reshape((heads * to,) + tuple(rest))


@register_mixer("paged_attention")
class PagedAttention(Part):
    graph_capturable = True
    accepts_normed_input = True         # `h` may be a `NormedInput`: the q|k|v product normalises it on the fly

    def __init__(self, rt: Runtime, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool, position: PartSpec, window: int | None = None, scale: float | None = None,
                 qk_norm_eps: float | None = None, v_head_dim: int | None = None, sink: bool = False,
                 names: dict | None = None, keep_first: int = 0, sink_value: float | None = None, head_gate: bool = False,
                 chunk: int | None = None, distance_slopes=None, qk_norm_weight: bool = True):
        super().__init__(rt)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        self.dk = head_dim
        self.dv = head_dim if v_head_dim is None else v_head_dim
        d = max(self.dk, self.dv)
        if not rt.exact:
            d = -(-d // 16) * 16                          # the bfloat16 attention kernels take multiples of 16
        else:
            d += d & 1                                    # the kernel that writes the pages works on pairs of dimensions
        if d != self.dk and qk_norm_eps is not None and qk_norm_weight:
            raise ValueError("a weighted q/k norm over a padded head is not supported")
        if chunk is not None and (window is not None or chunk < 1):
            raise ValueError("chunks are positive and stand instead of a window")
        if distance_slopes is not None and len(distance_slopes) != num_heads:
            raise ValueError(f"{len(distance_slopes)} distance slopes for {num_heads} query heads")
        self.chunk, self.qk_norm_weight = chunk, bool(qk_norm_weight)
        self.slopes = None if distance_slopes is None else \
            torch.tensor([float(v) for v in distance_slopes], dtype=torch.float32, device=rt.device)
        self.hidden, self.nq, self.nkv, self.d = hidden, num_heads, num_kv_heads, d
        self.qkv_bias, self.window = qkv_bias, window
        self.keep_first = int(keep_first) if window is not None else 0
        if sink and sink_value is not None:
            raise ValueError("a sink is either a tensor or a fixed number")
        self.sink_value, self.head_gate = sink_value, bool(head_gate)
        self.scale = head_dim ** -0.5 if scale is None else scale          # tensorline/paged.py:119
        self.position = POSITION_ENCODINGS.build(position, rt, head_dim=head_dim)
        self.qk_norm_eps = qk_norm_eps
        self.has_sink = bool(sink)
        self.names = {**_NAMES, **(names or {})}
        self.w_qkv = self.b_qkv = self.w_o = self.q_norm = self.k_norm = self.sink = self.w_gate = None

    def cache_need(self):
        return PagedKV(self.nkv, self.d, self.window, keep_first=self.keep_first, chunk=self.chunk)

    def expected_tensors(self, prefix):
        H, nq, nkv, dk, dv = self.hidden, self.nq, self.nkv, self.dk, self.dv
        n = {k: f"{prefix}.{v}" for k, v in self.names.items()}
        out = {n["q"]: TensorSpec((nq * dk, H)), n["k"]: TensorSpec((nkv * dk, H)),
               n["v"]: TensorSpec((nkv * dv, H)), n["o"]: TensorSpec((H, nq * dv))}
        if self.qkv_bias:
            out.update({n["q_bias"]: TensorSpec((nq * dk,)), n["k_bias"]: TensorSpec((nkv * dk,)),
                        n["v_bias"]: TensorSpec((nkv * dv,))})
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            out.update({n["q_norm"]: TensorSpec((dk,), init="ones"), n["k_norm"]: TensorSpec((dk,), init="ones")})
        if self.has_sink:
            out[n["sink"]] = TensorSpec((nq,))
        if self.head_gate:
            out[n["head_gate"]] = TensorSpec((nq, H))
        return out

    def bind(self, weights, prefix):
        nq, nkv, dk, dv, d = self.nq, self.nkv, self.dk, self.dv, self.d
        n = {k: f"{prefix}.{v}" for k, v in self.names.items()}
        heads = (("q", nq, dk), ("k", nkv, dk), ("v", nkv, dv))
        self.w_qkv = self._compute_copy(torch.cat([_pad_heads(weights[n[k]], h, size, d) for k, h, size in heads], dim=0))
        if self.qkv_bias:
            self.b_qkv = torch.cat([_pad_heads(weights[n[k + "_bias"]], h, size, d) for k, h, size in heads], dim=0).contiguous()
            if self.b_qkv.dtype not in (torch.float32, torch.bfloat16):
                self.b_qkv = self.b_qkv.float()
        w_o = weights[n["o"]]                            # [H, nq * dv]: zero columns behind every head's values
        if dv != d:
            w_o = _pad_heads(w_o.t().contiguous(), nq, dv, d).t()
        self.w_o = self._compute_copy(w_o)
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            self.q_norm = weights[n["q_norm"]].float().contiguous()
            self.k_norm = weights[n["k_norm"]].float().contiguous()
        elif self.qk_norm_eps is not None:
            self.q_norm = self.k_norm = torch.ones(d, dtype=torch.float32, device=self.w_o.device)
        if self.has_sink:
            self.sink = weights[n["sink"]].float().contiguous()
        elif self.sink_value is not None:
            self.sink = torch.full((nq,), float(self.sink_value), dtype=torch.float32, device=self.w_o.device)
        if self.head_gate:
            self.w_gate = weights[n["head_gate"]].contiguous()      # stored type; the gate's product accumulates in float32

    def forward(self, h, ctx, cache):
        nq, nkv, d = self.nq, self.nkv, self.d
        T = h.shape[0]
        gate = None
        if self.w_gate is not None:                      # one number per token and head, float32
            h = resolve(h)
            gate = torch.empty((T, nq), dtype=torch.float32, device=h.device)
            ops.small_proj(h, self.w_gate, None, gate)
        rotary = self.position.rotary()
        if not isinstance(rotary, Rotary):               # a plain (inv_freq, rot) pair means rotate-half pairing
            rotary = Rotary(*rotary)
        inv_freq, rot = rotary.inv_freq, rotary.rot
        plain = rotary.pairing == "half" and self.q_norm is None          # what the kernel's fast path covers
        qkv = matmul(h, self.w_qkv, may_defer=plain and rot == d and d % 16 == 0)
        pieces = None
        if isinstance(qkv, SplitSum):                    # a split-K product: the rotary kernel sums its pieces
            pieces = qkv.pieces
            qkv = torch.empty(qkv.shape, dtype=qkv.dtype, device=h.device)
        table = ctx.tables[cache.group]

        def rotary_kernel():
            ops.rope_kv_write(qkv, self.b_qkv, ctx.pos, ctx.req_slot, table, ctx.page_size, inv_freq, rot,
                              nq, nkv, d, cache.k, cache.v, write_kv=cache.owner, pieces=pieces, pairing=rotary.pairing,
                              q_norm=self.q_norm, k_norm=self.k_norm, norm_eps=self.qk_norm_eps or 0.0, norm_dim=self.dk)

        # A step of single tokens whose attention kernel can do bias, rotation and the page write of its own tokens
        # (the TMA decode kernel) needs no rotary kernel in front of it.
        fold = None
        if (ctx.decode_only and not ctx.force_exact_attention and qkv.dtype == torch.bfloat16 and pieces is None and plain
                and rot == d and self.sink is None and self._folds_rope(ctx)):
            fold = {"inv_freq": inv_freq, "bias": self.b_qkv, "write_kv": cache.owner, "unfold": rotary_kernel}
        else:
            rotary_kernel()
        o = torch.empty((T, nq * d), dtype=qkv.dtype, device=h.device)
        self.attend(qkv, o, ctx, cache, table, rope=fold, gate=gate)
        return matmul(o, self.w_o, may_defer=True, to_residual=True)     # the block's next norm adds it up

    def _folds_rope(self, ctx) -> bool:
        from .. import ops_attention
        return ops_attention.decode_takes_rope(ctx.B, self.d, ctx.page_size)

    def attend(self, qkv, o, ctx, cache, table, rope=None, gate=None):
        from . import attention_kernels
        attention_kernels.attend(self, qkv, o, ctx, cache, table, rope=rope, gate=gate)
