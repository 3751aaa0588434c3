"""Attention through a latent: the cache holds, per token, one normalised latent vector c and one rotated key part r.

    cq = norm(Wdq h; w_dq),  q = Wuq cq              per head [dk plain | dr to rotate]
    Wdkv h = [rank | dr]:    c = norm(first; w_dkv),  r = rot(rest, position)      one r for all heads
    k_head = Wuk_head c,  v_head = Wuv_head c
    score(t, j) = scale (q_plain . k_head(j) + rot(q_rot) . r(j)),  softmax over the window,  y = Wo [sum_j p_j v_head(j)]

Only c and r are cached.  The scores and the weighted sums are taken in the latent's space, which is the same arithmetic in
another order:  q_plain . (Wuk c) = (Wuk^T q_plain) . c  and  sum_j p_j Wuv c_j = Wuv (sum_j p_j c_j).  The pages then look
like ONE key/value head of size rank + dr (padded to what the attention kernels take) whose value is the key row itself, so
every paged attention kernel of the package serves this mixer unchanged (the value pages are the key pages: a token is
stored once); the output's first `rank` columns are sum_j p_j c_j, the rest is not read.  The two changes of space are
products per head (`ops.head_matmul`).  Norm statistics, angles, scores and softmax are float32 in both engines.

Options: `q_rank` None: the queries are one projection of the input (tensor `uq` [H (dk + dr), hidden]), there is no query
latent; the position encoding may pair (i, i + rot/2) or (2i, 2i + 1); `out_gate`: the heads' outputs, side by side, are
multiplied element by element by sigmoid(Wg h) (tensor `g` [H dv, hidden], float32 pre-activations: its rows ride in the
down product) before the output projection.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import PagedKV
from .base import POSITION_ENCODINGS, KVCacheView, Part, PartSpec, Rotary, Runtime, TensorSpec, register_mixer
from .linear import matmul, resolve

# from this many tokens on the bfloat16 engine takes the two products per head to the library (one batched product)
HEAD_PRODUCT_LIBRARY_MIN_TOKENS = 64

_NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "o": "o",
          "g": "g"}


@register_mixer("latent_attention")
class LatentAttention(Part):
    graph_capturable = True

    def __init__(self, rt: Runtime, hidden: int, num_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, q_rank: int | None,
                 kv_rank: int, scale: float, norm_eps: float, position: PartSpec, window: int | None = None,
                 names: dict | None = None, out_gate: bool = False):
        super().__init__(rt)
        self.hidden, self.H, self.dk, self.dr, self.dv = hidden, num_heads, head_dim, rot_dim, v_head_dim
        self.qr, self.rank, self.scale, self.eps, self.window = int(q_rank or 0), kv_rank, float(scale), float(norm_eps), window
        self.out_gate = bool(out_gate)
        d = kv_rank + rot_dim
        self.d = d if rt.exact else -(-d // 16) * 16     # the bfloat16 attention kernels take multiples of 16
        self.position = POSITION_ENCODINGS.build(position, rt, head_dim=rot_dim)
        self.names = {**_NAMES, **(names or {})}
        # what `attention_kernels.attend` reads of a mixer
        self.nq, self.nkv, self.sink = num_heads, 1, None
        self.w_down = self.w_uq = self.w_uk = self.w_uv = self.w_o = self.n_q = self.n_kv = None

    def cache_need(self):
        return PagedKV(1, self.d, self.window, shared_values=True)

    def expected_tensors(self, prefix):
        n = {k: f"{prefix}.{v}" for k, v in self.names.items()}
        W, H = self.hidden, self.H
        out = {n["uq"]: TensorSpec((H * (self.dk + self.dr), self.qr or W)),
               n["dkv"]: TensorSpec((self.rank + self.dr, W)), n["dkv_norm"]: TensorSpec((self.rank,), init="ones"),
               n["uk"]: TensorSpec((H * self.dk, self.rank)), n["uv"]: TensorSpec((H * self.dv, self.rank)),
               n["o"]: TensorSpec((W, H * self.dv))}
        if self.qr:
            out.update({n["dq"]: TensorSpec((self.qr, W)), n["dq_norm"]: TensorSpec((self.qr,), init="ones")})
        if self.out_gate:
            out[n["g"]] = TensorSpec((H * self.dv, W))
        return out

    def bind(self, weights, prefix):
        n = {k: f"{prefix}.{v}" for k, v in self.names.items()}
        H = self.H
        # the down product's float32 accumulators are kept as they are: they feed two norms
        down = ([weights[n["dq"]]] if self.qr else []) + [weights[n["dkv"]]] + ([weights[n["g"]]] if self.out_gate else [])
        self.w_down = self._compute_copy(torch.cat(down, dim=0))
        self.w_uq = self._compute_copy(weights[n["uq"]])
        self.w_uk = self._compute_copy(weights[n["uk"]].view(H, self.dk, self.rank))                       # [H, K = dk, N = rank]
        self.w_uv = self._compute_copy(weights[n["uv"]].view(H, self.dv, self.rank).transpose(1, 2))       # [H, K = rank, N = dv]
        self.w_o = self._compute_copy(weights[n["o"]])
        self.n_kv = weights[n["dkv_norm"]].contiguous()
        self.n_q = weights[n["dq_norm"]].to(self.n_kv.dtype).contiguous() if self.qr else None

    def forward(self, h, ctx, cache):
        H, d, dk, dr, rank = self.H, self.d, self.dk, self.dr, self.rank
        T = h.shape[0]
        act = self.rt.act_dtype
        rotary = self.position.rotary()
        if not isinstance(rotary, Rotary):
            rotary = Rotary(*rotary)
        table = ctx.tables[cache.group]
        h = resolve(h)
        down = self._down(h)
        cq = torch.empty((T, self.qr), dtype=act, device=down.device) if self.qr else None
        ops.latent_prep(down, self.qr, rank, dr, self.n_q, self.n_kv, self.eps, rotary.inv_freq, rotary.rot, ctx.pos, ctx.req_slot,
                        table, ctx.page_size, cq, cache.k, write_kv=cache.owner, pairing=rotary.pairing)
        q = resolve(matmul(cq if self.qr else h, self.w_uq))
        qa = torch.empty((T, H * d), dtype=act, device=q.device)
        self._per_head(q, self.w_uk, qa, dk, rank, dk + dr, d, ctx)
        ops.latent_qrot(q, dk, dr, rotary.inv_freq, rotary.rot, ctx.pos, qa, rank, H, pairing=rotary.pairing)
        o = torch.empty((T, H * d), dtype=act, device=q.device)
        from . import attention_kernels
        attention_kernels.attend(self, qa, o, ctx, KVCacheView(cache.k, cache.k, cache.group, cache.owner), table)
        ov = torch.empty((T, H * self.dv), dtype=act, device=q.device)
        self._per_head(o, self.w_uv, ov, rank, self.dv, d, self.dv, ctx)
        if self.out_gate:
            ops.sigmoid_gate(ov, down[:, self.qr + rank + dr:], ov)
        return matmul(ov, self.w_o)

    def _per_head(self, x, w, y, K, N, xs, ys, ctx):
        """y[t, h, :N] = x[t, h, :K] w[h] with the heads xs (ys) columns apart: the package's kernel, or for long bfloat16 steps
        one batched library product (as the engine's other long products are the library's)."""
        T, H = x.shape[0], self.H
        if x.dtype != torch.bfloat16 or T < HEAD_PRODUCT_LIBRARY_MIN_TOKENS or ctx.graph_max_ctx:
            ops.head_matmul(x, w, y, H, K, N, xs, ys)
            return
        out = torch.matmul(x.view(T, H, xs)[:, :, :K].transpose(0, 1), w)          # [H, T, N]
        y.view(T, H, ys)[:, :, :N].copy_(out.transpose(0, 1))
        ops.mark("library product")

    def _down(self, h):
        """[Wdq; Wdkv; Wg] h as float32 [T, qr + rank + dr (+ H dv)]."""
        return resolve(matmul(resolve(h), self.w_down, out_dtype=torch.float32))
