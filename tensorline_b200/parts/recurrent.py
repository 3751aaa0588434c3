"""Mixers that carry a matrix per head from token to token instead of keys and values.

    S_t = a_t S_(t-1) + b_t k_t v_t^T,    o_t = S_t^T q_t          S: [d, dv] per head, float32

Two kinds, one pipeline (one stacked projection, one scan kernel, one kernel for the per-head norm and the
gate, the output projection):

* `retention`: a_t is a fixed decay per head, b_t = 1; q and k are rotated by position and k is scaled by
  d^-1/2 after the rotation; every head's o is divided by its root mean square (no weight), multiplied by
  silu(g) with g one more projection of the input, and projected.
* `mlstm` (the matrix memory of the xLSTM: Beck et al., "xLSTM: Extended Long Short-Term Memory"): per head a
  log input gate i_t = cap tanh(x_i / cap) and a log forget gate f_t = logsigmoid(cap tanh(x_f / cap)) from two
  small projections with bias, stabilised by a running maximum m_t = max(f_t + m_(t-1), i_t) that starts at 0:
  a_t = exp(f_t + m_(t-1) - m_t), b_t = exp(i_t - m_t); a normaliser n_t follows the same recurrence with k
  alone, and o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6) with q scaled by d^-1/2.  Every head's o
  is divided by its root mean square, multiplied by a weight over all heads, by sigmoid(g), and projected.

The state lives in the request's state slot (`SlotState`), in float32, zero for a new request (which is also
m_0 = 0), in the scan kernel's own layout; the gates' pre-activations, the rotation, the exponentials and the
norms are float32 in both engines, and q, k, v and g are the stacked projection's float32 results (bfloat16 inputs and
weights in the bfloat16 engine, accumulated and kept in float32).
The mixers read the step from device tensors only, so steps of single tokens are captured in CUDA graphs.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import SlotState
from .base import POSITION_ENCODINGS, Part, PartSpec, Rotary, Runtime, TensorSpec, register_mixer
from .linear import matmul, resolve


class _MatrixState(Part):
    graph_capturable = True
    gated = False
    gate_act = "silu"

    def __init__(self, rt: Runtime, hidden: int, num_heads: int, head_dim: int, v_head_dim: int, norm_eps: float,
                 position: PartSpec | None = None, names: dict | None = None):
        super().__init__(rt)
        self.hidden, self.H, self.d, self.dv, self.eps = hidden, num_heads, head_dim, v_head_dim, norm_eps
        if head_dim > 256:
            raise ValueError(f"head_dim {head_dim}: the scan kernel keeps at most 256 rows of state a head")
        self.position = POSITION_ENCODINGS.build(position or PartSpec("none"), rt, head_dim=head_dim)
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", **(names or {})}
        self.w_in = self.w_o = None

    # -- state
    def _slices(self) -> int:
        return -(-self.dv // 16)                         # value columns a block of the scan kernel: ops.scan_columns()

    def _state_floats(self) -> int:
        """Floats a (head, slice) of the scan kernel keeps, as `ops.scan_state_floats` says on the device: R rows in each
        of its threads (IS threads a column, 16 columns and the normaliser's), then m."""
        rows, per_column = (4, 8) if self.d <= 32 else (8, 8) if self.d <= 64 else (8, 16) if self.d <= 128 else (8, 32)
        threads = -(-per_column * (17 if self.gated else 16) // 32) * 32
        return rows * threads + (4 if self.gated else 0)

    def cache_need(self):
        return SlotState((self.H * self._slices() * self._state_floats(),), "float32")

    # -- tensors
    def _projections(self):
        H, d, dv = self.H, self.d, self.dv
        return (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv))

    def expected_tensors(self, prefix):
        n = self.names
        out = {f"{prefix}.{n[k]}": TensorSpec((rows, self.hidden)) for k, rows in self._projections()}
        out[f"{prefix}.{n['o']}"] = TensorSpec((self.hidden, self.H * self.dv))
        return out

    def bind(self, weights, prefix):
        n = self.names
        self.w_in = self._compute_copy(torch.cat([weights[f"{prefix}.{n[k]}"] for k, _ in self._projections()], dim=0))
        self.w_o = self._compute_copy(weights[f"{prefix}.{n['o']}"])
        if self.rt.device.type == "cuda":
            if ops.scan_columns() != 16 or ops.scan_state_floats(self.d, self.gated) != self._state_floats():
                raise ops.KernelError("the scan kernel's state layout is not the one this mixer sizes its slots for")

    # -- one step
    def _scan(self, h, proj, ctx, state, o):
        raise NotImplementedError

    def _head_weight(self):
        return None

    def forward(self, h, ctx, cache):
        H, d, dv = self.H, self.d, self.dv
        T = h.shape[0]
        # q, k, v and g stay as the product accumulated them, in float32: what enters the recurrence is not rounded again
        # (rounding q and k to bfloat16 alone moved the logits of a small model by several per cent where n . q or
        # S^T q nearly cancel)
        proj = resolve(matmul(h, self.w_in, out_dtype=torch.float32))
        o = torch.empty((T, H * dv), dtype=torch.float32, device=h.device)
        self._scan(h, proj, ctx, cache.state, o)
        y = torch.empty((T, H * dv), dtype=h.dtype, device=h.device)
        ops.head_norm_gate(o, y, H, dv, self.eps, weight=self._head_weight(), gate=proj, gate_off=2 * H * d + H * dv,
                           act=self.gate_act)
        return matmul(y, self.w_o)


@register_mixer("retention")
class Retention(_MatrixState):
    def __init__(self, rt: Runtime, hidden: int, num_heads: int, head_dim: int, v_head_dim: int, decay, norm_eps: float,
                 position: PartSpec | None = None, names: dict | None = None):
        super().__init__(rt, hidden, num_heads, head_dim, v_head_dim, norm_eps, position, names)
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decays for {num_heads} heads")
        self.decay = torch.tensor([float(x) for x in decay], dtype=torch.float32, device=rt.device)

    def _scan(self, h, proj, ctx, state, o):
        H, d, dv = self.H, self.d, self.dv
        rotary = self.position.rotary()
        if not isinstance(rotary, Rotary):
            rotary = Rotary(*rotary)
        ops.linear_scan(proj, 0, H * d, 2 * H * d, H, d, dv, state, ctx.q_start, ctx.slots, ctx.pos, o, B=ctx.B,
                        decay=self.decay, inv_freq=rotary.inv_freq, rot=rotary.rot, pairing=rotary.pairing,
                        k_scale=d ** -0.5, single_tokens=ctx.decode_only)


@register_mixer("mlstm")
class MLSTM(_MatrixState):
    gated = True
    gate_act = "sigmoid"

    def __init__(self, rt: Runtime, hidden: int, num_heads: int, head_dim: int, v_head_dim: int, gate_cap: float,
                 norm_eps: float, names: dict | None = None, den_eps: float = 1e-6):
        super().__init__(rt, hidden, num_heads, head_dim, v_head_dim, norm_eps, None,
                         {"i": "i", "i_bias": "i.b", "f": "f", "f_bias": "f.b", "norm": "norm", **(names or {})})
        self.cap, self.den_eps = float(gate_cap), float(den_eps)
        self.w_gates = self.b_gates = self.head_weight = None

    def expected_tensors(self, prefix):
        n, H = self.names, self.H
        out = super().expected_tensors(prefix)
        out.update({f"{prefix}.{n['i']}": TensorSpec((H, self.hidden)), f"{prefix}.{n['i_bias']}": TensorSpec((H,)),
                    f"{prefix}.{n['f']}": TensorSpec((H, self.hidden)), f"{prefix}.{n['f_bias']}": TensorSpec((H,)),
                    f"{prefix}.{n['norm']}": TensorSpec((H * self.dv,), init="ones")})
        return out

    def bind(self, weights, prefix):
        super().bind(weights, prefix)
        n = self.names
        w = torch.cat([weights[f"{prefix}.{n['i']}"], weights[f"{prefix}.{n['f']}"]], dim=0)
        b = torch.cat([weights[f"{prefix}.{n['i_bias']}"], weights[f"{prefix}.{n['f_bias']}"]], dim=0)
        self.w_gates = w.contiguous()                    # stored type; the gates' product accumulates and stays in float32
        self.b_gates = b.to(w.dtype).contiguous()
        self.head_weight = weights[f"{prefix}.{n['norm']}"].contiguous()

    def _head_weight(self):
        return self.head_weight

    def _scan(self, h, proj, ctx, state, o):
        H, d, dv = self.H, self.d, self.dv
        gates = torch.empty((h.shape[0], 2 * H), dtype=torch.float32, device=h.device)
        ops.small_proj(h, self.w_gates, self.b_gates, gates)
        ops.linear_scan(proj, 0, H * d, 2 * H * d, H, d, dv, state, ctx.q_start, ctx.slots, ctx.pos, o, B=ctx.B,
                        gates=gates, cap=self.cap, q_scale=d ** -0.5, den_eps=self.den_eps, single_tokens=ctx.decode_only)
