"""The recurrent block with a real-gated linear recurrent unit (De et al., "Griffin: Mixing Gated Linear Recurrences with
Local Attention for Efficient Language Models").

    y = gelu_tanh(Wy h + by)                                     one branch, `width` channels
    u = conv(Wx h + bx)                                          the other: a causal convolution over time per channel (`taps`
                                                                 weights, the last on the current token, zeros before the start,
                                                                 a bias, no activation)
    r = sigmoid(Ra[b] u_b + ra_b),  i = sigmoid(Ri[b] u_b + ri_b)     u cut into `blocks` equal parts, a square matrix each
    log a = -sharpness * r * softplus(lam),  a = exp(log a)
    S <- a S + sqrt(1 - a^2) * i * u                             per channel, from S = 0, the first token like every other
    out = Wo (S * y)

Between steps a request keeps, in its state slots, S (float32 [width]) and the convolution's last `taps - 1` inputs
(float32); both start at zero.  Everything behind the two projections is float32 in both engines: the projections'
float32 accumulators are kept as they are, the gates' products, the decay and the state never leave float32.  The bfloat16
engine runs a long step's recurrence as chunks side by side (`ops.rglru_scan`); the float32 engine walks every step in
order, so that its results are the same floats however a prompt was cut.  The mixer
reads the step from device tensors only (single-token steps sit in CUDA graphs).
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import SlotState
from .base import Part, Runtime, TensorSpec, register_mixer
from .linear import matmul, resolve

# From this many tokens a bfloat16 step takes the gates' products, which are float32 products of a float32 input, as one
# batched library product on the tensor cores (the engine's other long products are the library's too) of the input cut
# into three bfloat16 parts; shorter steps and the float32 engine use the package's float32 kernel.
GATE_PRODUCT_LIBRARY_MIN_TOKENS = 256

_NAMES = {"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv": "conv", "conv_bias": "conv.b", "ra": "ra", "ra_bias": "ra.b",
          "ri": "ri", "ri_bias": "ri.b", "lam": "lam", "o": "o"}


@register_mixer("rglru")
class RGLRU(Part):
    graph_capturable = True

    def __init__(self, rt: Runtime, hidden: int, width: int, blocks: int, taps: int, sharpness: float = 8.0,
                 names: dict | None = None):
        super().__init__(rt)
        if width % blocks:
            raise ValueError(f"{width} channels are not a multiple of {blocks} blocks")
        if taps < 1:
            raise ValueError("the convolution needs at least one tap")
        self.hidden, self.W, self.blocks, self.taps, self.sharpness = hidden, width, blocks, taps, float(sharpness)
        self.bw = width // blocks
        self.names = {**_NAMES, **(names or {})}
        self.w_in = self.b_in = self.conv_w = self.conv_b = self.w_gates = self.w_gates3 = self.b_gates = self.lam = self.w_o = None

    def cache_need(self):
        need = {"memory": SlotState((self.W,), "float32")}
        if self.taps > 1:
            need["inputs"] = SlotState(((self.taps - 1) * self.W,), "float32")
        return need

    def expected_tensors(self, prefix):
        n = {k: f"{prefix}.{v}" for k, v in self.names.items()}
        H, W, nb, bw = self.hidden, self.W, self.blocks, self.bw
        return {n["y"]: TensorSpec((W, H)), n["y_bias"]: TensorSpec((W,)), n["x"]: TensorSpec((W, H)), n["x_bias"]: TensorSpec((W,)),
                n["conv"]: TensorSpec((W, self.taps)), n["conv_bias"]: TensorSpec((W,)),
                n["ra"]: TensorSpec((nb, bw, bw)), n["ra_bias"]: TensorSpec((nb, bw)),
                n["ri"]: TensorSpec((nb, bw, bw)), n["ri_bias"]: TensorSpec((nb, bw)),
                n["lam"]: TensorSpec((W,)), n["o"]: TensorSpec((H, W))}

    def bind(self, weights, prefix):
        n = {k: f"{prefix}.{v}" for k, v in self.names.items()}
        # one stacked projection: the gelu branch's rows, then the recurrent branch's
        self.w_in = self._compute_copy(torch.cat([weights[n["y"]], weights[n["x"]]], dim=0))
        self.b_in = torch.cat([weights[n["y_bias"]], weights[n["x_bias"]]]).float().contiguous()
        self.conv_w = weights[n["conv"]].float().contiguous()
        self.conv_b = weights[n["conv_bias"]].float().contiguous()
        # the gates' matrices per block as [in, r outputs | i outputs], in their stored type (products and sums are float32)
        self.w_gates = torch.cat([weights[n["ra"]].transpose(1, 2), weights[n["ri"]].transpose(1, 2)], dim=2).contiguous()
        # for long bfloat16 steps: the same three times over the input side, for the three parts of a float (`ops.split3`)
        self.w_gates3 = self.w_gates.repeat(1, 3, 1).contiguous() if self.w_gates.dtype == torch.bfloat16 else None
        self.b_gates = torch.cat([weights[n["ra_bias"]], weights[n["ri_bias"]]], dim=1).float().contiguous()      # [blocks, 2 bw]
        self.lam = weights[n["lam"]].float().contiguous()
        self.w_o = self._compute_copy(weights[n["o"]])

    def forward(self, h, ctx, cache):
        W, nb, bw = self.W, self.blocks, self.bw
        h = resolve(h)
        T = h.shape[0]
        proj = resolve(matmul(h, self.w_in, out_dtype=torch.float32))           # y | x before their biases, float32 accumulators
        u = torch.empty((T, W), dtype=torch.float32, device=h.device)
        inputs = cache["inputs"].state if self.taps > 1 else None
        ops.causal_conv(proj, W, self.b_in, W, self.conv_w, self.conv_b, inputs, ctx.q_start, ctx.slots, u, B=ctx.B,
                        max_q_len=ctx.max_q_len)
        by_block = h.dtype == torch.bfloat16 and T >= GATE_PRODUCT_LIBRARY_MIN_TOKENS and self.w_gates3 is not None and \
            not ctx.graph_max_ctx
        if by_block:                                     # one batched library product of the floats' three bfloat16 parts
            gates = torch.bmm(ops.split3(u, nb), self.w_gates3, out_dtype=torch.float32)        # [blocks, T, 2 bw]
            ops.mark("library product")
        else:
            gates = torch.empty((T, 2 * W), dtype=torch.float32, device=h.device)    # per block: r pre-activations, then i
            ops.head_matmul(u, self.w_gates, gates, nb, bw, 2 * bw, bw, 2 * bw)
        out = torch.empty((T, W), dtype=h.dtype, device=h.device)
        ops.rglru_scan(gates, self.b_gates, u, proj, self.b_in, self.lam, cache["memory"].state, ctx.q_start, ctx.slots, out,
                       B=ctx.B, blocks=nb, sharpness=self.sharpness, max_q_len=ctx.max_q_len, in_order=h.dtype == torch.float32,
                       by_block=by_block)
        return matmul(out, self.w_o, may_defer=True, to_residual=True)
