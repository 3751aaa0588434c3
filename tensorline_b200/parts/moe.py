"""Routed feed-forward (mixture of experts).

    z = h Wr^T + br                      router logits, float32 in both engines
    chosen: the `top` largest z;         weights = softmax over the chosen logits only
    y = sum_j weight_j * Wdown[e_j] act(Wup[e_j] h)          experts without biases, act = relu(.)^2

Options, all parameters of the one part: gated experts (`gated`: Wdown (act(Wgate x) * Wup x), tensors `gate`, `up`, `down`),
the activation (`relu_squared`, `silu`, `gelu_tanh`), the weights as the sigmoid of each chosen logit instead of the softmax
over the chosen (`scoring` "sigmoid": not renormalised), the weight on the expert's input instead of its output
(`weight_on` "input": y = sum_j expert_j(weight_j h), which differs because an expert is not linear), no router bias, and a
shared expert (`shared_inner`: one more gated unit of that size that every token runs, multiplied by sigmoid(w_sg . h), one
number a token; its row `sg` rides in the router's product; `shared_gate` False: added as it is; `shared_act_limit`: the
limit of its activation where that differs from the experts').

`scoring` "sigmoid_share" is the choice among groups: s = sigmoid(z); the choice scores are s + `correction` (a tensor of
one number an expert, `correction` True); the experts form `groups` equal groups of neighbours, a group's score is the sum
of its `group_score_top` largest choice scores, and only experts of the `keep_groups` best groups can be chosen (the
others count as minus infinity); the `top` largest choice scores among them are chosen, and their weights are their s
(without the correction) divided by the sum of the chosen s (+ 1e-20), times `route_scale`.  The activation
`swish_clamped` comes with `act_limit` and `act_alpha` (see parts/mlp.py).  `scoring` "softmax_share" is the same choice
with s = softmax(z) over all entries of the router.  `identity`: the router has that many entries behind the experts'
that stand for no matrices: an identity entry's output is the token's input itself (times its weight).

The experts' matrices are stacked ([E, F, K] and [E, K, F]) at load time.  Steps of few tokens stream, for every
(token, chosen expert) pair, that expert's rows (`ops.moe_up`, `ops.moe_down`): nothing is sorted and nothing comes
back to the host, so the step sits in a CUDA graph.  Steps of many tokens sort the pairs by expert on the device,
gather the tokens' rows in that order, every expert's run into `cap` rows of its own (the longest run, rounded up), and
run two batched dense products over all experts (the library's, as the engine's other long products are), which needs
the runs' bounds on the host.  The 32-bit engine streams always: a token's result is then the
same chain of additions in every step, whatever else the step holds.
"""
from __future__ import annotations

import os

import torch

from .. import ops
from .base import Part, Runtime, TensorSpec, register_feed_forward
from .linear import resolve

# up to this many tokens a step the experts are streamed pair by pair
STREAM_MAX_TOKENS = int(os.environ.get("TENSORLINE_B200_MOE_STREAM_MAX_TOKENS", 32))


@register_feed_forward("routed_experts")
class RoutedExperts(Part):
    graph_capturable = True              # a captured step streams the experts whatever its size (see forward)

    def __init__(self, rt: Runtime, hidden: int, inner: int, experts: int, top: int, activation: str = "relu_squared",
                 router_bias: bool = True, names: dict | None = None, gated: bool = False, scoring: str = "softmax_chosen",
                 weight_on: str = "output", shared_inner: int | None = None, shared_gate: bool = True,
                 act_limit: float | None = None, act_alpha: float = 1.0, shared_act_limit: float | None = None,
                 correction: bool = False, groups: int = 1, keep_groups: int = 1, group_score_top: int = 2,
                 route_scale: float = 1.0, identity: int = 0):
        super().__init__(rt)
        if activation not in ops.GATE_ACTS:
            raise ValueError(f"routed_experts runs one of {sorted(ops.GATE_ACTS)}, not {activation!r}")
        if scoring not in ("softmax_chosen", "sigmoid", "sigmoid_share", "softmax_share") or weight_on not in ("output", "input"):
            raise ValueError(f"routed_experts: scoring {scoring!r} / weight_on {weight_on!r} are not known")
        if identity < 0 or (identity and (scoring not in ("sigmoid_share", "softmax_share") or weight_on != "output")):
            raise ValueError("routed_experts: identity entries go with a share scoring and weights on the output")
        experts_real, experts = experts, experts + identity          # below, `experts` counts the router's entries
        if not 1 <= top <= min(experts, 32) or experts > 1024:
            raise ValueError(f"routed_experts: top {top} of {experts} experts is outside what the choice kernel takes")
        if (activation == "swish_clamped") != (act_limit is not None) or (activation == "swish_clamped" and not gated):
            raise ValueError("routed_experts: 'swish_clamped' is a gated unit and comes with act_limit, and only it")
        grouped = scoring in ("sigmoid_share", "softmax_share")
        if not grouped and (correction or groups != 1 or route_scale != 1.0):
            raise ValueError("routed_experts: a correction, groups and a scale of the weights belong to scoring 'sigmoid_share'")
        if grouped and (groups < 1 or experts % groups or not 1 <= keep_groups <= groups or group_score_top < 1
                        or top > keep_groups * (experts // groups)):
            raise ValueError(f"routed_experts: {experts} experts in {groups} groups, {keep_groups} kept, top {top}")
        self.hidden, self.inner, self.E, self.top, self.router_bias = hidden, inner, experts, top, router_bias
        self.E_real = experts_real
        self.activation, self.gated, self.scoring, self.weight_on = activation, bool(gated), scoring, weight_on
        self.act = activation if act_limit is None else (activation, float(act_limit), float(act_alpha))
        self.has_correction, self.groups, self.keep_groups = bool(correction), int(groups), int(keep_groups)
        self.group_score_top, self.route_scale = int(group_score_top), float(route_scale)
        self.names = {"router": "router", "router_bias": "router.b", "expert": "e{}", "up": "up", "down": "down", "gate": "gate",
                      "shared": "shared", "shared_gate": "shared.sg", "correction": "correction", **(names or {})}
        self.shared = None
        self.shared_gate = bool(shared_gate) and shared_inner is not None
        self.correction = None
        if shared_inner is not None:
            from .mlp import GatedMLP
            limit = act_limit if shared_act_limit is None else shared_act_limit
            self.shared = GatedMLP(rt, hidden, shared_inner, activation, {k: self.names[k] for k in ("gate", "up", "down")},
                                   act_limit=limit, act_alpha=act_alpha)
        self.w_router = self.b_router = self.w_up = self.w_down = None

    def _expert(self, prefix, e, which):
        return f"{prefix}.{self.names['expert'].format(e)}.{self.names[which]}"

    def expected_tensors(self, prefix):
        out = {f"{prefix}.{self.names['router']}": TensorSpec((self.E, self.hidden))}
        if self.router_bias:
            out[f"{prefix}.{self.names['router_bias']}"] = TensorSpec((self.E,))
        for e in range(self.E_real):
            if self.gated:
                out[self._expert(prefix, e, "gate")] = TensorSpec((self.inner, self.hidden))
            out[self._expert(prefix, e, "up")] = TensorSpec((self.inner, self.hidden))
            out[self._expert(prefix, e, "down")] = TensorSpec((self.hidden, self.inner))
        if self.shared is not None:
            out.update(self.shared.expected_tensors(f"{prefix}.{self.names['shared']}"))
            if self.shared_gate:
                out[f"{prefix}.{self.names['shared_gate']}"] = TensorSpec((1, self.hidden))
        if self.has_correction:
            out[f"{prefix}.{self.names['correction']}"] = TensorSpec((self.E,))
        return out

    def bind(self, weights, prefix):
        w_router = weights[f"{prefix}.{self.names['router']}"]
        if self.router_bias:
            self.b_router = weights[f"{prefix}.{self.names['router_bias']}"].to(w_router.dtype)
        if self.shared is not None:                      # the shared expert's gate is one more row of the router's product
            self.shared.bind(weights, f"{prefix}.{self.names['shared']}")
        if self.has_correction:
            self.correction = weights[f"{prefix}.{self.names['correction']}"].float().contiguous()
        if self.shared_gate:
            w_router = torch.cat([w_router, weights[f"{prefix}.{self.names['shared_gate']}"].to(w_router.dtype).view(1, -1)])
            if self.b_router is not None:
                self.b_router = torch.cat([self.b_router, self.b_router.new_zeros(1)])
        self.w_router = w_router.contiguous()
        if self.b_router is not None:
            self.b_router = self.b_router.contiguous()

        def stacked(e):                                  # a gated expert: its gate rows, then its up rows
            up = weights[self._expert(prefix, e, "up")]
            return torch.cat([weights[self._expert(prefix, e, "gate")], up]) if self.gated else up

        self.w_up = self._compute_copy(torch.stack([stacked(e) for e in range(self.E_real)]))
        self.w_down = self._compute_copy(torch.stack([weights[self._expert(prefix, e, "down")] for e in range(self.E_real)]))

    def forward(self, h, ctx):
        h = resolve(h)
        T, top, E = h.shape[0], self.top, self.E
        z = torch.empty((T, self.w_router.shape[0]), dtype=torch.float32, device=h.device)
        ops.small_proj(h, self.w_router, self.b_router, z)
        idx = torch.empty((T, top), dtype=torch.int32, device=h.device)
        wts = torch.empty((T, top), dtype=torch.float32, device=h.device)
        if self.scoring in ("sigmoid_share", "softmax_share"):
            ops.route_groups(z[:, :E], self.correction, top, self.groups, self.keep_groups, self.group_score_top, self.route_scale,
                             idx, wts, softmax=self.scoring == "softmax_share")
        else:
            ops.topk_softmax(z[:, :E], top, idx, wts, scoring=self.scoring)
        extra = extra_gate = None
        if self.shared is not None:
            extra, extra_gate = resolve(self.shared.forward(h, ctx)), (z[:, E] if self.shared_gate else None)
        on_input = self.weight_on == "input"
        y = torch.empty((T, self.hidden), dtype=h.dtype, device=h.device)
        if T <= STREAM_MAX_TOKENS or ctx.graph_max_ctx or self.rt.exact:
            a = torch.empty((T * top, self.inner), dtype=h.dtype, device=h.device)
            ops.moe_up(h, self.w_up, idx, a, act=self.act, gated=self.gated, in_scale=wts if on_input else None)
            ops.moe_down(a, self.w_down, idx, None if on_input else wts, y, extra=extra, extra_gate=extra_gate,
                         same=h if self.E_real < E else None)
            return y
        offsets, place_of, pair_at = ops.moe_sort(idx, E)
        bounds = offsets.tolist()                        # the one read-back of the step: where every expert's run ends
        longest = max(bounds[e + 1] - bounds[e] for e in range(E))
        cap = -(-longest // 64) * 64                     # rows every expert gets in the batched products
        rows = torch.empty((E * cap, self.hidden), dtype=h.dtype, device=h.device)
        ops.moe_gather(h, pair_at, idx, offsets, top, rows, cap=cap, scale=wts.view(-1) if on_input else None)
        R = self.E_real                                  # the entries behind it are identities: their rows pass as they are
        inner = torch.bmm(rows.view(E, cap, self.hidden)[:R], self.w_up.transpose(1, 2))         # [R, cap, F] or [R, cap, 2F]
        ops.mark("library product")
        if self.gated:
            act = torch.empty((R * cap, self.inner), dtype=h.dtype, device=h.device)
            ops.silu_mul(inner.view(R * cap, 2 * self.inner), act, act=self.act)
            inner = act.view(R, cap, self.inner)
        elif self.activation == "relu_squared":
            ops.relu_square(inner)
        else:
            raise NotImplementedError(f"long steps of experts without a gate run 'relu_squared', not {self.activation!r}")
        if R < E:
            outs = torch.empty((E, cap, self.hidden), dtype=h.dtype, device=h.device)
            torch.bmm(inner, self.w_down.transpose(1, 2), out=outs[:R])
            outs[R:].copy_(rows.view(E, cap, self.hidden)[R:])
        else:
            outs = torch.bmm(inner, self.w_down.transpose(1, 2))                                # [E, cap, K]
        ops.mark("library product")
        ops.moe_combine(outs.view(E * cap, self.hidden), place_of, idx, offsets, None if on_input else wts, y, cap=cap,
                        extra=extra, extra_gate=extra_gate)
        return y
