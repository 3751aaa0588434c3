"""The Sumuvik decoder as a `ModelSpec`.

The embedded tokens are multiplied by a constant.  Every layer is a parallel block: both sub-blocks read the same stream
through norms of their own (`norm1`, `norm2`: plain RMS norms in float32) and the stream takes the sum of their outputs.
A layer's mixer is either grouped-query attention (biases, interleaved rotary pairs over the first dimensions of a head
with stretched long wavelengths, a scale of its own, a sliding window that also keeps the first tokens of the sequence,
one more term exp(0) in every softmax denominator and a sigmoid gate per head on the way out) or the recurrent block of
Griffin (De et al., "Griffin: Mixing Gated Linear Recurrences with Local Attention for Efficient Language Models"): a
gelu branch beside a short causal convolution and the real-gated linear recurrent unit, whose gates are block-diagonal.
The feed-forward, where a layer has one, is a gated unit with a clamped swish, dense or as a mixture of experts whose
router scores are sigmoids, chosen with a correction and among the best groups of neighbouring experts only, weighted
by their share, beside a shared expert.  Tensor names: `embed`, `l<i>.norm1`, `l<i>.mix.*`, `l<i>.norm2`, `l<i>.mlp.*`,
`final.norm`, `head`, each tensor under its own name, biases with `.b`.
"""
from __future__ import annotations

from ..config.sumuvik import DenseSizes, SumuvikConfig
from ..parts import PartSpec
from .spec import LayerSpec, ModelSpec, RunEntry

_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "head_gate": "g"}
_GATE_UP_DOWN = {"gate": "gate", "up": "up", "down": "down"}
SWISH_ALPHA = 1.702                     # the design's constant in g * sigmoid(alpha g)
GROUP_SCORE_TOP = 2                     # a group of experts is judged by the sum of this many of its choice scores
RECURRENCE_SHARPNESS = 8.0              # log a = -sharpness * r * softplus(lam)


def describe_sumuvik(cfg: SumuvikConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("rms_norm", {"dim": W, "eps": eps, "tensor": "", "cast_first": False})
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "attention":
            s = m.rot.scaling
            scaling = None if s is None else {"factor": s.factor, "low": s.low, "high": s.high, "original": s.original}
            mixer = PartSpec("paged_attention", {
                "hidden": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                "qkv_bias": True, "scale": m.scale, "window": m.window, "keep_first": m.keep_first, "sink_value": 0.0,
                "head_gate": True, "names": _ATTENTION_NAMES,
                "position": PartSpec("rotary_interleaved", {"theta": m.rot.base, "rotary_dim": m.rot.dims, "scaling": scaling})})
        else:
            mixer = PartSpec("rglru", {"hidden": W, "width": m.width, "blocks": m.blocks, "taps": m.conv,
                                       "sharpness": RECURRENCE_SHARPNESS})
        ff = None
        if isinstance(layer.mlp, DenseSizes):
            ff = PartSpec("gated_mlp", {"hidden": W, "intermediate": layer.mlp.ff, "activation": "swish_clamped",
                                        "act_limit": layer.mlp.limit, "act_alpha": SWISH_ALPHA, "names": _GATE_UP_DOWN})
        elif layer.mlp is not None:
            f = layer.mlp
            ff = PartSpec("routed_experts", {
                "hidden": W, "inner": f.ff, "experts": f.experts, "top": f.top, "activation": "swish_clamped",
                "act_limit": f.limit, "act_alpha": SWISH_ALPHA, "gated": True, "router_bias": False,
                "scoring": "sigmoid_share", "correction": True, "groups": f.groups, "keep_groups": f.keep_groups,
                "group_score_top": GROUP_SCORE_TOP, "route_scale": f.scale,
                "shared_inner": None if f.shared is None else f.shared.ff, "shared_gate": False,
                "shared_act_limit": None if f.shared is None else f.shared.limit})
        block = PartSpec("parallel_residual", {"mixer": mixer, "feed_forward": ff, "norm1": norm, "norm2": norm,
                                               "names": {"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feed_forward": "mlp"}})
        layers.append(LayerSpec(block, f"l{i}"))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=W, layers=tuple(layers), run=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=norm, tie_word_embeddings=False, embedding_prefix="embed", final_norm_prefix="final.norm",
        head_prefix="head", embedding=PartSpec("token_table", {"tensor": "", "scale": cfg.embedding_scale}),
        head=PartSpec("linear", {"tensor": ""}))
