"""The Tenalorn decoder as a `ModelSpec`.

The embedded tokens are multiplied by a constant and take a row of a hashed table of token pairs (previous token, token).
The residual stream is kept as `streams` copies (hyper-connections: Zhu et al., "Hyper-Connections"): every sublayer reads a
learned combination of the copies through its norm (`norm1`, `norm2`: plain RMS norms in float32), and every copy then
becomes a learned combination of the old copies plus a learned multiple of the sublayer's output (`hc1.*`, `hc2.*`); the
model's norm reads their sum.  Without `streams` a layer is the ordinary pre-norm block.  A layer's mixer is either a pair
side by side, added with fixed weights: grouped-query attention without rotation whose q and k heads are divided by their
root mean square, whose scores lose a fixed slope per head times the distance to the key and whose queries see their own
chunk of the sequence only, beside the matrix memory of the xLSTM (Beck et al., "xLSTM: Extended Long Short-Term Memory");
or attention through a latent (a normalised latent and one rotated key part a token in the cache, interleaved rotary pairs)
with a sigmoid gate on the heads' outputs.  The feed-forward is a mixture of gated silu experts chosen by softmax scores plus
a correction, weighted by their share; the router's last entries are identity experts whose output is their input; a shared
expert runs for every token.  The logits pass cap * tanh(. / cap).  Tensor names: `embed`, `bigram`, `l<i>.norm1`,
`l<i>.hc1.*`, `l<i>.mix.*`, `l<i>.norm2`, `l<i>.hc2.*`, `l<i>.mlp.*`, `final.norm`, `head`, each tensor under its own name,
biases with `.b`.
"""
from __future__ import annotations

from ..config.tenalorn import TenalornConfig
from ..parts import PartSpec
from .spec import LayerSpec, ModelSpec, RunEntry

_QKVO = {"q": "q", "k": "k", "v": "v", "o": "o"}
SLOPE_EXPONENT = 8.0                    # head a of H loses 2^(-SLOPE_EXPONENT (a + 1) / H) a position of distance
DENOMINATOR_EPS = 1e-6                  # the matrix memory's o = S^T q / (max(|n . q|, exp(-m)) + this)


def distance_slopes(heads: int) -> list:
    return [2.0 ** (-SLOPE_EXPONENT * (a + 1) / heads) for a in range(heads)]


def describe_tenalorn(cfg: TenalornConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("rms_norm", {"dim": W, "eps": eps, "tensor": "", "cast_first": False})
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "parallel":
            a, b = m.left, m.right
            left = PartSpec("paged_attention", {
                "hidden": W, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
                "qkv_bias": False, "scale": a.scale, "chunk": a.chunk, "distance_slopes": distance_slopes(a.heads),
                "qk_norm_eps": eps, "qk_norm_weight": False, "names": _QKVO, "position": PartSpec("none")})
            right = PartSpec("mlstm", {"hidden": W, "num_heads": b.heads, "head_dim": b.dim, "v_head_dim": b.vdim,
                                       "gate_cap": b.gate_cap, "norm_eps": eps, "den_eps": DENOMINATOR_EPS})
            mixer = PartSpec("parallel_pair", {"hidden": W, "left": left, "right": right, "norm_eps": eps, "normed": False,
                                               "left_scale": m.left_scale, "right_scale": m.right_scale})
        else:
            mixer = PartSpec("latent_attention", {
                "hidden": W, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim,
                "q_rank": None, "kv_rank": m.kv_rank, "scale": m.scale, "norm_eps": eps, "out_gate": True, "names": {"uq": "q"},
                "position": PartSpec("rotary_interleaved", {"theta": m.rot.base, "rotary_dim": m.rot.dims})})
        ff = None
        if layer.mlp is not None:
            f = layer.mlp
            ff = PartSpec("routed_experts", {
                "hidden": W, "inner": f.ff, "experts": f.experts, "identity": f.identity, "top": f.top, "activation": "silu",
                "gated": True, "router_bias": False, "scoring": "softmax_share", "correction": True,
                "shared_inner": f.shared_ff, "shared_gate": False})
        names = {"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feed_forward": "mlp"}
        if cfg.streams is None:
            block = PartSpec("pre_norm", {"mixer": mixer, "feed_forward": ff, "norm1": norm, "norm2": norm, "names": names})
        else:
            block = PartSpec("hyper_connections", {"mixer": mixer, "feed_forward": ff, "norm1": norm, "norm2": norm,
                                                   "streams": cfg.streams, "names": names})
        layers.append(LayerSpec(block, f"l{i}"))
    if cfg.pairs is None:
        embedding = PartSpec("token_table", {"tensor": "", "scale": cfg.embedding_scale})
    else:
        embedding = PartSpec("token_pairs", {"tensor": "", "scale": cfg.embedding_scale, "buckets": cfg.pairs.buckets,
                                             "mul_prev": cfg.pairs.mul_prev, "mul_cur": cfg.pairs.mul_cur, "pairs_tensor": "bigram"})
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=W, layers=tuple(layers), run=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=norm, tie_word_embeddings=False, embedding_prefix="embed", final_norm_prefix="final.norm",
        head_prefix="head", embedding=embedding, head=PartSpec("linear", {"tensor": "", "softcap": cfg.logit_softcap}),
        streams=cfg.streams or 1)
