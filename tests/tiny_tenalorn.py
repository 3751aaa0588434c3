"""Tiny Tenalorn configurations of the tests and a helper that writes their model folders.

N1 to N6 differ in every size and option: two to five copies of the residual stream, one copy, and no copies at all (the
plain pre-norm block); with and without the table of token pairs and the cap on the logits; grouped and ungrouped heads,
value heads wider and narrower than query heads, head sizes that are no multiples of 16; chunks that are no multiples of
the page, of one page, of a single position, and no chunks; latents with a rotation over all, part or none of the shared
key part; routers with none to several identity entries, every entry chosen, with and without a shared expert; layers
without a feed-forward; pairs only; odd head sizes.  The attention scales are large, so that a softmax is
decided by few keys and a key that is wrongly seen (or not seen) shows; the forget gates of the matrix memory lie near
one, so that a lost or stale state shows many tokens later.
"""
from __future__ import annotations

import tempfile
from pathlib import Path

import torch

from tensorline_b200.config.tenalorn import TenalornConfig
from tensorline_b200.models import expected_tensors
from tensorline_b200.weights import write_random_model
from tensorline_b200.weights.safetensors_io import SafetensorsFile, write_safetensors


def _pair(heads, kv, dim, vdim, scale, chunk, rheads, rdim, rvdim, cap, ls, rs):
    left = {"dim": dim, "heads": heads, "kv_heads": kv, "scale": scale, "vdim": vdim}
    if chunk is not None:
        left["mask"] = {"size": chunk}
    return {"left": left, "left_scale": ls, "right": {"dim": rdim, "gate_cap": cap, "heads": rheads, "vdim": rvdim}, "right_scale": rs}


def _latent(heads, dim, rot_dim, vdim, rank, scale, base=None, dims=None):
    m = {"dim": dim, "heads": heads, "kv_rank": rank, "rot_dim": rot_dim, "scale": scale, "vdim": vdim}
    if rot_dim:
        m["rot"] = {"base": base, "dims": dims}
    return m


def _moe(ff, experts, identity, top, shared=None):
    out = {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "identity": identity, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def _model(vocab, width, eps, emb, layers, streams=None, pairs=None, cap=None):
    e = {"scale": emb}
    if pairs is not None:
        e["bigram"] = dict(zip(("buckets", "mul_cur", "mul_prev"), pairs))
    out = {"architecture": "Tenalorn", "embedding": e, "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if streams is not None:
        out["streams"] = streams
    if cap is not None:
        out["logit_softcap"] = cap
    return out


N1 = _model(131, 48, 1e-6, 3.0, [
    {"type": "parallel", "mixer": _pair(6, 2, 16, 24, 0.9, 11, 3, 8, 16, 10.0, 1.3, 0.6), "mlp": _moe(24, 6, 2, 3, 16)},
    {"type": "latent_attention", "mixer": _latent(3, 8, 8, 12, 20, 0.7, 100.0, 4), "mlp": _moe(20, 4, 1, 2)},
    {"type": "parallel", "mixer": _pair(2, 2, 32, 16, 0.25, 19, 2, 24, 8, 6.0, 0.8, 1.1), "mlp": None},
    {"type": "latent_attention", "mixer": _latent(4, 16, 4, 8, 12, 0.4, 10000.0, 4), "mlp": _moe(8, 3, 0, 3, 24)},
], streams=3, pairs=(61, 7, 13), cap=20.0)
N2 = _model(90, 72, 1e-5, 0.5, [
    {"type": "latent_attention", "mixer": _latent(2, 24, 16, 40, 32, 0.3, 500.0, 16), "mlp": _moe(16, 5, 3, 4, 56)},
    {"type": "parallel", "mixer": _pair(4, 1, 64, 64, 0.2, 64, 4, 16, 16, 15.0, 1.0, 1.0), "mlp": _moe(12, 2, 2, 1)},
    {"type": "parallel", "mixer": _pair(3, 3, 24, 40, 0.4, 33, 1, 40, 24, 8.0, 0.5, 2.0), "mlp": _moe(10, 8, 0, 2, 8)},
], streams=2, pairs=(200, 1, 3), cap=50.0)
# what the design may leave out: no copies of the stream (the plain pre-norm block), no table of pairs, no cap, no chunks
N3 = _model(77, 40, 1e-5, 2.0, [
    {"type": "parallel", "mixer": _pair(5, 5, 8, 8, 1.1, None, 2, 8, 12, 10.0, 1.0, 0.7), "mlp": _moe(24, 3, 1, 2, 16)},
    {"type": "latent_attention", "mixer": _latent(4, 12, 0, 20, 16, 0.5), "mlp": None},
])
# one copy of the stream (its tensors exist), chunks of a single position, odd head sizes, every router entry chosen
N4 = _model(64, 32, 1e-6, 1.0, [
    {"type": "latent_attention", "mixer": _latent(2, 8, 6, 8, 8, 0.6, 30.0, 6), "mlp": _moe(8, 2, 2, 4)},
    {"type": "parallel", "mixer": _pair(2, 1, 7, 9, 0.8, 1, 2, 8, 8, 10.0, 1.0, 1.0), "mlp": _moe(8, 3, 0, 3, 8)},
], streams=1, pairs=(5, 2, 3), cap=8.0)
# sizes that are multiples of nothing much: a width of 52, a vocabulary of 101, odd inner sizes, five copies, pairs only
N5 = _model(101, 52, 1e-5, 7.0, [
    {"type": "parallel", "mixer": _pair(5, 1, 12, 20, 0.5, 7, 5, 6, 10, 12.0, 1.2, 0.5), "mlp": _moe(18, 7, 3, 3, 10)},
    {"type": "parallel", "mixer": _pair(2, 1, 10, 6, 0.4, 40, 3, 12, 6, 9.0, 0.9, 0.9), "mlp": None},
], streams=5, pairs=(37, 11, 5))
# sizes that the tensor-core kernels take (heads of 128 and 64, values narrower and wider than the keys, pages of 32), for
# prompts of hundreds of tokens that cross several chunks
N6 = _model(300, 192, 1e-5, 4.0, [
    {"type": "parallel", "mixer": _pair(8, 2, 128, 64, 0.06, 150, 4, 64, 64, 12.0, 1.2, 0.5), "mlp": _moe(48, 12, 4, 4, 64)},
    {"type": "latent_attention", "mixer": _latent(4, 32, 32, 64, 96, 0.15, 10000.0, 32), "mlp": _moe(40, 8, 0, 2)},
    {"type": "parallel", "mixer": _pair(4, 4, 64, 128, 0.1, 96, 2, 128, 64, 10.0, 0.7, 1.0), "mlp": None},
], streams=4, pairs=(521, 3, 5), cap=25.0)
CONFIGS = {"N1": N1, "N2": N2, "N3": N3, "N4": N4, "N5": N5, "N6": N6}
PAGE_SIZE = {"N1": 8, "N2": 16, "N3": 4, "N4": 16, "N5": 16, "N6": 32}


def write_tiny_tenalorn(name: str, folder=None, seed: int = 0, config: dict | None = None, std: float = 0.12) -> Path:
    cfg = TenalornConfig.from_dict(config or CONFIGS[name])
    folder = Path(folder) if folder is not None else Path(tempfile.mkdtemp(prefix=f"tiny_{name}_"))
    write_random_model(folder, cfg, expected_tensors(cfg), seed=seed, std=std, norm_std=0.1)
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    g = torch.Generator().manual_seed(seed + 29)
    for n, t in tensors.items():
        if n.endswith(".mix") and ".hc" in n:                  # every copy mostly keeps itself and takes a little of the others
            tensors[n] = (torch.eye(t.shape[0]) + 0.3 * torch.randn(t.shape, generator=g)).to(t.dtype)
        elif n.endswith((".right.i", ".right.f", ".right.g", ".mix.g")):     # gates that move from token to token
            tensors[n] = (t.float() * 4.0).to(t.dtype)
        elif n.endswith(".f.b"):                               # forget gates near one: a far token still counts
            tensors[n] = (torch.rand(t.shape, generator=g) * 4.0 + 2.0).to(t.dtype)
        elif n.endswith(".router"):
            tensors[n] = (t.float() * 3.0).to(t.dtype)
        elif n.endswith(".correction"):                        # of the order of the scores: it changes which entries are chosen
            tensors[n] = (t.float() * 1.5).to(t.dtype)
        elif n.endswith((".gate", ".up")):
            tensors[n] = (t.float() * 2.5).to(t.dtype)
    write_safetensors(folder / "model.safetensors", tensors, {"format": "pt"})
    return folder
