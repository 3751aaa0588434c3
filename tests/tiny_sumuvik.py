"""Tiny Sumuvik configurations of the tests and a helper that writes their model folders.

S1 to S5 differ in every size and option: grouped and ungrouped heads, value heads wider and narrower than query heads,
head sizes that are no multiples of 16, windows that are no multiples of the page, kept first tokens fewer and more than
a page and more than the window, no kept tokens, no mask at all, a rotation over all, part or none of a head with and
without stretched wavelengths, convolutions of one to five taps, one to many blocks of gates, experts in one to four
groups of which one to all are kept, groups of a single expert, every allowed expert chosen, with and without a shared
expert, layers without a feed-forward, attention only and recurrence only.  The attention scales are large, so that a
softmax is decided by few keys and a key that is wrongly seen (or not seen) shows; the recurrence's decays lie between
0.5 and 0.999 a token, so that a lost or stale state shows many tokens later.
"""
from __future__ import annotations

import tempfile
from pathlib import Path

import torch

from tensorline_b200.config.sumuvik import SumuvikConfig
from tensorline_b200.models import expected_tensors
from tensorline_b200.weights import write_random_model
from tensorline_b200.weights.safetensors_io import SafetensorsFile, write_safetensors


def _att(heads, kv, dim, vdim, scale, mask, rot):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if mask is not None:
        m["mask"] = {"keep_first": mask[1], "size": mask[0]}
    return m


def _rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def _rec(width, blocks, conv):
    return {"width": width, "blocks": blocks, "conv": conv}


def _dense(ff, limit):
    return {"ff": ff, "kind": "dense", "limit": limit}


def _moe(ff, limit, experts, top, groups, keep, scale, shared=None):
    out = {"expert": {"ff": ff, "limit": limit}, "kind": "moe",
           "router": {"experts": experts, "groups": {"count": groups, "keep": keep}, "scale": scale, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def _model(vocab, width, eps, emb, layers):
    return {"architecture": "Sumuvik", "embedding": {"scale": emb}, "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


S1 = _model(131, 48, 1e-6, 3.0, [
    {"type": "attention", "mixer": _att(6, 2, 16, 24, 0.9, (11, 3), _rot(100.0, 8, (8.0, 1.0, 4.0, 16.0))), "mlp": _dense(56, 1.5)},
    {"type": "rglru", "mixer": _rec(40, 5, 4), "mlp": _moe(24, 2.5, 8, 2, 4, 2, 2.5, (16, 1.0))},
    {"type": "attention", "mixer": _att(2, 2, 32, 16, 0.5, (19, 10), _rot(10000.0, 32)), "mlp": _moe(20, 1.0, 6, 3, 2, 1, 1.0)},
    {"type": "rglru", "mixer": _rec(64, 1, 2), "mlp": None},
])
S2 = _model(90, 72, 1e-5, 0.5, [
    {"type": "rglru", "mixer": _rec(96, 3, 3), "mlp": _dense(100, 3.0)},
    {"type": "attention", "mixer": _att(4, 1, 64, 64, 0.3, (64, 17), _rot(500.0, 16, (4.0, 1.0, 2.0, 32.0))), "mlp": None},
    {"type": "rglru", "mixer": _rec(24, 24, 1), "mlp": _moe(16, 2.0, 9, 4, 3, 2, 0.7, (56, 2.0))},
    {"type": "attention", "mixer": _att(3, 3, 24, 40, 0.4, (33, 0), _rot(50.0, 0)), "mlp": _moe(8, 1.2, 4, 4, 1, 1, 1.5)},
])
# attention only: every page group can share prefixes; no mask in one layer, more kept tokens than the window in another
S3 = _model(77, 40, 1e-5, 2.0, [
    {"type": "attention", "mixer": _att(5, 5, 8, 8, 1.1, None, _rot(30.0, 8)), "mlp": _dense(24, 2.0)},
    {"type": "attention", "mixer": _att(4, 2, 20, 12, 0.8, (5, 9), _rot(1000.0, 10, (2.0, 1.0, 8.0, 64.0))), "mlp": _moe(32, 2.0, 4, 1, 4, 1, 3.0, (16, 0.8))},
])
# the recurrence only: no keys or values anywhere, so no page group at all
S4 = _model(64, 32, 1e-6, 1.0, [
    {"type": "rglru", "mixer": _rec(48, 2, 5), "mlp": None},
    {"type": "rglru", "mixer": _rec(32, 4, 4), "mlp": _moe(8, 4.0, 3, 3, 1, 1, 1.0)},
])
# sizes that are multiples of nothing much: a width of 52, a vocabulary of 101, odd inner sizes, a window of one token
S5 = _model(101, 52, 1e-5, 7.0, [
    {"type": "attention", "mixer": _att(5, 1, 12, 20, 0.5, (1, 2), _rot(30.0, 6)), "mlp": _dense(30, 1.1)},
    {"type": "rglru", "mixer": _rec(39, 3, 3), "mlp": _moe(18, 1.7, 10, 3, 5, 2, 2.0, (10, 2.2))},
    {"type": "attention", "mixer": _att(2, 1, 10, 6, 0.4, (40, 1), _rot(20.0, 4, (3.0, 1.0, 3.0, 8.0))), "mlp": None},
])
# sizes that the tensor-core kernels take (heads of 128 and 64, values narrower and wider than the keys, pages of 32), for
# prompts of hundreds of tokens: kept tokens over two key tiles far under the window, gates of four blocks, sixteen experts
S6 = _model(300, 192, 1e-5, 4.0, [
    {"type": "attention", "mixer": _att(8, 2, 128, 64, 0.12, (150, 70), _rot(10000.0, 64, (8.0, 1.0, 4.0, 128.0))),
     "mlp": _moe(48, 2.0, 16, 4, 4, 2, 2.0, (64, 1.5))},
    {"type": "rglru", "mixer": _rec(256, 4, 4), "mlp": _dense(320, 3.0)},
    {"type": "attention", "mixer": _att(4, 4, 64, 128, 0.2, (100, 0), _rot(1000.0, 64)), "mlp": None},
    {"type": "rglru", "mixer": _rec(128, 2, 3), "mlp": _moe(40, 1.5, 8, 2, 2, 2, 1.0)},
])
CONFIGS = {"S1": S1, "S2": S2, "S3": S3, "S4": S4, "S5": S5, "S6": S6}
PAGE_SIZE = {"S1": 8, "S2": 16, "S3": 4, "S4": 16, "S5": 16, "S6": 32}


def write_tiny_sumuvik(name: str, folder=None, seed: int = 0, config: dict | None = None, std: float = 0.12) -> Path:
    cfg = SumuvikConfig.from_dict(config or CONFIGS[name])
    folder = Path(folder) if folder is not None else Path(tempfile.mkdtemp(prefix=f"tiny_{name}_"))
    write_random_model(folder, cfg, expected_tensors(cfg), seed=seed, std=std, norm_std=0.1)
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    g = torch.Generator().manual_seed(seed + 23)
    for n, t in tensors.items():
        if n.endswith(".lam"):                                 # decays from about 0.5 to 0.999 a token
            tensors[n] = (torch.rand(t.shape, generator=g) * 5.0 - 7.0).to(t.dtype)
        elif n.endswith((".ra", ".ri", ".mix.g")):              # gates that move from token to token
            tensors[n] = (t.float() * 4.0).to(t.dtype)
        elif n.endswith(".conv"):
            tensors[n] = (t.float() * 4.0).to(t.dtype)
        elif n.endswith(".router"):
            tensors[n] = (t.float() * 3.0).to(t.dtype)
        elif n.endswith(".correction"):                        # of the order of the scores: it changes which experts are chosen
            tensors[n] = (t.float() * 3.0).to(t.dtype)
        elif n.endswith((".gate", ".up")):                     # pre-activations on both sides of the limits
            tensors[n] = (t.float() * 2.5).to(t.dtype)
    write_safetensors(folder / "model.safetensors", tensors, {"format": "pt"})
    return folder
