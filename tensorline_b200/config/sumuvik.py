"""`SumuvikConfig`: the config.json of a Sumuvik decoder, typed and validated.

The file is nested: `layers` lists the layers, each with its `type` (which mixer: "attention" or "rglru"), the mixer's
sizes under `mixer` and its feed-forward under `mlp` (null: none; `kind` "dense" or "moe"); `embedding.scale`, `norm.eps`,
`vocab` and `width` are the model's.  A key the design has is required and every error names its key.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, ConfigReader


@dataclass(frozen=True)
class FrequencyScaling:
    """Wavelengths above original / low are stretched by `factor`, those below original / high are kept, the ones
    between are blended."""
    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    scaling: FrequencyScaling | None = None


@dataclass(frozen=True)
class AttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None
    keep_first: int
    rot: Rotation


@dataclass(frozen=True)
class RecurrentSizes:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class DenseSizes:
    ff: int
    limit: float


@dataclass(frozen=True)
class MoESizes:
    ff: int
    limit: float
    experts: int
    top: int
    groups: int
    keep_groups: int
    scale: float
    shared: DenseSizes | None


@dataclass(frozen=True)
class SumuvikLayer:
    type: str
    mixer: object
    mlp: object | None


def _rotation(raw, where: str, most: int) -> Rotation:
    r = ConfigReader(raw, where)
    base, dims = r.float("base", positive=True), r.int("dims", min=0)
    if dims % 2 or dims > most:
        raise ConfigError(f"{where}: 'dims' {dims} must be even and at most {most}")
    scaling = None
    if r.any("scaling") is not None:
        s = ConfigReader(r.any("scaling"), f"{where}.scaling")
        scaling = FrequencyScaling(s.float("factor", positive=True), s.float("low", positive=True), s.float("high", positive=True),
                                   s.float("original", positive=True))
        if not scaling.high > scaling.low:
            raise ConfigError(f"{where}.scaling: 'high' {scaling.high} must exceed 'low' {scaling.low}")
    return Rotation(base, dims, scaling)


def _mixer(kind: str, raw, where: str):
    if not isinstance(raw, dict):
        raise ConfigError(f"{where}: 'mixer' must be an object")
    r = ConfigReader(raw, where)
    if kind == "attention":
        heads, kv = r.int("heads", min=1), r.int("kv_heads", min=1)
        if heads % kv:
            raise ConfigError(f"{where}: 'heads' {heads} is not a multiple of 'kv_heads' {kv}")
        dim = r.int("dim", min=1)
        window, keep = None, 0                           # no mask: every earlier key
        if r.any("mask") is not None:
            mask = ConfigReader(r.any("mask"), f"{where}.mask")
            window, keep = mask.int("size", min=1), mask.int("keep_first", 0, min=0)
        return AttentionSizes(heads, kv, dim, r.int("vdim", min=1), r.float("scale", positive=True), window, keep,
                              _rotation(r.any("rot"), f"{where}.rot", dim))
    if kind == "rglru":
        out = RecurrentSizes(r.int("width", min=1), r.int("blocks", min=1), r.int("conv", min=1))
        if out.width % out.blocks:
            raise ConfigError(f"{where}: 'width' {out.width} is not a multiple of 'blocks' {out.blocks}")
        return out
    raise ConfigError(f"{where}: layer type {kind!r} is neither 'attention' nor 'rglru'")


def _dense(raw, where: str) -> DenseSizes:
    r = ConfigReader(raw, where)
    return DenseSizes(r.int("ff", min=1), r.float("limit", positive=True))


def _mlp(raw, where: str):
    if raw is None:
        return None
    r = ConfigReader(raw, where)
    kind = r.str("kind")
    if kind == "dense":
        return _dense(raw, where)
    if kind != "moe":
        raise ConfigError(f"{where}: feed-forward kind {kind!r} is neither 'dense' nor 'moe'")
    e = _dense(r.any("expert"), f"{where}.expert")
    ro = ConfigReader(r.any("router"), f"{where}.router")
    g = ConfigReader(ro.any("groups"), f"{where}.router.groups")
    shared = r.any("shared")
    out = MoESizes(e.ff, e.limit, ro.int("experts", min=1), ro.int("top", min=1), g.int("count", min=1), g.int("keep", min=1),
                   ro.float("scale", positive=True), None if shared is None else _dense(shared, f"{where}.shared"))
    if out.experts % out.groups or out.keep_groups > out.groups:
        raise ConfigError(f"{where}.router: {out.experts} experts in {out.groups} groups of which {out.keep_groups} are kept")
    if out.top > out.keep_groups * (out.experts // out.groups):
        raise ConfigError(f"{where}.router: 'top' {out.top} exceeds the experts of the kept groups")
    return out


@dataclass(frozen=True)
class SumuvikConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "SumuvikConfig":
        r = ConfigReader(raw, where)
        layers_raw = r.any("layers")
        if not (isinstance(layers_raw, list) and layers_raw):
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            w = f"{where}: layers[{i}]"
            l = ConfigReader(lr, w)
            kind = l.str("type")
            layers.append(SumuvikLayer(kind, _mixer(kind, l.any("mixer"), f"{w}.mixer"), _mlp(l.any("mlp"), f"{w}.mlp")))
        norm = ConfigReader(r.any("norm"), f"{where}: norm")
        emb = ConfigReader(r.any("embedding"), f"{where}: embedding")
        return cls(architecture=r.str("architecture", "Sumuvik"), vocab=r.int("vocab", min=1), width=r.int("width", min=1),
                   norm_eps=norm.float("eps", positive=True), embedding_scale=emb.float("scale"), layers=tuple(layers))

    # what every engine front end asks of a configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    eos_token_id = None
    max_position_embeddings = None

    def to_json_dict(self) -> dict:
        def dense(m, kind=None):
            d = {"ff": m.ff, "limit": m.limit}
            if kind:
                d["kind"] = kind
            return d

        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == "attention":
                rot = {"base": m.rot.base, "dims": m.rot.dims}
                if m.rot.scaling is not None:
                    s = m.rot.scaling
                    rot["scaling"] = {"factor": s.factor, "high": s.high, "low": s.low, "original": s.original}
                mixer = {"dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads, "rot": rot, "scale": m.scale, "vdim": m.vdim}
                if m.window is not None:
                    mixer["mask"] = {"keep_first": m.keep_first, "size": m.window}
            else:
                mixer = {"blocks": m.blocks, "conv": m.conv, "width": m.width}
            if l.mlp is None:
                mlp = None
            elif isinstance(l.mlp, DenseSizes):
                mlp = dense(l.mlp, "dense")
            else:
                f = l.mlp
                mlp = {"expert": {"ff": f.ff, "limit": f.limit}, "kind": "moe",
                       "router": {"experts": f.experts, "groups": {"count": f.groups, "keep": f.keep_groups}, "scale": f.scale,
                                  "top": f.top}}
                if f.shared is not None:
                    mlp["shared"] = dense(f.shared)
            layers.append({"mixer": mixer, "mlp": mlp, "type": l.type})
        return {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale}, "layers": layers,
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    def num_parameters(self) -> int:
        from ..models.registry import expected_tensors
        n = 0
        for spec in expected_tensors(self).values():
            k = 1
            for s in spec.shape:
                k *= s
            n += k
        return n
