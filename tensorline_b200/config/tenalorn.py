"""`TenalornConfig`: the config.json of a Tenalorn decoder, typed and validated.

The file is nested: `layers` lists the layers, each with its `type` (which mixer: "parallel", a chunked attention beside a
matrix memory, or "latent_attention"), the mixer's sizes under `mixer` and its feed-forward under `mlp` (null: none; `kind`
"moe"); `embedding` holds the scale of the embedded tokens and, under `bigram`, the hash of the table of token pairs;
`streams` is the number of copies of the residual stream (absent: one plain stream), `logit_softcap` the cap on the logits
(absent: none); `norm.eps`, `vocab` and `width` are the model's.  A key the design always has is required and every error
names its key; a mask, the table of pairs, identity entries of a router and a shared expert may be absent.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, ConfigReader


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int


@dataclass(frozen=True)
class PairHash:
    """Row of the table of token pairs: (previous token * mul_prev + token * mul_cur) mod buckets; row `buckets` for a first token."""
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class ChunkAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int | None                   # positions a chunk; None: every earlier key is seen


@dataclass(frozen=True)
class MatrixMemorySizes:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ParallelSizes:
    left: ChunkAttentionSizes
    right: MatrixMemorySizes
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: Rotation


@dataclass(frozen=True)
class MoESizes:
    ff: int
    experts: int                        # experts with matrices
    identity: int                       # router entries behind them whose output is their input
    top: int
    shared_ff: int | None


@dataclass(frozen=True)
class TenalornLayer:
    type: str
    mixer: object
    mlp: MoESizes | None


def _rotation(raw, where, most) -> Rotation:
    if raw is None and most == 0:                        # nothing to rotate: the constants may be left out
        return Rotation(10000.0, 0)
    r = ConfigReader(raw if raw is not None else {}, where)
    rot = Rotation(r.float("base", positive=True), r.int("dims", min=0))
    if rot.dims % 2 or rot.dims > most:
        raise ConfigError(f"{where}: 'dims' {rot.dims} must be even and at most {most}")
    return rot


def _left(raw, where) -> ChunkAttentionSizes:
    r = ConfigReader(raw, where)
    heads, kv = r.int("heads", min=1), r.int("kv_heads", min=1)
    if heads % kv:
        raise ConfigError(f"{where}: 'heads' {heads} is not a multiple of 'kv_heads' {kv}")
    mask = r.any("mask")
    chunk = None if mask is None else ConfigReader(mask, f"{where}.mask").int("size", min=1)
    return ChunkAttentionSizes(heads, kv, r.int("dim", min=1), r.int("vdim", min=1), r.float("scale", positive=True), chunk)


def _right(raw, where) -> MatrixMemorySizes:
    r = ConfigReader(raw, where)
    return MatrixMemorySizes(r.int("heads", min=1), r.int("dim", min=1), r.int("vdim", min=1), r.float("gate_cap", positive=True))


def _mixer(kind: str, raw, where: str):
    if not isinstance(raw, dict):
        raise ConfigError(f"{where}: 'mixer' must be an object")
    r = ConfigReader(raw, where)
    if kind == "parallel":
        return ParallelSizes(_left(r.any("left"), f"{where}.left"), _right(r.any("right"), f"{where}.right"),
                             r.float("left_scale"), r.float("right_scale"))
    if kind == "latent_attention":
        rot_dim = r.int("rot_dim", min=0)
        return LatentAttentionSizes(r.int("heads", min=1), r.int("dim", min=1), rot_dim, r.int("vdim", min=1),
                                    r.int("kv_rank", min=1), r.float("scale", positive=True),
                                    _rotation(r.any("rot"), f"{where}.rot", rot_dim))
    raise ConfigError(f"{where}: layer type {kind!r} is neither 'parallel' nor 'latent_attention'")


def _mlp(raw, where: str):
    if raw is None:
        return None
    r = ConfigReader(raw, where)
    kind = r.str("kind")
    if kind != "moe":
        raise ConfigError(f"{where}: feed-forward kind {kind!r} is not 'moe'")
    e = ConfigReader(r.any("expert"), f"{where}.expert")
    ro = ConfigReader(r.any("router"), f"{where}.router")
    shared = r.any("shared")
    out = MoESizes(e.int("ff", min=1), ro.int("experts", min=1), ro.int("identity", 0, min=0), ro.int("top", min=1),
                   None if shared is None else ConfigReader(shared, f"{where}.shared").int("ff", min=1))
    if out.top > out.experts + out.identity:
        raise ConfigError(f"{where}.router: 'top' {out.top} exceeds the {out.experts} + {out.identity} entries")
    return out


@dataclass(frozen=True)
class TenalornConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    pairs: PairHash | None
    streams: int | None                 # None: one plain residual stream
    logit_softcap: float | None
    layers: tuple

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "TenalornConfig":
        r = ConfigReader(raw, where)
        layers_raw = r.any("layers")
        if not (isinstance(layers_raw, list) and layers_raw):
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            w = f"{where}: layers[{i}]"
            l = ConfigReader(lr, w)
            kind = l.str("type")
            layers.append(TenalornLayer(kind, _mixer(kind, l.any("mixer"), f"{w}.mixer"), _mlp(l.any("mlp"), f"{w}.mlp")))
        norm = ConfigReader(r.any("norm"), f"{where}: norm")
        emb = ConfigReader(r.any("embedding", {}), f"{where}: embedding")
        pairs = None
        if emb.any("bigram") is not None:
            b = ConfigReader(emb.any("bigram"), f"{where}: embedding.bigram")
            pairs = PairHash(b.int("buckets", min=1), b.int("mul_prev"), b.int("mul_cur"))
        return cls(architecture=r.str("architecture", "Tenalorn"), vocab=r.int("vocab", min=1), width=r.int("width", min=1),
                   norm_eps=norm.float("eps", positive=True), embedding_scale=emb.float("scale", 1.0), pairs=pairs,
                   streams=r.int("streams", None, min=1), logit_softcap=r.float("logit_softcap", None, positive=True),
                   layers=tuple(layers))

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
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == "parallel":
                a, b = m.left, m.right
                left = {"dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "scale": a.scale, "vdim": a.vdim}
                if a.chunk is not None:
                    left["mask"] = {"size": a.chunk}
                mixer = {"left": left, "left_scale": m.left_scale,
                         "right": {"dim": b.dim, "gate_cap": b.gate_cap, "heads": b.heads, "vdim": b.vdim},
                         "right_scale": m.right_scale}
            else:
                mixer = {"dim": m.dim, "heads": m.heads, "kv_rank": m.kv_rank, "rot_dim": m.rot_dim, "scale": m.scale, "vdim": m.vdim}
                if m.rot_dim:
                    mixer["rot"] = {"base": m.rot.base, "dims": m.rot.dims}
            mlp = None
            if l.mlp is not None:
                f = l.mlp
                mlp = {"expert": {"ff": f.ff}, "kind": "moe", "router": {"experts": f.experts, "identity": f.identity, "top": f.top}}
                if f.shared_ff is not None:
                    mlp["shared"] = {"ff": f.shared_ff}
            layers.append({"mixer": mixer, "mlp": mlp, "type": l.type})
        emb = {"scale": self.embedding_scale}
        if self.pairs is not None:
            emb["bigram"] = {"buckets": self.pairs.buckets, "mul_cur": self.pairs.mul_cur, "mul_prev": self.pairs.mul_prev}
        out = {"architecture": self.architecture, "embedding": emb, "layers": layers, "norm": {"eps": self.norm_eps},
               "vocab": self.vocab, "width": self.width}
        if self.streams is not None:
            out["streams"] = self.streams
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out

    def num_parameters(self) -> int:
        from ..models.registry import expected_tensors
        n = 0
        for spec in expected_tensors(self).values():
            k = 1
            for s in spec.shape:
                k *= s
            n += k
        return n
