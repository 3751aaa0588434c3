"""`ModelSpec`: a model as data, and `Model`, which builds and runs it.

    ModelSpec(vocab, hidden, layers=[LayerSpec...], run=[RunEntry...], final_norm, tied head, ...)

`layers` are the distinct sets of weights; `run` is the order in which they run, one
`RunEntry(layer, cache)` per executed block.  A layer may be named by several entries (shared
weights, each entry with a cache of its own), and an entry may name the cache of an *earlier*
entry in `reads_cache_of` (it then attends to that entry's keys and values and writes none).
The cache manager is told one need per cache-owning entry.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts import BLOCKS, EMBEDDINGS, HEADS, NORMS, POSITION_ENCODINGS, KVCacheView, PartSpec, Runtime, TensorSpec
from ..parts.linear import with_row


@dataclass(frozen=True)
class LayerSpec:
    block: PartSpec                     # params: mixer, feed_forward, norm1, norm2 (PartSpecs)
    prefix: str                         # tensor-name prefix of the layer, e.g. "model.layers.3"


@dataclass(frozen=True)
class RunEntry:
    layer: int                          # index into ModelSpec.layers
    reads_cache_of: int | None = None   # index of an earlier run entry whose cache this one reads
    add_row: int | None = None          # row of `ModelSpec.stream_rows` added to the residual stream in front of this entry


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    layers: tuple
    run: tuple
    final_norm: PartSpec
    tie_word_embeddings: bool
    embedding_prefix: str = "model.embed_tokens"
    final_norm_prefix: str = "model.norm"
    head_prefix: str = "lm_head"
    embedding_position: PartSpec | None = None        # an encoding added to the embedded tokens, if any
    embedding_position_prefix: str = "model.embed_positions"     # where its tensors live, if it has any
    eos_token_id: int | None = None
    max_position_embeddings: int | None = None
    embedding: PartSpec = PartSpec("token_table")     # built with vocab= and dim=; another kind may scale its rows
    head: PartSpec = PartSpec("linear")               # built with vocab=, dim= and tied=; another kind may add a bias or a cap
    embedding_norm: PartSpec | None = None            # a norm of the embedded tokens: the stream starts as its float32 result
    embedding_norm_prefix: str = "model.embed_norm"
    stream_rows: int = 0                              # > 0: a table [rows, hidden] of vectors that run entries add to the stream
    stream_rows_name: str = "model.stream_rows"       # (`RunEntry.add_row`: a pass over shared layers announces its number)
    stream_rows_eps: float = 1e-6                     # eps of the norms the addend travels to (they fold it into their kernel)
    streams: int = 1                                  # > 1: the residual stream is that many copies side by side, [T, streams * hidden]
                                                      # (blocks of kind "hyper_connections"; the model's norm reads their sum)


class Model:
    """The built model: parts on the device, bound to weights; `forward` runs one step."""

    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec, self.rt = spec, rt
        extra = {"copies": spec.streams} if spec.streams != 1 else {}
        self.embedding = EMBEDDINGS.build(spec.embedding, rt, vocab=spec.vocab_size, dim=spec.hidden_size, **extra)
        self.blocks = [BLOCKS.build(l.block, rt) for l in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm, rt)
        self.head = HEADS.build(spec.head, rt, vocab=spec.vocab_size, dim=spec.hidden_size, tied=spec.tie_word_embeddings)
        self.embedding_position = (POSITION_ENCODINGS.build(spec.embedding_position, rt)
                                   if spec.embedding_position else None)
        self.embedding_norm = NORMS.build(spec.embedding_norm, rt) if spec.embedding_norm else None
        self.stream_rows = None
        for i, e in enumerate(spec.run):
            if e.add_row is not None and not 0 <= e.add_row < spec.stream_rows:
                raise ValueError(f"run entry {i} adds row {e.add_row} of a table of {spec.stream_rows}")
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"run entry {i} names layer {e.layer}, the model has {len(self.blocks)}")
            if e.reads_cache_of is not None and not (0 <= e.reads_cache_of < i
                                                     and spec.run[e.reads_cache_of].reads_cache_of is None):
                raise ValueError(f"run entry {i} must read the cache of an earlier entry that owns one")

    # ---- weights
    def expected_tensors(self) -> dict:
        out = dict(self.embedding.expected_tensors(self.spec.embedding_prefix))
        if self.embedding_position is not None:
            out.update(self.embedding_position.expected_tensors(self.spec.embedding_position_prefix))
        if self.embedding_norm is not None:
            out.update(self.embedding_norm.expected_tensors(self.spec.embedding_norm_prefix))
        if self.spec.stream_rows:
            out[self.spec.stream_rows_name] = TensorSpec((self.spec.stream_rows, self.spec.hidden_size))
        for block, layer in zip(self.blocks, self.spec.layers):
            out.update(block.expected_tensors(layer.prefix))
        out.update(self.final_norm.expected_tensors(self.spec.final_norm_prefix))
        out.update(self.head.expected_tensors(self.spec.head_prefix))
        return out

    def bind(self, weights: dict) -> None:
        self.embedding.bind(weights, self.spec.embedding_prefix)
        if self.embedding_position is not None:
            self.embedding_position.bind(weights, self.spec.embedding_position_prefix)
        if self.embedding_norm is not None:
            self.embedding_norm.bind(weights, self.spec.embedding_norm_prefix)
        if self.spec.stream_rows:
            self.stream_rows = weights[self.spec.stream_rows_name].float().contiguous()      # they join a float32 sum
        for block, layer in zip(self.blocks, self.spec.layers):
            block.bind(weights, layer.prefix)
        self.final_norm.bind(weights, self.spec.final_norm_prefix)
        self.head.bind(weights, self.spec.head_prefix, self.embedding)

    # ---- caches
    def cache_needs(self) -> dict:
        """cache id (= index of the owning run entry) -> need."""
        needs = {}
        own = getattr(self.embedding, "cache_need", None)
        if own is not None and own() is not None:        # an embedding that keeps something of a request between steps
            needs["embedding"] = own()
        for i, e in enumerate(self.spec.run):
            if e.reads_cache_of is None:
                need = self.blocks[e.layer].cache_need()
                if isinstance(need, dict):               # a mixer made of several: one cache each, id (entry, name)
                    for name, n in need.items():
                        needs[(i, name)] = n
                elif need is not None:
                    needs[i] = need
        return needs

    def _cache_of(self, i: int, caches: dict):
        """What run entry i's block is handed: its view, or {name: view} for a block whose mixer keeps several."""
        need = self.blocks[self.spec.run[i].layer].cache_need()
        if isinstance(need, dict):
            return {name: caches[(i, name)] for name in need}
        return caches.get(i)

    def graph_capturable(self) -> bool:
        """Whether a step of single tokens can be captured in a CUDA graph: every part reads the step from
        device tensors only."""
        parts = [self.embedding, self.final_norm, self.head, *self.blocks]
        if self.embedding_position is not None:
            parts.append(self.embedding_position)
        if self.embedding_norm is not None:
            parts.append(self.embedding_norm)
        return all(getattr(p, "graph_capturable", False) for p in parts)

    # ---- one step
    def forward(self, ctx, caches: dict) -> torch.Tensor:
        """Logits [R, V] float32 at the rows `ctx.want_rows`; `caches`: cache id -> view."""
        if "embedding" in caches:
            x = self.embedding.forward(ctx.ids, ctx, caches["embedding"])
        else:
            x = self.embedding.forward(ctx.ids)
        if self.embedding_position is not None:
            self.embedding_position.on_embedding(x, ctx)
        if self.embedding_norm is not None:
            x = self.embedding_norm.norm_stream(x)
        pending = None
        for i, e in enumerate(self.spec.run):
            if e.add_row is not None:
                pending = with_row(x, pending, self.stream_rows[e.add_row], self.spec.stream_rows_eps)
            if e.reads_cache_of is None:
                cache = self._cache_of(i, caches)
            else:
                owner = self._cache_of(e.reads_cache_of, caches)
                cache = KVCacheView(owner.k, owner.v, owner.group, owner=False) if isinstance(owner, KVCacheView) else owner
            pending = self.blocks[e.layer].forward(x, pending, ctx, cache)
        if ctx.want_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=x.device)
        if getattr(self.head, "accepts_normed_input", False) and getattr(self.final_norm, "can_defer", False):
            h = self.final_norm.add_norm(x, pending, rows=ctx.want_rows, defer=True)
        else:
            h = self.final_norm.add_norm(x, pending, rows=ctx.want_rows)
        return self.head.forward(h)
