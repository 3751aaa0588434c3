"""The Tenalorn configuration, model description and cache bookkeeping, without a GPU."""
import copy

import pytest
import torch

from tensorline_b200.cache import CacheManager, PagedKV, SlotState
from tensorline_b200.config import ConfigError
from tensorline_b200.config.tenalorn import TenalornConfig
from tensorline_b200.models import build_model, expected_tensors
from tensorline_b200.models.registry import architecture, registered_architectures
from tensorline_b200.models.tenalorn import describe_tenalorn, distance_slopes
from tensorline_b200.parts import Runtime
from tests.tiny_tenalorn import CONFIGS


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_round_trip_and_registry(name):
    cfg = TenalornConfig.from_dict(CONFIGS[name])
    assert cfg.to_json_dict() == CONFIGS[name]
    assert "Tenalorn" in registered_architectures() and architecture("Tenalorn").config_class is TenalornConfig
    assert cfg.vocab_size == CONFIGS[name]["vocab"] and cfg.hidden_size == CONFIGS[name]["width"]
    assert cfg.num_parameters() > 0
    spec = describe_tenalorn(cfg)
    assert [e.layer for e in spec.run] == list(range(len(cfg.layers)))
    kind = "pre_norm" if "streams" not in CONFIGS[name] else "hyper_connections"
    assert all(l.block.kind == kind for l in spec.layers) and spec.streams == CONFIGS[name].get("streams", 1)
    assert spec.embedding.kind == ("token_pairs" if "bigram" in CONFIGS[name]["embedding"] else "token_table")
    assert spec.head.params["softcap"] == CONFIGS[name].get("logit_softcap")


def test_tensor_names_and_shapes():
    names = expected_tensors(TenalornConfig.from_dict(CONFIGS["N1"]))
    want = {"embed": (131, 48), "bigram": (62, 48), "final.norm": (48,), "head": (131, 48), "l0.norm1": (48,), "l0.norm2": (48,),
            "l0.hc1.in": (3,), "l0.hc1.out": (3,), "l0.hc1.mix": (3, 3), "l0.hc2.mix": (3, 3),
            "l0.mix.left.q": (96, 48), "l0.mix.left.k": (32, 48), "l0.mix.left.v": (48, 48), "l0.mix.left.o": (48, 144),
            "l0.mix.right.q": (24, 48), "l0.mix.right.k": (24, 48), "l0.mix.right.v": (48, 48), "l0.mix.right.g": (48, 48),
            "l0.mix.right.o": (48, 48), "l0.mix.right.norm": (48,), "l0.mix.right.i": (3, 48), "l0.mix.right.i.b": (3,),
            "l0.mix.right.f": (3, 48), "l0.mix.right.f.b": (3,),
            "l0.mlp.router": (8, 48), "l0.mlp.correction": (8,), "l0.mlp.e5.gate": (24, 48), "l0.mlp.e0.up": (24, 48), "l0.mlp.e3.down": (48, 24),
            "l0.mlp.shared.gate": (16, 48), "l0.mlp.shared.up": (16, 48), "l0.mlp.shared.down": (48, 16),
            "l1.mix.q": (48, 48), "l1.mix.dkv": (28, 48), "l1.mix.dkv.norm": (20,), "l1.mix.uk": (24, 20), "l1.mix.uv": (36, 20),
            "l1.mix.g": (36, 48), "l1.mix.o": (48, 36), "l1.mlp.router": (5, 48), "l3.mlp.router": (3, 48)}
    for k, shape in want.items():
        assert tuple(names[k].shape) == shape, k
    assert names["l2.norm2"].optional                                      # a layer without a feed-forward
    for absent in ("l0.mlp.e6.up", "l1.mlp.shared.gate", "l2.hc2.in", "l0.mix.left.q.b", "l0.mix.left.out", "l1.mix.dq", "l1.mix.dq.norm",
                   "l1.mix.uq", "l0.mix.left.q_norm", "l0.mlp.router.b", "l0.mlp.shared.sg"):
        assert absent not in names, absent
    plain = expected_tensors(TenalornConfig.from_dict(CONFIGS["N3"]))       # one plain stream: no such tensors, no table of pairs
    assert not any(".hc" in k for k in plain) and "bigram" not in plain


def test_the_slopes_of_the_heads():
    assert distance_slopes(4) == [0.25, 0.0625, 0.015625, 0.00390625]
    assert distance_slopes(1) == [2.0 ** -8] and len(distance_slopes(6)) == 6


def test_what_the_cache_manager_is_asked_for():
    rt = Runtime(torch.device("cpu"), torch.float32, 8)
    needs = build_model(TenalornConfig.from_dict(CONFIGS["N1"]), rt).cache_needs()
    assert needs["embedding"] == SlotState((1,), "int32")
    assert needs[(0, "left")] == PagedKV(2, 24, None, chunk=11) and needs[(2, "left")] == PagedKV(2, 32, None, chunk=19)
    assert isinstance(needs[(0, "right")], SlotState) and needs[(0, "right")].dtype == "float32"
    assert needs[1] == PagedKV(1, 28, None, shared_values=True) and needs[3] == PagedKV(1, 16, None, shared_values=True)
    n3 = build_model(TenalornConfig.from_dict(CONFIGS["N3"]), rt).cache_needs()
    assert "embedding" not in n3 and n3[(0, "left")] == PagedKV(5, 8, None)
    rt16 = Runtime(torch.device("cpu"), torch.bfloat16, 8)                  # bfloat16 pages: multiples of 16
    assert build_model(TenalornConfig.from_dict(CONFIGS["N5"]), rt16).cache_needs()[(0, "left")] == PagedKV(1, 32, None, chunk=7)


def test_pages_of_chunks_that_lie_behind_are_given_back():
    """A group of chunked attention keeps the pages from its request's current chunk on; groups with other chunks, and those
    that keep everything, keep their own books."""
    needs = {0: PagedKV(1, 8, None, chunk=20), 1: PagedKV(1, 8, None, chunk=7), 2: PagedKV(1, 8, None), 3: SlotState((4,))}
    cm = CacheManager(needs, page_size=4, num_pages=40, max_num_seqs=2, max_model_len=160, prefix_caching=False)
    assert len(cm.groups) == 3 and [g.chunk for g in cm.groups] == [20, 7, None]
    assert cm.admit("a") == 0 and cm.grow("a", 0, 30)
    cm.advance("a", 30, None)                              # the next query is position 30: chunks start at 20 and at 28
    held = [cm.pages("a", g) for g in range(3)]
    assert [p >= 0 for p in held[0]] == [False] * 5 + [True] * 3
    assert [p >= 0 for p in held[1]] == [False] * 7 + [True]
    assert all(p >= 0 for p in held[2])
    assert cm.grow("a", 30, 41)
    cm.advance("a", 41, None)                              # 41: chunks start at 40 and at 35
    assert [p >= 0 for p in cm.pages("a", 0)] == [False] * 10 + [True]
    assert [p >= 0 for p in cm.pages("a", 1)] == [False] * 8 + [True] * 3
    cm.check()
    cm.release("a")
    assert all(g.pool.num_free == g.pool.num_pages for g in cm.groups)
    with pytest.raises(ValueError):
        CacheManager({0: PagedKV(1, 8, 5, chunk=4)}, page_size=4, num_pages=4, max_num_seqs=1, max_model_len=16)


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "attention", "type"), (("layers", 0, "mixer", "left", "kv_heads"), 4, "kv_heads"),
    (("layers", 1, "mixer", "rot", "dims"), 5, "dims"), (("layers", 0, "mlp", "router", "top"), 9, "top"),
    (("layers", 0, "mlp", "kind"), "dense", "kind"), (("streams",), 0, "streams"), (("logit_softcap",), -1.0, "logit_softcap"),
    (("layers", 0, "mixer", "left", "mask", "size"), 0, "size"), (("embedding", "bigram", "buckets"), 0, "buckets"),
])
def test_errors_name_their_key(path, value, word):
    raw = copy.deepcopy(CONFIGS["N1"])
    node = raw
    for k in path[:-1]:
        node = node[k]
    node[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        TenalornConfig.from_dict(raw)


def test_a_missing_key_is_an_error():
    for path in (("vocab",), ("norm",), ("layers", 0, "mixer", "left_scale"), ("layers", 0, "mixer", "right", "gate_cap"),
                 ("layers", 1, "mixer", "kv_rank"), ("layers", 0, "mlp", "router", "experts")):
        raw = copy.deepcopy(CONFIGS["N1"])
        node = raw
        for k in path[:-1]:
            node = node[k]
        del node[path[-1]]
        with pytest.raises(ConfigError):
            TenalornConfig.from_dict(raw)
