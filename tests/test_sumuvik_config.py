"""The Sumuvik configuration, model description, frequency table and cache bookkeeping, without a GPU."""
import copy

import pytest
import torch

from tensorline_b200.cache import CacheManager, PagedKV, SlotState
from tensorline_b200.config import ConfigError
from tensorline_b200.config.sumuvik import SumuvikConfig
from tensorline_b200.models import build_model, expected_tensors
from tensorline_b200.models.registry import architecture, registered_architectures
from tensorline_b200.models.sumuvik import describe_sumuvik
from tensorline_b200.parts import POSITION_ENCODINGS, PartSpec, Runtime
from tests.plain.sumuvik_plain import frequencies
from tests.tiny_sumuvik import CONFIGS


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_round_trip_and_registry(name):
    cfg = SumuvikConfig.from_dict(CONFIGS[name])
    assert cfg.to_json_dict() == CONFIGS[name]
    assert "Sumuvik" in registered_architectures() and architecture("Sumuvik").config_class is SumuvikConfig
    assert cfg.vocab_size == CONFIGS[name]["vocab"] and cfg.hidden_size == CONFIGS[name]["width"]
    assert cfg.num_parameters() > 0
    spec = describe_sumuvik(cfg)
    assert [e.layer for e in spec.run] == list(range(len(cfg.layers))) and all(l.block.kind == "parallel_residual" for l in spec.layers)
    assert spec.embedding.params["scale"] == CONFIGS[name]["embedding"]["scale"]


def test_tensor_names_and_shapes():
    names = expected_tensors(SumuvikConfig.from_dict(CONFIGS["S1"]))
    want = {"embed": (131, 48), "final.norm": (48,), "head": (131, 48), "l0.norm1": (48,), "l0.norm2": (48,),
            "l0.mix.q": (96, 48), "l0.mix.q.b": (96,), "l0.mix.k": (32, 48), "l0.mix.k.b": (32,), "l0.mix.v": (48, 48), "l0.mix.v.b": (48,),
            "l0.mix.g": (6, 48), "l0.mix.o": (48, 144), "l0.mlp.gate": (56, 48), "l0.mlp.up": (56, 48), "l0.mlp.down": (48, 56),
            "l1.mix.y": (40, 48), "l1.mix.y.b": (40,), "l1.mix.x": (40, 48), "l1.mix.x.b": (40,), "l1.mix.conv": (40, 4), "l1.mix.conv.b": (40,),
            "l1.mix.ra": (5, 8, 8), "l1.mix.ra.b": (5, 8), "l1.mix.ri": (5, 8, 8), "l1.mix.ri.b": (5, 8), "l1.mix.lam": (40,), "l1.mix.o": (48, 40),
            "l1.mlp.router": (8, 48), "l1.mlp.correction": (8,), "l1.mlp.e7.gate": (24, 48), "l1.mlp.e0.up": (24, 48), "l1.mlp.e3.down": (48, 24),
            "l1.mlp.shared.gate": (16, 48), "l1.mlp.shared.up": (16, 48), "l1.mlp.shared.down": (48, 16),
            "l2.mlp.router": (6, 48), "l3.mix.conv": (64, 2), "l3.mix.ra": (1, 64, 64)}
    for k, shape in want.items():
        assert tuple(names[k].shape) == shape, k
    assert names["l3.norm2"].optional                                      # a layer without a feed-forward
    for absent in ("l1.mlp.shared.sg", "l1.mlp.router.b", "l1.mlp.e8.up", "l2.mlp.shared.gate", "l0.mix.sink", "l0.mix.o.b", "l1.mix.g"):
        assert absent not in names, absent


def test_what_the_cache_manager_is_asked_for():
    rt = Runtime(torch.device("cpu"), torch.float32, 8)
    needs = build_model(SumuvikConfig.from_dict(CONFIGS["S1"]), rt).cache_needs()
    assert needs[0] == PagedKV(2, 24, 11, keep_first=3) and needs[2] == PagedKV(2, 32, 19, keep_first=10)
    assert needs[(1, "memory")] == SlotState((40,), "float32") and needs[(1, "inputs")] == SlotState((3 * 40,), "float32")
    assert needs[(3, "memory")] == SlotState((64,), "float32") and needs[(3, "inputs")] == SlotState((64,), "float32")
    s2 = build_model(SumuvikConfig.from_dict(CONFIGS["S2"]), rt).cache_needs()
    assert (2, "inputs") not in s2 and (2, "memory") in s2                 # one tap: nothing to remember of the inputs
    s3 = build_model(SumuvikConfig.from_dict(CONFIGS["S3"]), rt).cache_needs()
    assert s3[0] == PagedKV(5, 8, None) and s3[1] == PagedKV(2, 20, 5, keep_first=9)
    # in bfloat16 the pages take the larger of the two head sizes, rounded up to the kernels' multiple of 16
    rt16 = Runtime(torch.device("cpu"), torch.bfloat16, 8)
    assert build_model(SumuvikConfig.from_dict(CONFIGS["S5"]), rt16).cache_needs()[0] == PagedKV(1, 32, 1, keep_first=2)


@pytest.mark.parametrize("key,value,text", [
    (("layers", 0, "type"), "conv", "neither 'attention' nor 'rglru'"),
    (("layers", 0, "mixer", "kv_heads"), 4, "not a multiple"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "even"),
    (("layers", 0, "mixer", "rot", "scaling", "high"), 0.5, "must exceed"),
    (("layers", 1, "mixer", "blocks"), 3, "not a multiple"),
    (("layers", 1, "mlp", "router", "groups", "count"), 3, "groups"),
    (("layers", 1, "mlp", "router", "top"), 5, "exceeds"),
    (("layers", 0, "mlp", "kind"), "sparse", "neither 'dense' nor 'moe'"),
    (("embedding",), None, "embedding"),
])
def test_errors_name_their_key(key, value, text):
    raw = copy.deepcopy(CONFIGS["S1"])
    at = raw
    for k in key[:-1]:
        at = at[k]
    at[key[-1]] = value
    with pytest.raises(ConfigError, match=text):
        SumuvikConfig.from_dict(raw)
    missing = copy.deepcopy(CONFIGS["S1"])
    del missing["layers"][0]["mlp"]["limit"]
    with pytest.raises(ConfigError, match="limit"):
        SumuvikConfig.from_dict(missing)


@pytest.mark.parametrize("rot", [
    {"base": 250.0, "dims": 16, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64.0}},     # all three ranges
    {"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "low": 2.0, "high": 3.0, "original": 1000.0}},
    {"base": 50.0, "dims": 6}, {"base": 7.0, "dims": 0}])
def test_stretched_frequencies(rot):
    rt = Runtime(torch.device("cpu"), torch.float32, 8)
    enc = POSITION_ENCODINGS.build(PartSpec("rotary_interleaved", {"theta": rot["base"], "rotary_dim": rot["dims"], "scaling": rot.get("scaling")}),
                                   rt, head_dim=32)
    r = enc.rotary()
    want = torch.tensor(frequencies(rot), dtype=torch.float64)
    assert r.rot == rot["dims"] and r.pairing == "interleaved" and r.inv_freq.dtype == torch.float32
    assert torch.allclose(r.inv_freq.double(), want, rtol=1e-7, atol=0)
    if rot.get("scaling") and rot["dims"] == 16:                         # the table holds kept, blended and stretched pairs
        plain = torch.tensor(frequencies({"base": rot["base"], "dims": rot["dims"]}), dtype=torch.float64)
        ratio = want / plain
        assert float(ratio[0]) == 1.0 and float(ratio[-1]) == 0.25 and any(0.25 < float(x) < 1.0 for x in ratio)


def test_kept_first_pages_stay_while_the_window_moves_on():
    """A window of 10 with 6 kept first positions on pages of 4: pages 0 and 1 are never given back, the pages between them and
    the window are, and come back to the pool; a group without kept positions gives back everything behind its window."""
    needs = {0: PagedKV(1, 16, 10, keep_first=6), 1: PagedKV(1, 16, 10)}
    m = CacheManager(needs, page_size=4, num_pages=12, max_num_seqs=2, max_model_len=96, prefix_caching=False)
    assert len(m.groups) == 2 and m.groups[0].keep_first == 6 and m.groups[1].keep_first == 0
    assert m.admit("a") == 0
    pos = 0
    for n in (7, 9, 1, 1, 14, 1, 8):                                      # 41 tokens in portions and single tokens
        assert m.grow("a", pos, pos + n)
        pos += n
        m.advance("a", pos, None)
        m.check()
        first_needed = max(0, pos - 10 + 1) // 4
        kept, plain = m.pages("a", 0), m.pages("a", 1)
        assert all(p >= 0 for p in kept[:2]), "the pages of the kept positions are held for the request's life"
        assert all((p >= 0) == (i < 2 or i >= first_needed) for i, p in enumerate(kept))
        assert all((p >= 0) == (i >= first_needed) for i, p in enumerate(plain))
        row = m.groups[0].table[m.slot("a")]
        assert all(row[i] == (p if p >= 0 else m.groups[0].scratch_page) for i, p in enumerate(kept))
    assert m.num_free_pages(0) == 12 - (2 + len(kept) - first_needed) and m.num_free_pages(1) == 12 - (len(plain) - first_needed)
    # what the request could still take counts the kept pages as held, not as returning
    assert m.room_for("a", pos) == (len(kept) + m.num_free_pages(0)) * 4 - pos < (len(plain) + m.num_free_pages(1)) * 4 - pos
    m.release("a")
    m.check()
    assert m.num_free_pages(0) == m.num_free_pages(1) == 12
    assert m.can_ever_hold(48) and not CacheManager(needs, page_size=4, num_pages=5, max_num_seqs=1, max_model_len=48).can_ever_hold(48)


def test_a_shared_prefix_of_a_window_with_kept_positions_brings_the_kept_pages():
    """Attention only (no state of fixed size), so prefixes are shared: a second request with the same first 24 tokens takes
    the kept pages and the pages its window reaches from the first one, and nothing in between."""
    needs = {0: PagedKV(1, 16, 6, keep_first=5)}
    m = CacheManager(needs, page_size=4, num_pages=16, max_num_seqs=2, max_model_len=64, prefix_caching=True)
    toks = list(range(100, 130))
    assert m.admit("a", toks) == 0 and m.grow("a", 0, 30)
    m.advance("a", 30, toks)
    held = m.pages("a", 0)
    assert [p >= 0 for p in held] == [True, True, False, False, False, False, True, True]
    other = toks[:26] + [7, 8, 9]
    m.release("a")                                         # its pages stay findable until something else needs the room
    assert m.admit("b", other) == 24                       # six full pages agree
    pages = m.pages("b", 0)
    assert [p >= 0 for p in pages] == [True, True, False, False, True, True] and pages[:2] == held[:2]
    row = m.groups[0].table[m.slot("b")]
    assert all(row[i] == (p if p >= 0 else m.groups[0].scratch_page) for i, p in enumerate(pages))
    assert m.grow("b", 24, 29)
    m.check()
