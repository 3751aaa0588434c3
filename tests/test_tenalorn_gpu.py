"""The Tenalorn decoder on the GPU against the plain implementation: every new kernel alone against a float64 loop written
here from its formula, then whole models (tiny configurations that differ in every size) replayed whole, with the last
tokens one by one, in portions down to two tokens, and mixed in a pool so small that pages and state slots are used
again; the edges of the chunks in prompts and in decoding; the previous token across portions and slots; decoding from
CUDA graphs; greedy generation through `Engine.generate` and the scheduler."""

import copy
import json
import subprocess
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from tests.gpu_helpers import BF16, F32, assert_close, i32, table_tensor
from tests.plain import tenalorn_plain as plain_model
from tests.plain.tenalorn_plain import PlainTenalorn, greedy_generate, logits_of
from tests.test_replay_gpu import cuts_changing, cuts_last32, cuts_whole, replay, steps_alone, steps_decode_together, steps_mixed
from tests.tiny import random_tokens
from tests.tiny_tenalorn import CONFIGS, PAGE_SIZE, write_tiny_tenalorn

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16]
F32_ATOL = 5e-5
BF16_REL = 0.05
LENGTHS = {"N1": [1, 5, 17, 70, 33, 130, 64], "N2": [7, 40, 64, 97, 2, 150]}
F64 = torch.float64


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def tol(adt):
    return F32 if adt == torch.float32 else BF16


# ------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("S,W", [(4, 48), (1, 203), (3, 1024), (5, 52), (2, 5120), (16, 40)])
def test_copies_of_the_stream_are_rebuilt_read_and_normed_in_one_kernel(adt, S, W):
    from tensorline_b200 import ops
    T = 9
    x0 = rnd(T, S * W, seed=1, scale=3.0)
    a, b = rnd(T, W, seed=2, dtype=adt), rnd(T, W, seed=3, dtype=adt)
    mix = torch.eye(S) + rnd(S, S, seed=4, scale=0.4)
    out, read, w = rnd(S, seed=5), rnd(S, seed=6), rnd(W, seed=7, dtype=adt)
    eps = 1e-5

    def plain(x, y, mix, out, read):
        X = x.double().view(T, S, W)
        if mix is not None:
            X = torch.einsum("sr,tsw->trw", mix.double(), X) + out.double()[None, :, None] * y[:, None, :]
        u = X.sum(1) if read is None else torch.einsum("r,trw->tw", read.double(), X)
        return X.reshape(T, S * W), u, plain_model.normed(u, w.double(), eps)

    # two addends with weights of their own, every copy rebuilt in place
    x = x0.clone().cuda()
    h = torch.empty(T, W, dtype=adt, device="cuda")
    u = torch.empty(T, W, dtype=torch.float32, device="cuda")
    ops.stream_step(x, S, a=a.cuda(), alpha=1.3, b=b.cuda(), beta=-0.6, mix=mix.cuda(), out=out.cuda(), read=read.cuda(), w=w.cuda(),
                    eps=eps, h=h, u=u)
    X, U, H = plain(x0, 1.3 * a.double() - 0.6 * b.double(), mix, out, read)
    assert_close(x, X, "copies", **F32)
    assert_close(u, U, "what is read", rtol=2e-5, atol=1e-4)
    assert_close(h, H, "normed", **tol(adt))
    # one addend, the plain sum, picked rows: the copies stay as they are
    x = x0.clone().cuda()
    rows = [7, 0, 3]
    h = torch.empty(3, W, dtype=adt, device="cuda")
    ops.stream_step(x, S, a=a.cuda(), mix=mix.cuda(), out=out.cuda(), w=w.cuda(), eps=eps, h=h, rows=i32(rows))
    assert torch.equal(x.cpu(), x0)
    assert_close(h, plain(x0, a.double(), mix, out, None)[2][rows], "picked rows", **tol(adt))
    # nothing to rebuild: a read and a norm
    h = torch.empty(T, W, dtype=adt, device="cuda")
    ops.stream_step(x, S, read=read.cuda(), w=w.cuda(), eps=eps, h=h)
    assert torch.equal(x.cpu(), x0)
    assert_close(h, plain(x0, None, None, None, read)[2], "read alone", **tol(adt))


@pytest.mark.parametrize("wdt", DT)
@pytest.mark.parametrize("copies", [1, 3])
def test_embedding_with_a_table_of_token_pairs_across_portions_and_slots(wdt, copies):
    """Three steps over four request slots: the previous token of a portion's first row comes from the slot (left there by
    the request's portion before, not by the slot's former owner and not by the row in front, which is another request's),
    a request's first token takes the table's last row, and a request may be left out of a step."""
    from tensorline_b200 import ops
    V, H, buckets, mp, mc = 50, 24, 13, 7, 5
    table, pairs = rnd(V, H, seed=1, dtype=wdt), rnd(buckets + 1, H, seed=2, dtype=wdt)
    seqs = {"a": random_tokens(V, 9, seed=3), "b": random_tokens(V, 4, seed=4), "c": random_tokens(V, 6, seed=5)}
    slot = {"a": 2, "b": 0, "c": 0}                          # c takes b's slot after b has ended
    steps = [[("a", 3), ("b", 4)], [("c", 2), ("a", 1)], [("a", 5), ("c", 4)]]
    last = torch.full((5,), 49, dtype=torch.int32, device="cuda")
    at = {k: 0 for k in seqs}
    cfg = {"scale": 2.5, "bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}
    want = {k: plain_model.embed(v, {"embed": table.double(), "bigram": pairs.double()}, cfg) for k, v in seqs.items()}
    for step in steps:
        ids, pos, req, q_start, slots = [], [], [], [0], []
        for rid, n in step:
            ids += seqs[rid][at[rid]:at[rid] + n]
            pos += list(range(at[rid], at[rid] + n))
            req += [slot[rid]] * n
            q_start.append(len(ids))
            slots.append(slot[rid])
        x = torch.empty(len(ids), copies * H, dtype=torch.float32, device="cuda")
        ops.embed_streams(x, table.cuda(), i32(ids), scale=2.5, copies=copies, pairs=pairs.cuda(), mul_prev=mp, mul_cur=mc,
                          pos=i32(pos), req_slot=i32(req), last_token=last)
        ops.remember_last(i32(ids), i32(q_start), i32(slots), last, len(step))
        row = 0
        for rid, n in step:
            for c in range(copies):
                assert_close(x[row:row + n, c * H:(c + 1) * H], want[rid][at[rid]:at[rid] + n], f"{rid} copy {c}", **F32)
            row += n
            at[rid] += n
    assert all(at[k] == len(v) for k, v in seqs.items())


def _chunk_attention_rows(q, k, v, pos_q, scale, chunk, slopes):
    """q [n, nq, d] at positions pos_q over k, v [len, nkv, d]: keys j <= p of p's own chunk, scores less slope * (p - j)."""
    n, nq, d = q.shape
    g = nq // k.shape[1]
    out = torch.empty(n, nq, v.shape[2], dtype=F64)
    for i, p in enumerate(pos_q):
        js = [j for j in range(p + 1) if chunk is None or j // chunk == p // chunk]
        dist = torch.tensor([float(p - j) for j in js], dtype=F64)
        for h in range(nq):
            s = (k[js, h // g] @ q[i, h]) * scale - (slopes[h] * dist if slopes is not None else 0.0)
            out[i, h] = torch.softmax(s, 0) @ v[js, h // g]
    return out


CHUNK_CASES = [  # nq, nkv, d, page, context lengths before the step, tokens in the step, chunk, slopes
    (4, 2, 16, 4, [0, 5, 31], [9, 1, 2], 6, True),
    (3, 1, 32, 8, [0, 130], [70, 3], 24, True),
    (8, 1, 64, 16, [300, 0, 65, 129], [1, 1, 1, 1], 96, True),         # single tokens; one at a chunk's first position + 12
    (6, 2, 48, 16, [63, 64, 1399], [1, 1, 1], 100, True),
    (4, 1, 64, 16, [119, 120, 239, 240], [1, 1, 1, 1], 120, True),     # the last position of a chunk and the first of the next
    (14, 2, 64, 64, [15, 0], [17, 200], 64, True),                     # chunks of exactly one page and one tile
    (5, 5, 80, 32, [257], [1], 33, False),                             # chunks without slopes
    (8, 2, 64, 8, [500, 129], [1, 1], None, True),                     # slopes without chunks: every earlier key
    (7, 1, 128, 16, [0, 700, 41], [200, 37, 90], 50, True),
    (2, 1, 64, 16, [0], [400], 1, True),                               # chunks of the token itself
    (4, 2, 64, 16, [100, 0, 517], [900, 300, 140], 130, True),         # long portions over several chunks
    (8, 2, 128, 32, [1000], [3], 2048, True),                          # a chunk longer than the request
]


@pytest.mark.parametrize("case", CHUNK_CASES, ids=[f"q{c[0]}kv{c[1]}d{c[2]}p{c[3]}c{c[6]}s{int(c[7])}" for c in CHUNK_CASES])
@pytest.mark.parametrize("kernel", ["exact_f32", "exact_bf16", "tensor_core_bf16", "tcgen05_bf16", "step_bf16"])
def test_attention_over_chunks_with_distance_slopes(case, kernel):
    """Decode and prefill attention over scattered pages, queries seeing their own chunk only and scores losing a slope per
    head times the distance, against the plain formula.  In the first request the first key of the last query's chunk and
    the key just in front of it carry planted scores: the query must see the one and not the other."""
    from tensorline_b200 import ops, ops_attention, ops_gemm
    nq, nkv, d, ps, ctx_lens, step_lens, chunk, sloped = case
    if kernel == "tcgen05_bf16" and (d % 64 or ps > 64):
        pytest.skip("the tcgen05 kernel takes head sizes that are multiples of 64")
    adt = torch.float32 if kernel == "exact_f32" else torch.bfloat16
    scale = 1.3 * d ** -0.5
    slopes = torch.tensor([2.0 ** (-6.0 * (h + 1) / nq) for h in range(nq)]) if sloped else None
    B = len(ctx_lens)
    max_pages, num_pages = 128, 300
    kps = torch.full((num_pages + 1, nkv, ps, d), 37.0, dtype=adt)
    vps = torch.full_like(kps, -53.0)
    rows, qs, want, pos_all, slot_all = [], [], [], [], []
    for b in range(B):
        n = ctx_lens[b] + step_lens[b]
        k, v = rnd(n, nkv, d, seed=20 + b, dtype=adt), rnd(n, nkv, d, seed=40 + b, dtype=adt)
        q = rnd(step_lens[b], nq, d, seed=60 + b, scale=2.0, dtype=adt)
        p_last = n - 1
        first = (p_last // chunk) * chunk if chunk else 0
        if b == 0 and first >= 1 and p_last > first:
            q[-1] *= 0; q[-1, :, 0] = 6.0
            k[first] *= 0; k[first, :, 0] = 6.0
            k[first - 1] *= 0; k[first - 1, :, 0] = 9.0
        need = -(-n // ps)
        gen = torch.Generator().manual_seed(100 + b)
        mine = (torch.randperm(num_pages // B, generator=gen)[:need] * B + b).tolist()
        for i in range(n):
            kps[mine[i // ps], :, i % ps] = k[i]
            vps[mine[i // ps], :, i % ps] = v[i]
        rows.append(mine)
        pq = list(range(ctx_lens[b], n))
        want.append(_chunk_attention_rows(q.double(), k.double(), v.double(), pq, scale, chunk,
                                          None if slopes is None else slopes.double()))
        qs.append(q)
        pos_all += pq
        slot_all += [b] * step_lens[b]
    q_all = torch.cat(qs).reshape(-1, nq * d).cuda()
    T = q_all.shape[0]
    out = torch.zeros(T, nq * d, dtype=adt, device="cuda")
    table = table_tensor(rows, max_pages, num_pages)
    kd, vd = kps.cuda(), vps.cuda()
    sl = None if slopes is None else slopes.cuda()
    q_start = [0]
    for n in step_lens:
        q_start.append(q_start[-1] + n)
    if kernel.startswith("exact"):
        ops.attn_tokenwise(q_all, nq * d, out, kd, vd, table, ps, i32(pos_all), i32(slot_all), nq, nkv, d, None, scale, chunk=chunk,
                           slopes=sl)
    elif kernel == "tensor_core_bf16":
        args = (q_all, nq * d, out, kd, vd, table, ps, i32(q_start), i32(ctx_lens), i32(list(range(B))))
        if all(n == 1 for n in step_lens):
            span = max(c + 1 for c in ctx_lens)
            if chunk:
                span = min(span, chunk + 63)
            for splits_wanted in (1, 3, 64):            # one range, a few, and more ranges than tiles
                tiles = -(-span // 64)
                splits = min(splits_wanted, tiles)
                rng = -(-tiles // splits) * 64
                splits = -(-tiles * 64 // rng)
                po = torch.full((B, nq, splits, d), float("nan"), device="cuda")
                pml = torch.full((B, nq, splits, 2), float("nan"), device="cuda")
                out.zero_()
                ops_attention.decode(*args, B, nq, nkv, d, None, scale, rng, splits, po, pml, mask_chunk=chunk, slopes=sl)
                assert_close(out.view(T, nq, d), torch.cat(want), f"decode, {splits} ranges", **BF16)
            out.zero_()
        ops_attention.prefill(*args, q_start, nq, nkv, d, None, scale, chunk=chunk, slopes=sl)
    elif kernel == "tcgen05_bf16":                      # the one-tile kernel
        ops_attention.prefill_tc(q_all, nq * d, out, kd, vd, table, ps, i32(q_start), i32(ctx_lens), i32(list(range(B))), q_start,
                                 nq, nkv, d, None, scale, chunk=chunk, slopes=sl)
    else:                                               # the step's own choice of kernels
        qkv = torch.zeros(T, (nq + 2 * nkv) * d, dtype=adt, device="cuda")
        qkv[:, :nq * d] = q_all
        ctx = SimpleNamespace(B=B, T=T, decode_only=all(n == 1 for n in step_lens), page_size=ps, q_start=i32(q_start), start_pos=i32(ctx_lens),
                              slots=i32(list(range(B))), h_q_start=q_start, h_start_pos=list(ctx_lens), h_slots=list(range(B)),
                              graph_max_ctx=0, max_ctx=max(c + n for c, n in zip(ctx_lens, step_lens)), scratch={})
        ops_attention.attend_bf16(qkv, out, ctx, kd, vd, table, nq, nkv, d, None, scale, chunk=chunk, slopes=sl)
    ops_gemm.check_status()
    assert_close(out.view(T, nq, d), torch.cat(want), kernel, **tol(adt))
    # the oracle itself tells chunks that are one position off, and slopes that are left out
    n0 = ctx_lens[0] + step_lens[0]
    first = ((n0 - 1) // chunk) * chunk if chunk else 0
    if first >= 1 and n0 - 1 > first:
        k0 = torch.stack([kps[rows[0][i // ps], :, i % ps] for i in range(n0)]).double()
        v0 = torch.stack([vps[rows[0][i // ps], :, i % ps] for i in range(n0)]).double()
        last = qs[0][-1:].double()
        right = _chunk_attention_rows(last, k0, v0, [n0 - 1], scale, chunk, None if slopes is None else slopes.double())
        for c2 in (chunk + 1, chunk - 1) if chunk > 1 else (chunk + 1,):
            if ((n0 - 1) // c2) * c2 == first:
                continue
            other = _chunk_attention_rows(last, k0, v0, [n0 - 1], scale, c2, None if slopes is None else slopes.double())
            assert float((other - right).abs().max()) > 1e-3, f"chunks of {c2} must show"


@pytest.mark.parametrize("E,ident,top", [(8, 4, 3), (6, 2, 3), (4, 0, 4), (2, 2, 1), (5, 3, 8), (60, 4, 8), (3, 1, 2)])
def test_choice_by_share_of_a_softmax_with_identity_entries(E, ident, top):
    """The router's choice (softmax over all entries, a correction that only steers the choice, weights by share) and the
    streamed experts, where an entry behind the experts' stands for the token's own row."""
    from tensorline_b200 import ops
    T, K, F, N = 23, 40, 24, E + ident
    h = rnd(T, K, seed=1)
    w = {"router": rnd(N, K, seed=2, scale=0.5), "correction": rnd(N, seed=3, scale=0.1)}
    for e in range(E):
        w.update({f"e{e}.gate": rnd(F, K, seed=10 + e, scale=0.3), f"e{e}.up": rnd(F, K, seed=40 + e, scale=0.3),
                  f"e{e}.down": rnd(K, F, seed=70 + e, scale=0.3)})
    c = {"router": {"experts": E, "identity": ident, "top": top}}
    want_route = plain_model.route(h.double(), {k: v.double() for k, v in w.items()}, c)
    z = (h.double() @ w["router"].double().T).float().cuda()
    idx = torch.empty(T, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(T, top, dtype=torch.float32, device="cuda")
    ops.route_groups(z, w["correction"].cuda(), top, 1, 1, 2, 1.0, idx, wts, softmax=True)
    got = [sorted(zip(idx[t].tolist(), wts[t].tolist())) for t in range(T)]
    for t in range(T):
        ref = sorted(want_route[t])
        assert [e for e, _ in got[t]] == [e for e, _ in ref], f"token {t}"
        assert_close(torch.tensor([x for _, x in got[t]]), torch.tensor([x for _, x in ref]), f"weights of token {t}", **F32)
    assert ident == 0 or any(e >= E for row in got for e, _ in row), "no identity entry was ever chosen"
    w_up = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(E)]).cuda()
    w_down = torch.stack([w[f"e{e}.down"] for e in range(E)]).cuda()
    a = torch.full((T * top, F), float("nan"), dtype=torch.float32, device="cuda")
    y = torch.empty(T, K, dtype=torch.float32, device="cuda")
    ops.moe_up(h.cuda(), w_up, idx, a, act="silu", gated=True)
    ops.moe_down(a, w_down, idx, wts, y, same=h.cuda())
    assert_close(y, plain_model.experts(h.double(), {k: v.double() for k, v in w.items()}, c), "experts", rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("adt", DT)
def test_latent_rows_with_neighbouring_pairs_and_no_query_latent(adt):
    from tensorline_b200 import ops
    T, rank, dr, rot, more, ps, d = 7, 12, 8, 6, 5, 4, 24
    down = rnd(T, rank + dr + more, seed=1)
    wkv = rnd(rank, seed=2, dtype=adt)
    pos = [0, 1, 2, 9, 10, 3, 40]
    slot = [0, 0, 0, 1, 1, 0, 2]
    table = table_tensor([[3, 5], [1, 1, 7], [2] * 11], 12, 8)
    pages = torch.zeros(9, 1, ps, d, dtype=adt, device="cuda")
    inv = torch.tensor([30.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32)
    ops.latent_prep(down.cuda(), 0, rank, dr, None, wkv.cuda(), 1e-5, inv.cuda(), rot, i32(pos), i32(slot), table, ps, None, pages,
                    pairing="interleaved")
    H, dk = 3, 5
    q = rnd(T, H * (dk + dr), seed=3, dtype=adt)
    qa = torch.full((T, H * d), float("nan"), dtype=adt, device="cuda")
    ops.latent_qrot(q.cuda(), dk, dr, inv.cuda(), rot, i32(pos), qa, rank, H, pairing="interleaved")
    for t in range(T):
        c = plain_model.normed(down[t, :rank].double(), wkv.double(), 1e-5)
        turned = plain_model.turn_pairs(torch.stack([torch.zeros(dr, dtype=F64)] * pos[t] + [down[t, rank:rank + dr].double()]),
                                        {"base": 30.0}, rot)[-1]
        row = pages[table[slot[t], pos[t] // ps], 0, pos[t] % ps]
        assert_close(row, torch.cat([c, turned, torch.zeros(d - rank - dr, dtype=F64)]), f"page row of token {t}", **tol(adt))
        for a in range(H):
            src = q[t].view(H, dk + dr)[a, dk:].double()
            tq = plain_model.turn_pairs(torch.stack([torch.zeros(dr, dtype=F64)] * pos[t] + [src]), {"base": 30.0}, rot)[-1]
            assert_close(qa[t].view(H, d)[a, rank:], torch.cat([tq, torch.zeros(d - rank - dr, dtype=F64)]), f"query {t}, head {a}", **tol(adt))


@pytest.mark.parametrize("adt", DT)
def test_cap_on_the_logits_and_sigmoid_gate(adt):
    from tensorline_b200 import ops
    z = rnd(5, 77, seed=1, scale=40.0)
    zc = z.clone().cuda()
    ops.softcap(zc, 30.0)
    assert_close(zc, 30.0 * torch.tanh(z.double() / 30.0), "cap", **F32)
    o, g = rnd(6, 40, seed=2, dtype=adt), rnd(6, 90, seed=3, scale=3.0)
    y = torch.empty(6, 40, dtype=adt, device="cuda")
    ops.sigmoid_gate(o.cuda(), g.cuda()[:, 50:], y)
    assert_close(y, o.double() * plain_model.sig(g[:, 50:].double()), "gate", **tol(adt))


# ------------------------------------------------------------------------------------------ whole models
@pytest.fixture(scope="module", params=["N1", "N2"])
def model(request, tmp_path_factory):
    name = request.param
    folder = write_tiny_tenalorn(name, tmp_path_factory.mktemp(f"tiny_{name}"))
    plain = PlainTenalorn(folder)
    V = CONFIGS[name]["vocab"]
    reqs = {f"r{i}": random_tokens(V, n, seed=100 + i) for i, n in enumerate(LENGTHS[name])}
    want = {rid: logits_of(plain, toks) for rid, toks in reqs.items()}
    return dict(name=name, folder=folder, reqs=reqs, want=want, page=PAGE_SIZE[name], vocab=V, plain=plain)


def check(model, dtype, got, what):
    """32-bit: every position within F32_ATOL (times the largest |logit| where that is above one), but for one position in a
    hundred, which may be off by ten times that: the plain model itself, run in float32, is off by four times the bound at such
    a position (a denominator of the matrix memory near a cancellation), measured on the largest tiny model.  bfloat16: the largest logit
    error of a position as a share of the request's largest |logit|: four positions in five within BF16_REL, every one within
    that largest |logit| (a score near a tie picks another entry in bfloat16; the 32-bit runs pin those positions)."""
    assert got, "nothing was compared"
    over = hard = 0
    for (rid, p), row in got.items():
        ref = model["want"][rid][p]
        err = float((row - ref).abs().max())
        if dtype == "float32":
            bound = F32_ATOL * max(1.0, float(ref.abs().max()))
            assert err <= 10 * bound, f"{what}: request {rid} position {p}: max abs err {err:.3e} > {10 * bound:.3e}"
            hard += err > bound
        else:
            top = float(model["want"][rid].abs().max())
            assert err <= top, f"{what}: request {rid} position {p}: max abs err {err:.3e} > {top:.3e}"
            over += err > BF16_REL * top
    assert over <= 0.2 * len(got), f"{what}: {over} of {len(got)} positions are beyond the bfloat16 bound"
    assert hard <= 0.01 * len(got), f"{what}: {hard} of {len(got)} positions are beyond the 32-bit bound"


def test_the_model_is_chosen_by_its_configuration_and_every_layer_matches(model):
    """The sum of the stream's copies after every layer, 32-bit engine against the plain model."""
    from tensorline_b200 import ops
    from tensorline_b200.parts.linear import StreamUpdate, WeightedPair
    from tensorline_b200.replay import TraceSession, make_runner
    runner, cfg = make_runner(model["folder"], "float32", 256, page_size=model["page"], max_live=2)
    assert type(cfg).__name__ == "TenalornConfig" and cfg.to_json_dict() == CONFIGS[model["name"]]
    seen = []
    W = CONFIGS[model["name"]]["width"]
    for blk in runner.model.blocks:
        def fwd(x, pending, ctx, cache, orig=blk.forward):
            out = orig(x, pending, ctx, cache)
            assert isinstance(out, StreamUpdate)
            v = out.value
            kw = dict(a=v.a, alpha=v.alpha, b=v.b, beta=v.beta) if isinstance(v, WeightedPair) else dict(a=v)
            u = torch.empty((x.shape[0], W), dtype=torch.float32, device=x.device)
            ops.stream_step(x, x.shape[1] // W, mix=out.mix, out=out.out, u=u, rows=i32(list(range(x.shape[0]))), **kw)
            seen.append(u.double().cpu())
            return out
        blk.forward = fwd
    toks = model["reqs"]["r2"]
    TraceSession(runner).run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": ["a"]})
    want = []
    logits_of(model["plain"], toks, want)
    assert len(seen) == len(want) == len(CONFIGS[model["name"]]["layers"])
    for i, (g, w) in enumerate(zip(seen, want)):
        assert_close(g, w, f"sum of the copies after layer {i}", rtol=5e-5, atol=F32_ATOL * max(1.0, float(w.abs().max())))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_schedules_agree_with_the_plain_model(model, dtype):
    results = {}
    for what, cuts in (("whole", cuts_whole), ("last 32 one by one", cuts_last32), ("changing portions", cuts_changing)):
        results[what] = replay(model, dtype, steps_alone(model, cuts), max_tokens=192)
        check(model, dtype, results[what], what)
        assert len(results[what]) == sum(len(t) for t in model["reqs"].values())
    for seed in (1, 2):
        steps, peak = steps_mixed(model, seed)
        assert max(len(s["entries"]) for s in steps) >= 3
        total = sum(-(-len(t) // model["page"]) * model["page"] for t in model["reqs"].values())
        assert peak < total, "the pool must be too small to hold all requests: pages and slots have to be used again"
        results[f"mixed {seed}"] = replay(model, dtype, steps, max_tokens=peak)
        check(model, dtype, results[f"mixed {seed}"], f"mixed {seed}")
        assert len(results[f"mixed {seed}"]) == len(results["whole"])
    if dtype == "float32":                                  # one order of additions per position
        for what, got in results.items():
            for key, row in got.items():
                assert torch.equal(row, results["whole"][key]), f"{what} differs from whole at {key}"


def test_the_forms_of_long_steps_agree_with_the_plain_model(model, monkeypatch):
    """The bfloat16 engine's forms for long steps (experts sorted and run as batched products, identity entries passing their
    rows; the latent's products per head through one batched product) taken from two tokens on."""
    from tensorline_b200.parts import latent, moe
    monkeypatch.setattr(moe, "STREAM_MAX_TOKENS", 1)
    monkeypatch.setattr(latent, "HEAD_PRODUCT_LIBRARY_MIN_TOKENS", 2)
    for what, steps, most in (("whole", steps_alone(model, cuts_whole), 192), ("changing portions", steps_alone(model, cuts_changing), 192),
                              ("mixed", *steps_mixed(model, 3))):
        got = replay(model, "bfloat16", steps, max_tokens=most)
        check(model, "bfloat16", got, f"long forms, {what}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(model, dtype):
    """A one-token prompt, then 150 tokens decoded one by one: the matrix memory, the previous token and the pages are
    carried through 150 launches, and every chunk's edge is passed by decoded tokens."""
    toks = random_tokens(model["vocab"], 151, seed=7)
    want = logits_of(model["plain"], toks)
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    steps[-1]["end"] = ["x"]
    m2 = dict(model, reqs={"x": toks}, want={"x": want})
    got = replay(m2, dtype, steps, max_tokens=160)
    check(m2, dtype, got, "token by token")
    assert sorted(p for _, p in got) == list(range(151))


def _other_chunks(raw, by):
    raw = copy.deepcopy(raw)
    for layer in raw["layers"]:
        if "mask" in layer["mixer"].get("left", {}):
            layer["mixer"]["left"]["mask"]["size"] += by
    return raw


def test_edges_of_chunks_and_what_the_plain_model_tells(model):
    """The plain model with every chunk one position longer or shorter gives other logits from the first position on that a
    chunk's edge cuts, and the plain model with another hash of the token pairs from the second token on: a key that is
    wrongly seen (or not seen) and a wrong previous token show.  The engine follows the right one: whole, with the tokens around every edge decoded one by one, and in portions that end on
    both sides of the edges."""
    toks = random_tokens(model["vocab"], 90, seed=11)
    right = logits_of(model["plain"], toks)
    sizes = sorted({l["mixer"]["left"]["mask"]["size"] for l in CONFIGS[model["name"]]["layers"] if "mask" in l["mixer"].get("left", {})})
    first = sizes[0]                                        # the first position that a chunk's edge cuts
    for by in (-1, 1):
        other = PlainTenalorn(model["folder"])
        other.cfg = _other_chunks(other.cfg, by)
        gap = (logits_of(other, toks) - right).abs().max(1).values
        assert float(gap[:first - 1].max()) == 0.0
        assert float(gap.max()) > 100 * F32_ATOL, f"the plain model must tell chunks that are one position off ({by})"
    other = PlainTenalorn(model["folder"])
    other.cfg = copy.deepcopy(other.cfg)
    other.cfg["embedding"]["bigram"]["mul_prev"] += 1
    gap = (logits_of(other, toks) - right).abs().max(1).values
    assert float(gap[0]) == 0.0 and float(gap[1:].median()) > 100 * F32_ATOL, "the previous token must show"
    m2 = dict(model, reqs={"w": toks}, want={"w": right})
    edges = sorted({e * k + j for e in sizes for k in (1, 2, 3) for j in (-1, 0, 1) if 0 < e * k + j < 90})
    cuts = [[90], [first - 1] + [1] * (91 - first), [e2 - e1 for e1, e2 in zip([0] + edges, edges + [90]) if e2 > e1]]
    for dtype in ("float32", "bfloat16"):
        for c in cuts:
            assert sum(c) == 90
            got = replay(m2, dtype, steps_alone(m2, lambda n, c=c: c), max_tokens=96)
            check(m2, dtype, got, f"chunk edges, portions {c[:4]}...")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_graphs_agree_with_eager_steps(model, dtype):
    """Steps of single tokens replayed from CUDA graphs (state slots are fixed addresses, padding rows use the spare
    slot): three live requests in the bucket of four, shrinking as they end; 32-bit: the bits of the eager steps."""
    rids = ["r3", "r5", "r2"]
    steps, decode_steps = steps_decode_together(model, rids, tail=12)
    eager = replay(model, dtype, steps, max_tokens=512)
    graphs = {}

    def after(runner):
        graphs["replays"] = runner.graph_replays
    got = replay(model, dtype, steps, max_tokens=512, graphs=True, after=after)
    assert graphs["replays"] == decode_steps
    check(model, dtype, got, "decode graphs")
    if dtype == "float32":
        for key, row in got.items():
            assert torch.equal(row, eager[key]), f"graph replay differs from the eager step at {key}"


def test_greedy_generation_through_the_engine_and_its_scheduler(model):
    """`Engine.generate`: five prompts through three slots and a small pool (queueing, slots and pages used again,
    portions of 16 tokens), 32-bit, against greedy decoding with the plain model."""
    from tensorline_b200 import Engine, SamplingParams
    prompts = [random_tokens(model["vocab"], n, seed=50 + n) for n in (9, 2, 40, 5, 21)]
    want = [greedy_generate(model["plain"], p, 8) for p in prompts]
    for graphs in (False, True):
        eng = Engine(str(model["folder"]), dtype="float32", block_size=model["page"], num_blocks=160 // model["page"], max_num_seqs=3,
                     max_model_len=64, max_batched_tokens=16, cuda_graphs=graphs, overlap=graphs)
        got = [o.token_ids for o in eng.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
        assert got == want, f"graphs {graphs}: {got} != {want}"
        st = eng.stats()
        assert st["free_pages"] == st["num_pages"] and st["max_running_seen"] == 3 and (st["graph_replays"] > 0) == graphs


@pytest.mark.parametrize("name", ["N3", "N4", "N5", "N6"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_further_shapes_of_the_design(name, dtype, tmp_path):
    """One plain stream without a table of pairs, a cap or chunks; one copy with its tensors, chunks of a single position and
    every router entry chosen; sizes that are multiples of nothing much with five copies; sizes that the tensor-core kernels
    take, with prompts of hundreds of tokens over several chunks: whole requests, changing portions and a small pool against
    the plain model."""
    folder = write_tiny_tenalorn(name, tmp_path / name)
    plain = PlainTenalorn(folder)
    V = CONFIGS[name]["vocab"]
    lengths = [290, 3, 400, 130] if name == "N6" else [3, 50, 1, 81, 33]
    reqs = {f"r{i}": random_tokens(V, n, seed=300 + i) for i, n in enumerate(lengths)}
    m = dict(name=name, folder=folder, reqs=reqs, want={r: logits_of(plain, t) for r, t in reqs.items()}, page=PAGE_SIZE[name], vocab=V)
    whole = replay(m, dtype, steps_alone(m, cuts_whole), max_tokens=max(128, -(-max(lengths) // 64) * 64))
    check(m, dtype, whole, "whole")
    cut = replay(m, dtype, steps_alone(m, cuts_changing), max_tokens=max(128, -(-max(lengths) // 64) * 64))
    check(m, dtype, cut, "changing portions")
    steps, peak = steps_mixed(m, 3, max_live=3)
    mixed = replay(m, dtype, steps, max_tokens=peak)
    check(m, dtype, mixed, "mixed")
    if dtype == "float32":
        assert all(torch.equal(cut[k], whole[k]) and torch.equal(mixed[k], whole[k]) for k in whole)


def test_generate_from_the_command_line(model, capsys):
    """The `tensorline` command with token ids, 32-bit, against greedy decoding with the plain model."""
    from tensorline_b200 import cli
    assert cli.main(["--model", str(model["folder"]), "--dtype", "float32", "--prompt-ids", "5,9,40,17", "--prompt-ids", "7",
                     "--max-tokens", "5", "--ignore-eos", "--block-size", str(model["page"]), "--num-blocks", "16",
                     "--max-num-seqs", "4", "--max-model-len", "64"]) == 0
    import json
    lines = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert [l["token_ids"] for l in lines] == [greedy_generate(model["plain"], [5, 9, 40, 17], 5), greedy_generate(model["plain"], [7], 5)]


def test_the_replay_program_with_this_design(model, tmp_path):
    """`bin/trace_run` itself, 32-bit: JSON lines in, `done <step>` lines and <step>.f32 files out; a request that is left
    out of a step, one that starts in another's freed slot, portions of two tokens."""
    if model["name"] != "N1":
        pytest.skip("one configuration is enough for the command-line protocol")
    reqs = model["reqs"]
    a, b, c = reqs["r3"], reqs["r4"], reqs["r2"]
    lines = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:2], "want": [1]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[2:], "want": [len(b) - 3]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[30:32], "want": []}, {"id": "c", "tokens": c, "want": [len(c) - 1]}], "end": ["c"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[32:], "want": [len(a) - 33]}], "end": ["a"]},
    ]
    out = tmp_path / "out"
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(model["folder"]), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "128", "--page-size", "8", "--max-live", "2"],
                          input="".join(json.dumps(l) + "\n" for l in lines), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    assert sorted(p.name for p in out.iterdir()) == ["0.f32", "1.f32", "2.f32", "3.f32"]
    V = model["vocab"]
    got = {n: torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, V).astype(np.float64)) for n in range(4)}
    assert [got[n].shape[0] for n in range(4)] == [3, 1, 1, 1]
    wa, wb, wc = model["want"]["r3"], model["want"]["r4"], model["want"]["r2"]
    for row, ref in ((got[0][0], wa[0]), (got[0][1], wa[29]), (got[0][2], wb[1]), (got[1][0], wb[-1]), (got[2][0], wc[-1]), (got[3][0], wa[-1])):
        assert float((row - ref).abs().max()) <= F32_ATOL * max(1.0, float(ref.abs().max()))
