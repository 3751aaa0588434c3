"""The Sumuvik decoder on the GPU against the plain implementation: every new kernel alone against a float64 loop written
here from its formula, then whole models (tiny configurations that differ in every size) replayed whole, with the last
tokens one by one, in portions down to two tokens, and mixed in a pool so small that pages and state slots are used
again; the edges of windows and of the kept first tokens in prompts and in decoding; the one in the softmax's
denominator; decoding from CUDA graphs; greedy generation through `Engine.generate` and the scheduler."""

import copy
from types import SimpleNamespace

import pytest
import torch

from tests.gpu_helpers import BF16, F32, assert_close, i32, table_tensor
from tests.plain import sumuvik_plain as plain_model
from tests.plain.sumuvik_plain import PlainSumuvik, forward, greedy_generate
from tests.test_replay_gpu import cuts_changing, cuts_last32, cuts_whole, replay, steps_alone, steps_decode_together, steps_mixed
from tests.tiny import random_tokens
from tests.tiny_sumuvik import CONFIGS, PAGE_SIZE, write_tiny_sumuvik

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16]
F32_ATOL = 5e-5
BF16_REL = 0.05
LENGTHS = {"S1": [1, 5, 17, 70, 33, 130, 64], "S2": [7, 40, 64, 97, 2, 150]}
F64 = torch.float64


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def tol(adt):
    return F32 if adt == torch.float32 else BF16


# ------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("H", [48, 203, 1024, 5120, 12288, 20480])
def test_two_norms_of_one_stream_and_the_sum_of_two_outputs(adt, H):
    """x += a + b; h1 = x / rms(x) * w1, h2 = x / rms(x) * w2; with one addend, with none, with one norm, with picked rows."""
    from tensorline_b200 import ops
    T, eps = 9, 1e-5
    x0 = rnd(T, H, seed=1, scale=3.0)
    a, b = rnd(T, H, seed=2, scale=0.3, dtype=adt), rnd(T, H, seed=3, scale=0.3, dtype=adt)
    w1, w2 = (1 + rnd(H, seed=4, scale=0.2)).to(torch.bfloat16), (1 + rnd(H, seed=5, scale=0.2)).to(torch.bfloat16)

    def unit(v):
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)
    for aa, bb in ((a, b), (a, None), (None, None)):
        want_x = x0.double() + (0 if aa is None else aa.double()) + (0 if bb is None else bb.double())
        x = x0.clone().cuda()
        h1, h2 = torch.empty(T, H, dtype=adt, device="cuda"), torch.empty(T, H, dtype=adt, device="cuda")
        ops.add_rmsnorm_pair(x, None if aa is None else aa.cuda(), None if bb is None else bb.cuda(), w1.cuda(), w2.cuda(), h1, h2, eps)
        assert_close(x, want_x, "stream", **F32)
        assert_close(h1, unit(want_x) * w1.double(), "first norm", **tol(adt))
        assert_close(h2, unit(want_x) * w2.double(), "second norm", **tol(adt))
        rows = i32([7, 0, 3])
        x2, g1 = x0.clone().cuda(), torch.empty(3, H, dtype=adt, device="cuda")
        ops.add_rmsnorm_pair(x2, None if aa is None else aa.cuda(), None if bb is None else bb.cuda(), w1.cuda(), None, g1, None, eps, rows=rows)
        assert torch.equal(x2.cpu(), x0) and torch.equal(g1, h1[rows.long()])
    with pytest.raises(ops.KernelError):
        ops.add_rmsnorm_pair(x0.clone().cuda(), None, b.cuda(), w1.cuda(), None, h1, None, eps)


@pytest.mark.parametrize("wdt", DT)
def test_embedding_rows_times_a_constant(wdt):
    from tensorline_b200 import ops
    table = rnd(50, 72, seed=1, dtype=wdt)
    ids = [3, 49, 0, 3, 17]
    x = torch.empty(5, 72, dtype=torch.float32, device="cuda")
    ops.embed(x, table.cuda(), i32(ids), scale=16.5)
    assert torch.equal(x.cpu(), table[ids].float() * 16.5)
    ops.embed(x, table.cuda(), i32(ids))
    assert torch.equal(x.cpu(), table[ids].float())


def _swish_clamped(g, u, limit, alpha):
    g, u = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
    return g * plain_model.sig(alpha * g) * (u + 1.0)


@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("block", [None, 8])
def test_clamped_swish(adt, block):
    """Pre-activations on both sides of the limits, also far beyond them; the plain layout and gate and up in blocks."""
    from tensorline_b200 import ops
    I, limit, alpha = 72, 1.5, 1.702
    g, u = rnd(37, I, seed=1, scale=2.5, dtype=adt), rnd(37, I, seed=2, scale=2.5, dtype=adt)
    g[0, :4], u[0, :4] = torch.tensor([40.0, -40.0, 1.5, -1.5]).to(adt), torch.tensor([-30.0, 30.0, 1.5, -1.5]).to(adt)
    if block is None:
        gu = torch.cat([g, u], dim=1)
    else:
        gu = torch.stack((g.view(37, I // block, block), u.view(37, I // block, block)), dim=2).reshape(37, 2 * I)
    out = torch.empty(37, I, dtype=adt, device="cuda")
    ops.silu_mul(gu.contiguous().cuda(), out, block=block, act=("swish_clamped", limit, alpha))
    assert_close(out, _swish_clamped(g.double(), u.double(), limit, alpha), "clamped swish", **tol(adt))
    with pytest.raises(ops.KernelError):
        ops.silu_mul(gu.contiguous().cuda(), out, block=block, act="swish_clamped")          # its constants are missing


@pytest.mark.parametrize("T", [8, 37, 700])
def test_clamped_swish_in_the_epilogue_of_the_tensor_core_products(T):
    """Both tcgen05 products with the clamped swish in their epilogue: bit for bit the product, stored in bfloat16,
    followed by the activation kernel, and the formula in float64; another launch with other constants follows them."""
    from tensorline_b200 import ops, ops_gemm
    I, K = 320, 520
    x = rnd(T, K, seed=1, dtype=torch.bfloat16).cuda()
    g, u = rnd(I, K, seed=2, scale=0.1, dtype=torch.bfloat16), rnd(I, K, seed=3, scale=0.1, dtype=torch.bfloat16)
    w = torch.stack((g.view(I // 64, 64, K), u.view(I // 64, 64, K)), dim=1).reshape(2 * I, K).contiguous().cuda()
    gd, ud = x.double().cpu() @ g.double().T, x.double().cpu() @ u.double().T
    for act in (("swish_clamped", 1.25, 1.702), ("swish_clamped", 3.0, 1.0)):
        if T <= 64:
            kw = dict(swap=1, bn=16 if T <= 16 else 64, splits=1)
            got, gu = ops_gemm.gemm_tc(x, w, gated=act, **kw), ops_gemm.gemm_tc(x, w, **kw)
        else:
            got, gu = ops_gemm.gemm_tc2(x, w, gated=act), ops_gemm.gemm_tc2(x, w)
        ops_gemm.check_status()
        two_pass = torch.empty(T, I, dtype=torch.bfloat16, device="cuda")
        ops.silu_mul(gu, two_pass, block=64, act=act)
        assert torch.equal(got, two_pass)
        assert float((gd.abs() > act[1]).double().mean()) > 0.02, "some pre-activations must lie beyond the limit"
        assert_close(got, _swish_clamped(gd, ud, act[1], act[2]), "clamped swish in the epilogue", rtol=3e-2, atol=3e-2)


def _masked_attention_rows(q, k, v, pos_q, scale, window, keep, sink, gate):
    """q [n, nq, d] at positions pos_q over k, v [len, nkv, d]: keys j <= p with p - j < window or j < keep; the denominator
    also holds exp(sink) (a number or None); row (i, h) times sigmoid(gate[i, h]) (or no gate)."""
    n, nq, d = q.shape
    g = nq // k.shape[1]
    out = torch.empty(n, nq, v.shape[2], dtype=F64)
    for i, p in enumerate(pos_q):
        js = [j for j in range(p + 1) if window is None or p - j < window or j < keep]
        for h in range(nq):
            s = (k[js, h // g] @ q[i, h]) * scale
            m = max(float(s.max()), sink if sink is not None else -1e300)
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(torch.tensor(sink - m, dtype=F64)) if sink is not None else 0.0)
            o = (e / den) @ v[js, h // g]
            out[i, h] = o * (plain_model.sig(gate[i, h]) if gate is not None else 1.0)
    return out


MASK_CASES = [  # nq, nkv, d, page, context lengths before the step, tokens in the step, window, kept first
    (4, 2, 16, 4, [0, 5, 31], [9, 1, 2], 6, 3),
    (3, 1, 32, 8, [0, 130], [70, 3], 24, 9),
    (8, 1, 64, 16, [300, 0, 65, 129], [1, 1, 1, 1], 96, 20),          # single tokens: the window has left the kept keys far behind
    (6, 2, 48, 16, [63, 64, 1399], [1, 1, 1], 100, 70),               # kept keys over more than one tile of 64
    (14, 2, 64, 64, [15, 0], [17, 200], 100, 64),                     # kept keys exactly one page and one tile
    (5, 5, 80, 32, [257], [1], 33, 1),
    (8, 2, 64, 8, [500, 129], [1, 1], 200, 130),
    (7, 1, 128, 16, [0, 700, 41], [200, 37, 90], 64, 5),
    (4, 4, 16, 2, [30], [150], 50, 200),                              # more kept keys than the request has tokens: every key stays
    (2, 1, 64, 16, [0], [400], 1, 2),                                 # a window of the token itself beside two kept keys
    (6, 2, 64, 16, [1000, 90], [1, 1], 128, 0),                       # no kept keys: the plain window
    (4, 2, 64, 16, [100, 0, 517], [900, 300, 140], 130, 70),          # long portions: kept keys over two tiles, far under the window
    (8, 2, 128, 32, [0], [700], 200, 64),                             # kept keys exactly one tile
]


@pytest.mark.parametrize("case", MASK_CASES, ids=[f"q{c[0]}kv{c[1]}d{c[2]}p{c[3]}w{c[6]}k{c[7]}" for c in MASK_CASES])
@pytest.mark.parametrize("kernel", ["exact_f32", "exact_bf16", "tensor_core_bf16", "tcgen05_bf16", "step_bf16"])
def test_attention_with_kept_first_keys_a_one_in_the_denominator_and_a_gate(case, kernel):
    """Decode and prefill attention over scattered pages with a window that also keeps the first keys, against the plain
    formula.  In the first request a kept key far behind the window and the key at the window's edge carry planted scores:
    the last query must give most of its weight to them, and none to the planted key just outside both."""
    from tensorline_b200 import ops, ops_attention, ops_gemm
    nq, nkv, d, ps, ctx_lens, step_lens, window, keep = case
    if kernel == "tcgen05_bf16" and (d % 64 or ps > 64):
        pytest.skip("the tcgen05 kernel takes head sizes that are multiples of 64")
    adt = torch.float32 if kernel == "exact_f32" else torch.bfloat16
    scale = 1.3 * d ** -0.5
    B = len(ctx_lens)
    max_pages, num_pages = 128, 300
    kps = torch.full((num_pages + 1, nkv, ps, d), 37.0, dtype=adt)
    vps = torch.full_like(kps, -53.0)
    sink = torch.zeros(nq)
    rows, qs, want, pos_all, slot_all, gates = [], [], [], [], [], []
    for b in range(B):
        n = ctx_lens[b] + step_lens[b]
        k, v = rnd(n, nkv, d, seed=20 + b, dtype=adt), rnd(n, nkv, d, seed=40 + b, dtype=adt)
        q = rnd(step_lens[b], nq, d, seed=60 + b, scale=2.0, dtype=adt)
        gate = rnd(step_lens[b], nq, seed=80 + b, scale=2.0)
        p_last = n - 1
        if b == 0 and n > window + keep + 2 and keep > 0:
            # the last query: a kept key (far behind the window), the first key inside the window, and two keys that it must
            # not see (the first one behind the kept keys, the last one in front of the window) with the largest score of all
            q[-1] *= 0; q[-1, :, 0] = 6.0
            for j, val in ((keep - 1, 6.0), (p_last - window + 1, 6.0), (keep, 9.0), (p_last - window, 9.0)):
                k[j] *= 0; k[j, :, 0] = val
        need = -(-n // ps)
        gen = torch.Generator().manual_seed(100 + b)
        mine = (torch.randperm(num_pages // B, generator=gen)[:need] * B + b).tolist()
        for i in range(n):
            kps[mine[i // ps], :, i % ps] = k[i]
            vps[mine[i // ps], :, i % ps] = v[i]
        rows.append(mine)
        pq = list(range(ctx_lens[b], n))
        want.append(_masked_attention_rows(q.double(), k.double(), v.double(), pq, scale, window, keep, 0.0, gate.double()))
        qs.append(q); gates.append(gate)
        pos_all += pq
        slot_all += [b] * step_lens[b]
    q_all = torch.cat(qs).reshape(-1, nq * d).cuda()
    gate_all = torch.cat(gates).cuda()
    T = q_all.shape[0]
    out = torch.zeros(T, nq * d, dtype=adt, device="cuda")
    table = table_tensor(rows, max_pages, num_pages)
    kd, vd = kps.cuda(), vps.cuda()
    q_start = [0]
    for n in step_lens:
        q_start.append(q_start[-1] + n)
    if kernel.startswith("exact"):
        ops.attn_tokenwise(q_all, nq * d, out, kd, vd, table, ps, i32(pos_all), i32(slot_all), nq, nkv, d, window, scale,
                           sink=sink.cuda(), keep_first=keep, gate=gate_all)
    elif kernel == "tensor_core_bf16":
        args = (q_all, nq * d, out, kd, vd, table, ps, i32(q_start), i32(ctx_lens), i32(list(range(B))))
        if all(n == 1 for n in step_lens):
            span = max(c + 1 for c in ctx_lens)
            span = min(span, window + 63 + ops_attention.kept_span(keep))
            for splits_wanted in (1, 3, 64):            # one range, a few, and more ranges than tiles
                tiles = -(-span // 64)
                splits = min(splits_wanted, tiles)
                chunk = -(-tiles // splits) * 64
                splits = -(-tiles * 64 // chunk)
                po = torch.full((B, nq, splits, d), float("nan"), device="cuda")
                pml = torch.full((B, nq, splits, 2), float("nan"), device="cuda")
                out.zero_()
                ops_attention.decode(*args, B, nq, nkv, d, window, scale, chunk, splits, po, pml, sink=sink.cuda(), keep_first=keep)
                ops.head_gate(out, gate_all, nq, d)
                assert_close(out.view(T, nq, d), torch.cat(want), f"decode, {splits} ranges", **BF16)
            out.zero_()
        ops_attention.prefill(*args, q_start, nq, nkv, d, window, scale, sink=sink.cuda(), keep_first=keep)
        ops.head_gate(out, gate_all, nq, d)
    elif kernel == "tcgen05_bf16":                      # the one-tile kernel walks the kept tiles, then the window's
        ops_attention.prefill_tc(q_all, nq * d, out, kd, vd, table, ps, i32(q_start), i32(ctx_lens), i32(list(range(B))), q_start,
                                 nq, nkv, d, window, scale, sink=sink.cuda(), keep_first=keep)
        ops.head_gate(out, gate_all, nq, d)
    else:                                               # the step's own choice of kernels
        qkv = torch.zeros(T, (nq + 2 * nkv) * d, dtype=adt, device="cuda")
        qkv[:, :nq * d] = q_all
        ctx = SimpleNamespace(B=B, T=T, decode_only=all(n == 1 for n in step_lens), page_size=ps, q_start=i32(q_start), start_pos=i32(ctx_lens),
                              slots=i32(list(range(B))), h_q_start=q_start, h_start_pos=list(ctx_lens), h_slots=list(range(B)),
                              graph_max_ctx=0, max_ctx=max(c + n for c, n in zip(ctx_lens, step_lens)), scratch={})
        ops_attention.attend_bf16(qkv, out, ctx, kd, vd, table, nq, nkv, d, window, scale, sink=sink.cuda(), keep_first=keep)
        ops.head_gate(out, gate_all, nq, d)
    ops_gemm.check_status()
    assert_close(out.view(T, nq, d), torch.cat(want), kernel, **tol(adt))
    # the oracle itself tells a window, a number of kept keys or a denominator that is off by one
    n0 = ctx_lens[0] + step_lens[0]
    if n0 > window + keep + 2 and keep > 0:
        k0 = torch.stack([kps[rows[0][i // ps], :, i % ps] for i in range(n0)]).double()
        v0 = torch.stack([vps[rows[0][i // ps], :, i % ps] for i in range(n0)]).double()
        last = qs[0][-1:].double()
        right = _masked_attention_rows(last, k0, v0, [n0 - 1], scale, window, keep, 0.0, None)
        for w2, k2, s2 in ((window + 1, keep, 0.0), (window, keep + 1, 0.0), (window - 1, keep, 0.0) if window > 1 else (window, keep - 1, 0.0)):
            other = _masked_attention_rows(last, k0, v0, [n0 - 1], scale, w2, k2, s2, None)
            assert float((other - right).abs().max()) > 1e-3, f"window {w2}, kept {k2}, sink {s2} must show"


def _conv_plain(x, w, bias, lens):
    out, t0 = torch.zeros_like(x), 0
    for n in lens:
        out[t0:t0 + n] = plain_model.short_convolution(x[t0:t0 + n], w, bias)
        t0 += n
    return out


def _run_in_cuts(lens, cuts, slots, step):
    """Calls step(rows, q_start, live slots) for every launch of a schedule: cut[b] tokens of request b (0: left out)."""
    B = len(lens)
    starts = [sum(lens[:b]) for b in range(B)]
    done = [0] * B
    for cut in cuts:
        rows, q_start, live = [], [0], []
        for b in range(B):
            n = min(cut[b], lens[b] - done[b])
            if n > 0:
                rows += list(range(starts[b] + done[b], starts[b] + done[b] + n)); done[b] += n
                q_start.append(len(rows)); live.append(slots[b])
        if rows:
            step(rows, q_start, live)
    assert done == list(lens)


CUTS = [[1000] * 4, [1, 5, 2, 3], [2, 2, 2, 2], [16, 1, 0, 7], [3, 16, 16, 16], [1, 1, 1, 1], [40, 40, 40, 40], [1000] * 4]
LENS = [1, 37, 90, 64]


@pytest.mark.parametrize("W,taps", [(40, 4), (96, 3), (24, 1), (64, 2), (39, 5), (300, 4)])
def test_convolution_in_one_step_and_in_portions(W, taps):
    """The causal convolution with its bias over four requests in one launch, and in portions of all sizes (single tokens,
    portions shorter than the taps, requests left out of a step) with the inputs carried in the state slots of requests
    that came in another order; the input sits behind other columns of a wider row and gets a bias of its own."""
    from tensorline_b200 import ops
    T, off = sum(LENS), 17
    proj = rnd(T, off + W + 5, seed=1, scale=1.5)
    in_bias, w, cb = rnd(off + W, seed=2), rnd(W, taps, seed=3, scale=0.8), rnd(W, seed=4)
    want = _conv_plain(proj[:, off:off + W].double() + in_bias[off:].double(), w.double(), cb.double(), LENS)
    slots = [5, 0, 3, 1]
    for cuts in ([[1000] * 4], CUTS[1:]):
        state = torch.zeros(7, max(taps - 1, 1) * W, device="cuda") if taps > 1 else None
        if state is not None:
            state[2] = 7.0; state[4] = -3.0; state[6] = 1.0          # other requests' slots
        got = torch.zeros(T, W)

        def step(rows, q_start, live):
            out = torch.empty(len(rows), W, device="cuda")
            ops.causal_conv(proj[rows].contiguous().cuda(), off, in_bias.cuda(), W, w.cuda(), cb.cuda(), state, i32(q_start), i32(live), out,
                            B=len(live), max_q_len=max(b - a for a, b in zip(q_start, q_start[1:])))
            got[rows] = out.cpu()
        _run_in_cuts(LENS, cuts, slots, step)
        assert_close(got, want, f"convolution, {len(cuts)} launches", **F32)
        if state is not None:
            assert float(state[2].min()) == 7.0 and float(state[4].max()) == -3.0 and float(state[6].min()) == 1.0
            for b, slot in enumerate(slots):                         # the slot holds the request's last taps - 1 inputs, zeros before its start
                t1 = sum(LENS[:b + 1])
                x = proj[t1 - LENS[b]:t1, off:off + W] + in_bias[off:]
                x = torch.cat([torch.zeros(taps - 1, W), x])[-(taps - 1):]
                assert_close(state[slot].view(taps - 1, W), x, "the inputs a request keeps", **F32)


def _scan_plain(gates, gb, u, ypre, yb, lam, nb, lens, sharp=8.0):
    T, W = u.shape
    bw = W // nb
    out, t0, last = torch.zeros(T, W, dtype=F64), 0, []
    soft = torch.log1p(torch.exp(lam))
    for n in lens:
        S = torch.zeros(W, dtype=F64)
        for t in range(t0, t0 + n):
            z = (gates[t] + gb).view(nb, 2, bw)
            r, i = plain_model.sig(z[:, 0]).reshape(W), plain_model.sig(z[:, 1]).reshape(W)
            a = torch.exp(-sharp * r * soft)
            S = a * S + torch.sqrt(1 - a * a) * i * u[t]
            out[t] = S * plain_model.gelu_tanh(ypre[t] + yb)
        last.append(S)
        t0 += n
    return out, last


@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("W,nb", [(40, 5), (96, 3), (24, 24), (64, 1), (39, 3), (520, 4)])
def test_recurrence_in_one_step_and_in_portions(adt, W, nb):
    """The gated linear recurrence over four requests in one launch and in portions, the state carried in the requests'
    slots; decays from one half to nearly one a token."""
    from tensorline_b200 import ops
    T = sum(LENS)
    gates, gb = rnd(T, 2 * W, seed=1, scale=2.0), rnd(2 * W, seed=2)
    u, proj, yb = rnd(T, W, seed=3), rnd(T, W + 9, seed=4), rnd(W + 9, seed=5)
    lam = torch.rand(W, generator=torch.Generator().manual_seed(6)) * 6.0 - 8.0
    lam[0] = 30.0                                                      # softplus beyond where exp overflows in float32: a = exp(-8 r 30) = 0
    want, last = _scan_plain(gates.double(), gb.double(), u.double(), proj[:, 9:].double(), yb[9:].double(), lam.double(), nb, LENS)
    slots = [5, 0, 3, 1]
    results = []
    for cuts in ([[1000] * 4], CUTS[1:], [[7, 5, 13, 9]] * 13):
        state = torch.zeros(7, W, device="cuda")
        state[2] = 7.0
        got = torch.zeros(T, W)

        def step(rows, q_start, live):
            out = torch.empty(len(rows), W, dtype=adt, device="cuda")
            ops.rglru_scan(gates[rows].contiguous().cuda(), gb.cuda(), u[rows].contiguous().cuda(), proj[rows].contiguous().cuda(), yb.cuda(),
                           lam.cuda(), state, i32(q_start), i32(live), out, B=len(live), blocks=nb, sharpness=8.0,
                           max_q_len=max(b - a for a, b in zip(q_start, q_start[1:])), y_off=9)
            got[rows] = out.float().cpu()
        _run_in_cuts(LENS, cuts, slots, step)
        assert_close(got, want, f"recurrence, {len(cuts)} launches", **tol(adt))
        for b, slot in enumerate(slots):
            assert_close(state[slot], last[b], "the state a request keeps", **F32)
        assert float(state[2].min()) == 7.0
        results.append((got, state.cpu()))
    assert torch.equal(results[1][1], results[2][1]), "the state after short steps does not depend on how the tokens were cut"


@pytest.mark.parametrize("W,nb,T", [(40, 5, 300), (39, 3, 257), (512, 2, 64), (96, 1, 1)])
def test_a_float_in_three_parts_and_the_gates_from_them(W, nb, T):
    """Three bfloat16 parts sum to the float within one part in 2^24 (values of every size, zeros, tiny ones), and the batched
    product of the parts with bfloat16 weights stacked three times is the float32 product."""
    from tensorline_b200 import ops
    bw = W // nb
    x = rnd(T, W, seed=21) * torch.exp(rnd(T, W, seed=22) * 6.0)
    x[0, :3] = torch.tensor([0.0, 1e-30, -3.0e38 / 1e4])
    parts = ops.split3(x.cuda(), nb)
    assert parts.shape == (nb, T, 3 * bw) and parts.dtype == torch.bfloat16
    back = parts.double().cpu().view(nb, T, 3, bw).sum(2).permute(1, 0, 2).reshape(T, W)
    assert float(((back - x.double()).abs() / x.double().abs().clamp_min(1e-30)).max()) <= 2.0 ** -23
    w = rnd(nb, bw, 2 * bw, seed=23).to(torch.bfloat16)
    got = torch.bmm(parts, w.cuda().repeat(1, 3, 1), out_dtype=torch.float32).cpu()
    want = torch.einsum("tbk,bkn->btn", x.double().view(T, nb, bw), w.double())
    scale = torch.einsum("tbk,bkn->btn", x.double().abs().view(T, nb, bw), w.double().abs())
    assert float(((got.double() - want).abs() / scale.clamp_min(1e-30)).max()) < 4e-6


@pytest.mark.parametrize("by_block", [False, True])
@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("W,nb", [(40, 5), (130, 2), (520, 4)])
def test_recurrence_of_long_steps_in_chunks(adt, W, nb, by_block):
    """Steps long enough to run as chunks side by side: requests that end one token before, at and one token after a chunk's
    edge, a single token and a request of many chunks in one launch, then the same requests in portions whose edges fall
    inside chunks, and continued token by token from the state the long step left."""
    from tensorline_b200 import ops
    C = ops.rglru_chunk()
    lens = [2 * C - 1, 2 * C, 2 * C + 1, 1, 9 * C + 5, C]
    T = sum(lens)
    gates, gb = rnd(T, 2 * W, seed=11, scale=2.0), rnd(2 * W, seed=12)
    u, proj, yb = rnd(T, W, seed=13), rnd(T, W, seed=14), rnd(W, seed=15)
    lam = torch.rand(W, generator=torch.Generator().manual_seed(16)) * 6.0 - 8.0
    want, last = _scan_plain(gates.double(), gb.double(), u.double(), proj.double(), yb.double(), lam.double(), nb, lens)
    slots = [4, 6, 0, 2, 1, 5]
    n = len(lens)
    tail = [[0, 0, 0, 0, 1, 0]] * 6
    for cuts in ([[10 ** 6] * n], [[2 * C + 1] * n, [3 * C - 2] * n, [10 ** 6] * n], [[5, 0, 0, 0, 9 * C - 1, 0], [10 ** 6] * n],
                 [[10 ** 6, 10 ** 6, 10 ** 6, 10 ** 6, 9 * C - 1, 10 ** 6]] + tail):
        state = torch.full((8, W), float("nan"), device="cuda")
        state[slots] = 0.0
        state[3] = 7.0
        got = torch.zeros(T, W)

        def step(rows, q_start, live):
            out = torch.empty(len(rows), W, dtype=adt, device="cuda")
            g = gates[rows].contiguous()
            if by_block:                                               # as a batched product per block leaves them
                g = g.view(len(rows), nb, 2 * (W // nb)).transpose(0, 1).contiguous()
            ops.rglru_scan(g.cuda(), gb.cuda(), u[rows].contiguous().cuda(), proj[rows].contiguous().cuda(), yb.cuda(),
                           lam.cuda(), state, i32(q_start), i32(live), out, B=len(live), blocks=nb, sharpness=8.0,
                           max_q_len=max(b - a for a, b in zip(q_start, q_start[1:])), by_block=by_block)
            got[rows] = out.float().cpu()
        _run_in_cuts(lens, cuts, slots, step)
        assert_close(got, want, f"recurrence in chunks, {len(cuts)} launches", **tol(adt))
        for b, slot in enumerate(slots):
            assert_close(state[slot], last[b], "the state a request keeps", **F32)
        assert float(state[3].min()) == 7.0 and bool(torch.isnan(state[7]).all())


@pytest.mark.parametrize("decoded", [0, 300])
def test_recurrence_keeps_a_far_token(decoded):
    """One channel with a decay of almost one is written once, at the first token, and read 700 tokens later (after a prompt,
    or after a prompt and 300 single tokens): losing, zeroing or mixing up the state shows as a wrong value there."""
    from tensorline_b200 import ops
    W, T = 32, 700
    gates = torch.zeros(T, 2 * W)
    gates[:, :W] = -9.0                                                # r small: the state hardly decays
    gates[:, W:] = -30.0                                               # i = 0: nothing is written ...
    gates[0, W:] = 30.0                                                # ... but at the first token
    u, proj = torch.ones(T, W) * 3.0, torch.ones(T, W) * 2.0
    gb, yb, lam = torch.zeros(2 * W), torch.zeros(W), torch.full((W,), -4.0)
    want, _ = _scan_plain(gates.double(), gb.double(), u.double(), proj.double(), yb.double(), lam.double(), 1, [T])
    assert float(want[-1, 0]) > 0.5 * float(want[0, 0]) > 0.01
    state = torch.zeros(3, W, device="cuda")
    got = torch.zeros(T, W)
    cuts = [T - decoded] + [1] * decoded
    t0 = 0
    for n in cuts:
        out = torch.empty(n, W, device="cuda")
        ops.rglru_scan(gates[t0:t0 + n].contiguous().cuda(), gb.cuda(), u[t0:t0 + n].contiguous().cuda(), proj[t0:t0 + n].contiguous().cuda(),
                       yb.cuda(), lam.cuda(), state, i32([0, n]), i32([1]), out, B=1, blocks=1, sharpness=8.0, max_q_len=n)
        got[t0:t0 + n] = out.cpu()
        t0 += n
    assert_close(got, want, "a far token through the state", **F32)


@pytest.mark.parametrize("E,top,groups,keep", [(8, 2, 4, 2), (6, 3, 2, 1), (9, 4, 3, 2), (4, 4, 1, 1), (4, 1, 4, 1), (10, 3, 5, 2), (64, 8, 8, 4),
                                               (256, 8, 8, 4), (3, 3, 1, 1), (14, 5, 2, 1)])
def test_choice_of_experts_among_groups(E, top, groups, keep):
    """Sigmoid scores with a correction of their own size (choice scores on both sides of zero), the best groups by the sum
    of their two largest, the largest choice scores inside them, weights from the scores without the correction."""
    from tensorline_b200 import ops
    T, scale = 50, 2.5
    z = rnd(T, E + 3, seed=1, scale=2.0)
    corr = rnd(E, seed=2, scale=0.8) - 0.5
    idx = torch.empty(T, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(T, top, dtype=torch.float32, device="cuda")
    ops.route_groups(z.cuda()[:, :E], corr.cuda(), top, groups, keep, 2, scale, idx, wts)
    r = {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}, "scale": scale}
    outside = 0
    for t in range(T):
        chosen, weights = plain_model.choose_experts(z[t, :E].double(), corr.double(), r)
        assert idx[t].tolist() == chosen, f"token {t}"
        assert_close(wts[t], torch.tensor(weights), "weights", **F32)
        c = plain_model.sig(z[t, :E].double()) + corr.double()
        outside += sorted(range(E), key=lambda e: (-float(c[e]), e))[:top] != chosen
    if keep < groups and top < E and E // groups > 1:       # (a group of one expert is judged by that expert alone)
        assert outside > 0, "the groups must keep some token from the experts it would choose without them"
    ops.route_groups(z.cuda()[:, :E], None, top, groups, keep, 2, 1.0, idx, wts)
    assert_close(wts.sum(1), torch.ones(T), "weights without a scale add up to one", **F32)


# ------------------------------------------------------------------------------------------ whole models
@pytest.fixture(scope="module", params=["S1", "S2"])
def model(request, tmp_path_factory):
    name = request.param
    folder = write_tiny_sumuvik(name, tmp_path_factory.mktemp(f"tiny_{name}"))
    plain = PlainSumuvik(folder)
    V = CONFIGS[name]["vocab"]
    reqs = {f"r{i}": random_tokens(V, n, seed=100 + i) for i, n in enumerate(LENGTHS[name])}
    want = {rid: forward(plain, toks) for rid, toks in reqs.items()}
    return dict(name=name, folder=folder, reqs=reqs, want=want, page=PAGE_SIZE[name], vocab=V, plain=plain)


def check(model, dtype, got, what):
    """32-bit: every position within F32_ATOL (times the largest |logit| where that is above one).  bfloat16: the largest logit
    error of a position as a share of the request's largest |logit|: four positions in five within BF16_REL, every one within
    that largest |logit| (a sigmoid score near a tie picks another expert in bfloat16; the 32-bit runs pin those positions)."""
    assert got, "nothing was compared"
    over = 0
    for (rid, p), row in got.items():
        ref = model["want"][rid][p]
        err = float((row - ref).abs().max())
        if dtype == "float32":
            bound = F32_ATOL * max(1.0, float(ref.abs().max()))
            assert err <= bound, f"{what}: request {rid} position {p}: max abs err {err:.3e} > {bound:.3e}"
        else:
            top = float(model["want"][rid].abs().max())
            assert err <= top, f"{what}: request {rid} position {p}: max abs err {err:.3e} > {top:.3e}"
            over += err > BF16_REL * top
    assert over <= 0.2 * len(got), f"{what}: {over} of {len(got)} positions are beyond the bfloat16 bound"


def test_the_model_is_chosen_by_its_configuration_and_every_layer_matches(model):
    """Residual stream after every layer, 32-bit engine against the plain model."""
    from tensorline_b200.parts.linear import PairSum, resolve
    from tensorline_b200.replay import TraceSession, make_runner
    runner, cfg = make_runner(model["folder"], "float32", 256, page_size=model["page"], max_live=2)
    assert type(cfg).__name__ == "SumuvikConfig" and cfg.to_json_dict() == CONFIGS[model["name"]]
    seen = []
    for blk in runner.model.blocks:
        def fwd(x, pending, ctx, cache, orig=blk.forward):
            out = orig(x, pending, ctx, cache)
            add = out.a.double() + out.b.double() if isinstance(out, PairSum) else resolve(out).double()
            seen.append((x.double() + add).cpu())
            return out
        blk.forward = fwd
    toks = model["reqs"]["r2"]
    TraceSession(runner).run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": ["a"]})
    want = []
    forward(model["plain"], toks, want)
    assert len(seen) == len(want) == len(CONFIGS[model["name"]]["layers"])
    for i, (g, w) in enumerate(zip(seen, want)):
        assert_close(g, w, f"residual stream after layer {i}", rtol=5e-5, atol=5e-5)


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
    """The bfloat16 engine's forms for long steps (the gates from three parts of a float through a batched product, the
    recurrence in chunks side by side) taken from two tokens on: whole prompts, changing portions and mixed batches."""
    from tensorline_b200.parts import rglru
    monkeypatch.setattr(rglru, "GATE_PRODUCT_LIBRARY_MIN_TOKENS", 2)
    for what, steps, most in (("whole", steps_alone(model, cuts_whole), 192), ("changing portions", steps_alone(model, cuts_changing), 192),
                              ("mixed", *steps_mixed(model, 3))):
        got = replay(model, "bfloat16", steps, max_tokens=most)
        check(model, "bfloat16", got, f"long forms, {what}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(model, dtype):
    """A one-token prompt, then 150 tokens decoded one by one: states and windows are carried through 150 launches, every
    window passes over decoded tokens and over page borders, and the kept first tokens fall far behind it."""
    toks = random_tokens(model["vocab"], 151, seed=7)
    want = forward(model["plain"], toks)
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    steps[-1]["end"] = ["x"]
    m2 = dict(model, reqs={"x": toks}, want={"x": want})
    got = replay(m2, dtype, steps, max_tokens=160)
    check(m2, dtype, got, "token by token")
    assert sorted(p for _, p in got) == list(range(151))


def _other_masks(raw, window_by=0, keep_by=0):
    raw = copy.deepcopy(raw)
    for layer in raw["layers"]:
        if "mask" in layer["mixer"]:
            layer["mixer"]["mask"]["size"] += window_by
            if layer["mixer"]["mask"]["keep_first"] > 0 or keep_by > 0:
                layer["mixer"]["mask"]["keep_first"] += keep_by
    return raw


def test_edges_of_windows_and_of_the_kept_tokens_in_prompts_and_in_decoding(model):
    """The plain model with every window, or every number of kept tokens, one off gives other logits from the first position
    on that a mask cuts, and so does the plain model without the one in the denominators: a key that is wrongly seen (or not
    seen) and a lost term show.  The engine follows the right one: whole, with the tokens around every edge decoded one by one,
    and in portions that end on both sides of the edges."""
    toks = random_tokens(model["vocab"], 90, seed=11)
    right = forward(model["plain"], toks)
    masks = [l["mixer"]["mask"] for l in CONFIGS[model["name"]]["layers"] if "mask" in l["mixer"]]
    windows = sorted({m["size"] for m in masks})
    first = windows[0]                                      # the first position whose smallest window leaves a key out
    for kw in (dict(window_by=-1), dict(window_by=1), dict(keep_by=-1), dict(keep_by=1)):
        other = PlainSumuvik(model["folder"])
        other.cfg = _other_masks(other.cfg, **kw)
        gap = (forward(other, toks) - right).abs().max(1).values
        assert float(gap[:first - 1].max()) == 0.0
        assert float(gap.max()) > 100 * F32_ATOL, f"the plain model must tell masks that are one token off ({kw})"
    other = PlainSumuvik(model["folder"])
    other.one_in_denominator = False
    assert float((forward(other, toks) - right).abs().max(1).values.median()) > 100 * F32_ATOL, "the one in the denominator must show"
    m2 = dict(model, reqs={"w": toks}, want={"w": right})
    edges = sorted({e + k for m in masks for e in (m["size"], m["keep_first"], m["size"] + m["keep_first"]) for k in (-1, 0, 1)
                    if 0 < e + k < 90})
    cuts = [[90], [first - 1] + [1] * (91 - first), [e2 - e1 for e1, e2 in zip([0] + edges, edges + [90]) if e2 > e1]]
    for dtype in ("float32", "bfloat16"):
        for c in cuts:
            assert sum(c) == 90
            got = replay(m2, dtype, steps_alone(m2, lambda n, c=c: c), max_tokens=96)
            check(m2, dtype, got, f"mask edges, portions {c[:4]}...")


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


@pytest.mark.parametrize("name", ["S3", "S4", "S5", "S6"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_further_shapes_of_the_design(name, dtype, tmp_path):
    """Attention only (a layer without a mask, more kept tokens than the window, groups of one expert; prefixes could be
    shared); the recurrence only (no page group at all, every expert chosen); sizes that are multiples of nothing much and a
    window of the token itself; sizes that the tensor-core kernels take, with prompts of hundreds of tokens (the tcgen05 prompt
    kernel over kept first keys, the recurrence in chunks, the gates from three parts of a float): whole requests, changing
    portions and a small pool against the plain model."""
    folder = write_tiny_sumuvik(name, tmp_path / name)
    plain = PlainSumuvik(folder)
    V = CONFIGS[name]["vocab"]
    lengths = [290, 3, 400, 130] if name == "S6" else [3, 50, 1, 81, 33]
    reqs = {f"r{i}": random_tokens(V, n, seed=300 + i) for i, n in enumerate(lengths)}
    m = dict(name=name, folder=folder, reqs=reqs, want={r: forward(plain, t) for r, t in reqs.items()}, page=PAGE_SIZE[name], vocab=V)
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
