"""A plain, slow implementation of the Sumuvik decoder, used only as the oracle of the tests.

Whole sequences, no cache, no batching, one function per mechanism, float64 on the CPU, written from the design's
equations in the notation below; it shares no code with the package under test.

Notation.  x_t: residual stream at token t (positions from 0); W: matrices stored [out, in], applied as W h;
n(v; w) = v / sqrt(mean(v^2) + eps) * w with the model's eps; sig = the logistic function.

  start      x = embed[token] * embedding.scale
  layer      x <- x + (mixer(n(x; norm1)) + ff(n(x; norm2)))        both read the same x; a layer may have no ff
  attention  q = Wq h + bq, k = Wk h + bk, v = Wv h + bv; query head a reads KV head a // (heads / kv_heads);
             q and k turned by position over their first rot.dims dimensions, pairs (2i, 2i + 1);
             key j is seen from t if j <= t and (t - j < mask.size or j < mask.keep_first); no mask: every j <= t;
             p_tj = exp(s_tj) / (1 + sum_j exp(s_tj)), s_tj = scale q_t . k_j;  o_t = sum_j p_tj v_j;
             head a of o_t times sig(Wg h_t)_a;  y = Wo o
  turning    angle t * f_i, f_i = base^(-2i / dims), stretched where rot.scaling says: wavelength l = 2 pi / f;
             l < original / high: f; l > original / low: f / factor; else with s = (original / l - low) / (high - low):
             (1 - s) f / factor + s f;   (u, v) -> (u cos - v sin, v cos + u sin)
  rglru      y = gelu_tanh(Wy h + by);  u = conv(Wx h + bx): per channel, taps weights, the last on the current token,
             zeros before the start, plus conv.b;  u in `blocks` equal parts, r = sig(Ra_b u_b + ra.b_b), i = sig(Ri_b u_b + ri.b_b);
             a = exp(-8 r softplus(lam));  S <- a S + sqrt(1 - a^2) i u, S = 0 before the first token;  out = Wo (S y)
  unit       g = min(Wgate h, limit), u = clamp(Wup h, -limit, limit);  Wdown (g sig(1.702 g) (u + 1))
  experts    s = sig(Wrouter h), c = s + correction; groups.count equal groups of neighbours, a group's score is the sum of
             its two largest c; experts outside the groups.keep best groups cannot be chosen; the `top` largest c are;
             weights s_e / (sum of the chosen s + 1e-20) * router.scale;  y = sum_e weight_e unit_e(h) + shared unit(h)
  output     logits = Whead n(x; final.norm)
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

from tests.plain.qwen2_plain import read_safetensors

F64 = torch.float64


def normed(v, w, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * w


def sig(z):
    return 1.0 / (1.0 + torch.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def frequencies(rot):
    """f_i of the pairs, with the long wavelengths stretched."""
    dims = rot["dims"]
    out = []
    for i in range(dims // 2):
        f = float(rot["base"]) ** (-2.0 * i / dims)
        sc = rot.get("scaling")
        if sc:
            l = 2.0 * math.pi / f
            if l > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif l >= sc["original"] / sc["high"]:
                s = (sc["original"] / l - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return out


def turn_pairs(x, rot, pos=None):
    """x [T, heads, d]: dimensions (2i, 2i + 1) below rot.dims turned by the token's position."""
    x = x.clone()
    T = x.shape[0]
    where = torch.tensor([float(t if pos is None else pos[t]) for t in range(T)], dtype=F64)
    for i, f in enumerate(frequencies(rot)):
        a = (where * f)[:, None]
        u, v = x[:, :, 2 * i].clone(), x[:, :, 2 * i + 1].clone()
        x[:, :, 2 * i] = u * torch.cos(a) - v * torch.sin(a)
        x[:, :, 2 * i + 1] = v * torch.cos(a) + u * torch.sin(a)
    return x


def sees(t, j, mask):
    if j > t:
        return False
    return mask is None or t - j < mask["size"] or j < mask.get("keep_first", 0)


def softmax_with_one(scores):
    """exp(s_j) / (1 + sum exp(s_j)) without overflow."""
    m = max(float(scores.max()), 0.0)
    e = torch.exp(scores - m)
    return e / (math.exp(-m) + e.sum())


def attention(h, w, c, one_in_denominator=True):
    T = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = (h @ w["q"].T + w["q.b"]).view(T, H, d)
    k = (h @ w["k"].T + w["k.b"]).view(T, G, d)
    v = (h @ w["v"].T + w["v.b"]).view(T, G, dv)
    q, k = turn_pairs(q, c["rot"]), turn_pairs(k, c["rot"])
    gate = sig(h @ w["g"].T)
    o = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        kv = a // (H // G)
        for t in range(T):
            js = [j for j in range(t + 1) if sees(t, j, c.get("mask"))]
            s = (k[js, kv] @ q[t, a]) * c["scale"]
            p = softmax_with_one(s) if one_in_denominator else torch.softmax(s, 0)
            o[t, a] = (p @ v[js, kv]) * gate[t, a]
    return o.reshape(T, H * dv) @ w["o"].T


def short_convolution(x, taps_w, bias):
    """x [T, C], taps_w [C, taps]: out_t = bias + sum_k taps_w[:, k] x_(t - (taps - 1) + k), zeros before the start."""
    T, taps = x.shape[0], taps_w.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        acc = bias.clone()
        for k in range(taps):
            j = t - (taps - 1) + k
            if j >= 0:
                acc = acc + taps_w[:, k] * x[j]
        out[t] = acc
    return out


def rglru(h, w, c, state_out=None):
    T, width, nb = h.shape[0], c["width"], c["blocks"]
    y = gelu_tanh(h @ w["y"].T + w["y.b"])
    u = short_convolution(h @ w["x"].T + w["x.b"], w["conv"], w["conv.b"])
    bw = width // nb
    S = torch.zeros(width, dtype=F64)
    out = torch.zeros(T, width, dtype=F64)
    soft = torch.log1p(torch.exp(w["lam"]))
    for t in range(T):
        r, i = torch.zeros(width, dtype=F64), torch.zeros(width, dtype=F64)
        for b in range(nb):
            part = u[t, b * bw:(b + 1) * bw]
            r[b * bw:(b + 1) * bw] = sig(w["ra"][b] @ part + w["ra.b"][b])
            i[b * bw:(b + 1) * bw] = sig(w["ri"][b] @ part + w["ri.b"][b])
        a = torch.exp(-8.0 * r * soft)
        S = a * S + torch.sqrt(1.0 - a * a) * i * u[t]
        out[t] = S * y[t]
    if state_out is not None:
        state_out.append(S)
    return out @ w["o"].T


def clamped_unit(h, w, limit):
    g = torch.clamp(h @ w["gate"].T, max=limit)
    u = torch.clamp(h @ w["up"].T, -limit, limit)
    return (g * sig(1.702 * g) * (u + 1.0)) @ w["down"].T


def choose_experts(z, correction, r):
    """z [E] router logits of one token -> (chosen experts in the order chosen, their weights)."""
    E, top = r["experts"], r["top"]
    count, keep = r["groups"]["count"], r["groups"]["keep"]
    s = sig(z)
    c = s + correction
    per = E // count
    scores = []
    for g in range(count):
        members = sorted((float(c[e]) for e in range(g * per, (g + 1) * per)), reverse=True)
        scores.append(sum(members[:2]))
    kept = sorted(range(count), key=lambda g: (-scores[g], g))[:keep]
    allowed = [e for e in range(E) if e // per in kept]
    chosen = sorted(allowed, key=lambda e: (-float(c[e]), e))[:top]
    total = sum(float(s[e]) for e in chosen) + 1e-20
    return chosen, [float(s[e]) / total * r["scale"] for e in chosen]


def experts(h, w, c, sub):
    out = torch.zeros_like(h)
    z = h @ w["router"].T
    for t in range(h.shape[0]):
        chosen, weights = choose_experts(z[t], w["correction"], c["router"])
        for e, we in zip(chosen, weights):
            out[t] += we * clamped_unit(h[t:t + 1], sub(f"e{e}"), c["expert"]["limit"])[0]
    if c.get("shared"):
        out = out + clamped_unit(h, sub("shared"), c["shared"]["limit"])
    return out


class PlainSumuvik:
    def __init__(self, folder):
        folder = Path(folder)
        self.cfg = json.loads((folder / "config.json").read_text())
        self.w = {k: v.to(F64) for k, v in read_safetensors(folder / "model.safetensors").items()}
        self.one_in_denominator = True                   # tests switch it off to see that the term shows

    def sub(self, prefix):
        n = len(prefix) + 1
        return {k[n:]: v for k, v in self.w.items() if k.startswith(prefix + ".")}


def forward(model: PlainSumuvik, tokens, layers_out=None):
    """Logits [T, vocab] float64 of a whole sequence; `layers_out` collects the stream after every layer."""
    cfg, w = model.cfg, model.w
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(list(tokens))] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        h = normed(x, w[f"l{i}.norm1"], eps)
        mix = model.sub(f"l{i}.mix")
        if layer["type"] == "attention":
            y = attention(h, mix, layer["mixer"], model.one_in_denominator)
        else:
            y = rglru(h, mix, layer["mixer"])
        if layer["mlp"] is not None:
            h2 = normed(x, w[f"l{i}.norm2"], eps)
            ff = model.sub(f"l{i}.mlp")
            if layer["mlp"]["kind"] == "dense":
                y = y + clamped_unit(h2, ff, layer["mlp"]["limit"])
            else:
                y = y + experts(h2, ff, layer["mlp"], lambda name, i=i: model.sub(f"l{i}.mlp.{name}"))
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return normed(x, w["final.norm"], eps) @ w["head"].T


def greedy_generate(model: PlainSumuvik, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(forward(model, toks)[-1].argmax()))
    return toks[len(prompt):]
