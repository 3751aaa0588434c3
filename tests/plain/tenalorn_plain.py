"""A plain, slow implementation of the Tenalorn decoder, used only as the oracle of the tests.

Whole sequences, no cache, no batching, one function per mechanism, float64 on the CPU, written from the design's
equations in the notation below; it shares no code with the package under test.

Notation.  Tokens t = 0, 1, ... of one sequence; W: matrices stored [out, in], applied as W h; sig = the logistic function;
n(v; w) = v / sqrt(mean(v^2) + eps) * w and u(v) = v / sqrt(mean(v^2) + eps) with the model's eps.

  start      e_t = embed[tok_t] * embedding.scale + bigram[r_t];  r_t = (tok_(t-1) * mul_prev + tok_t * mul_cur) mod buckets,
             r_0 = buckets (the table's last row);  streams X_1 .. X_S all start as e
  sublayer   (q = 1: mixer, q = 2: feed-forward)  z = sum_s in_q[s] X_s;  y = sublayer(n(z; norm_q));
             X_t' = sum_s mix_q[s, t] X_s + out_q[t] y   for every t from the old streams
  parallel   left_scale * left(h) + right_scale * right(h)
  left       q = Wq h, k = Wk h, v = Wv h; query head a reads KV head a // (heads / kv_heads); every head of q and k through u;
             s_tj = scale q_t . k_j - slope_a (t - j), slope_a = 2^(-8 (a + 1) / heads); j is seen from t if j <= t and
             t // size = j // size; softmax over the seen keys; y = Wo (heads side by side)
  right      q = Wq h / sqrt(dim), k = Wk h, v = Wv h per head; i = cap tanh((Wi h + bi) / cap),
             f = logsig(cap tanh((Wf h + bf) / cap));  m_t = max(f + m_(t-1), i), m before the start = 0;
             S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T, N_t the same with k alone, both 0 before the start;
             o = S_t^T q / (max(|N_t . q|, exp(-m_t)) + 1e-6);  y = Wo (u(o) per head, side by side, * norm * sig(Wg h))
  latent     q = Wq h, per head [dim plain | rot_dim turned];  Wdkv h = [kv_rank | rot_dim]: c = n(first; dkv.norm), r = the rest,
             turned, one for all heads;  k_a = Wuk_a c, v_a = Wuv_a c;  s_tj = scale (q_plain . k_a(j) + q_turned . r(j)), every
             j <= t, softmax;  y = Wo ((heads side by side) * sig(Wg h))
  turning    pairs (2i, 2i + 1), i < dims / 2, angle t * base^(-2i / dims):  (u, v) -> (u cos - v sin, v cos + u sin)
  experts    p = softmax(Wrouter h) over experts + identity entries; c = p + correction; the `top` largest c are chosen;
             weights p_e / (sum of the chosen p + 1e-20); an entry e >= experts gives h itself; an expert gives
             Wdown (silu(Wgate h) * Wup h);  y = sum_e weight_e out_e + shared unit(h)
             without `streams` in the configuration there is one stream and X' = X + y
  output     logits = cap tanh(Whead n(sum_s X_s; final.norm) / cap), cap = logit_softcap
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


def unit(v, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def sig(z):
    return 1.0 / (1.0 + torch.exp(-z))


def log_sig(z):
    return -torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, max=0.0)


def silu(z):
    return z * sig(z)


def bigram_rows(tokens, c):
    rows, prev = [], None
    for t in tokens:
        rows.append(c["buckets"] if prev is None else (prev * c["mul_prev"] + t * c["mul_cur"]) % c["buckets"])
        prev = t
    return rows


def embed(tokens, w, c):
    e = w["embed"][tokens] * c["scale"]
    if c.get("bigram") is not None:
        e = e + w["bigram"][bigram_rows(tokens, c["bigram"])]
    return e


def turn_pairs(x, rot, dims):
    """x [T, ..., d]: dimensions (2i, 2i + 1) below `dims` turned by the token's position."""
    x = x.clone()
    T = x.shape[0]
    where = torch.arange(T, dtype=F64).view(T, *([1] * (x.dim() - 2)))
    for i in range(dims // 2):
        a = where * float(rot["base"]) ** (-2.0 * i / dims)
        p, q = x[..., 2 * i].clone(), x[..., 2 * i + 1].clone()
        x[..., 2 * i] = p * torch.cos(a) - q * torch.sin(a)
        x[..., 2 * i + 1] = q * torch.cos(a) + p * torch.sin(a)
    return x


def chunk_attention(h, w, c, eps):
    T = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = unit((h @ w["q"].T).view(T, H, d), eps)
    k = unit((h @ w["k"].T).view(T, G, d), eps)
    v = (h @ w["v"].T).view(T, G, dv)
    size = c["mask"]["size"] if c.get("mask") else None
    o = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        kv = a // (H // G)
        slope = 2.0 ** (-8.0 * (a + 1) / H)
        for t in range(T):
            js = [j for j in range(t + 1) if size is None or j // size == t // size]
            s = (k[js, kv] @ q[t, a]) * c["scale"] - slope * torch.tensor([float(t - j) for j in js], dtype=F64)
            o[t, a] = torch.softmax(s, 0) @ v[js, kv]
    return o.reshape(T, H * dv) @ w["o"].T


def matrix_memory(h, w, c, eps):
    T = h.shape[0]
    H, d, dv, cap = c["heads"], c["dim"], c["vdim"], float(c["gate_cap"])
    q = (h @ w["q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w["k"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, dv)
    gi = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    gf = log_sig(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    o = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        S, N, m = torch.zeros(d, dv, dtype=F64), torch.zeros(d, dtype=F64), 0.0
        for t in range(T):
            m_new = max(float(gf[t, a]) + m, float(gi[t, a]))
            keep, take = math.exp(float(gf[t, a]) + m - m_new), math.exp(float(gi[t, a]) - m_new)
            S = keep * S + take * torch.outer(k[t, a], v[t, a])
            N = keep * N + take * k[t, a]
            m = m_new
            o[t, a] = (S.T @ q[t, a]) / (max(abs(float(N @ q[t, a])), math.exp(-m)) + 1e-6)
    y = unit(o, eps).reshape(T, H * dv) * w["norm"] * sig(h @ w["g"].T)
    return y @ w["o"].T


def parallel(h, w, c, eps):
    left = chunk_attention(h, {k[5:]: v for k, v in w.items() if k.startswith("left.")}, c["left"], eps)
    right = matrix_memory(h, {k[6:]: v for k, v in w.items() if k.startswith("right.")}, c["right"], eps)
    return c["left_scale"] * left + c["right_scale"] * right


def latent_attention(h, w, c, eps):
    T = h.shape[0]
    H, d, dr, dv, rank = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"]
    q = (h @ w["q"].T).view(T, H, d + dr)
    down = h @ w["dkv"].T
    lat = normed(down[:, :rank], w["dkv.norm"], eps)
    r = down[:, rank:]
    if dr:
        q = torch.cat([q[..., :d], turn_pairs(q[..., d:], c["rot"], c["rot"]["dims"])], dim=-1)
        r = turn_pairs(r, c["rot"], c["rot"]["dims"])
    k = (lat @ w["uk"].T).view(T, H, d)
    v = (lat @ w["uv"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        s = (q[:, a, :d] @ k[:, a].T + q[:, a, d:] @ r.T) * c["scale"]
        s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), float("-inf"))
        o[:, a] = torch.softmax(s, -1) @ v[:, a]
    return (o.reshape(T, H * dv) * sig(h @ w["g"].T)) @ w["o"].T


def gated_unit(h, w):
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def route(h, w, c):
    """[(entry, weight)] of every token."""
    p = torch.softmax(h @ w["router"].T, -1)
    choice = p + w["correction"]
    out = []
    for t in range(h.shape[0]):
        chosen = torch.topk(choice[t], c["router"]["top"]).indices.tolist()
        total = sum(float(p[t, e]) for e in chosen) + 1e-20
        out.append([(e, float(p[t, e]) / total) for e in chosen])
    return out


def experts(h, w, c):
    E = c["router"]["experts"]
    y = torch.zeros_like(h)
    for t, chosen in enumerate(route(h, w, c)):
        for e, weight in chosen:
            if e >= E:
                y[t] += weight * h[t]
            else:
                y[t] += weight * gated_unit(h[t], {k: w[f"e{e}.{k}"] for k in ("gate", "up", "down")})
    if c.get("shared") is not None:
        y = y + gated_unit(h, {k: w[f"shared.{k}"] for k in ("gate", "up", "down")})
    return y


def sub(w, prefix):
    return {k[len(prefix) + 1:]: v for k, v in w.items() if k.startswith(prefix + ".")}


def streams_step(X, hc, norm_w, eps, fn):
    """One sublayer over the streams X [S, T, W]; without hyper-connection tensors (`hc` empty) the one stream takes the sum."""
    if not hc:
        return X + fn(normed(X[0], norm_w, eps))[None]
    z = torch.einsum("s,stw->tw", hc["in"], X)
    y = fn(normed(z, norm_w, eps))
    return torch.einsum("sr,stw->rtw", hc["mix"], X) + hc["out"][:, None, None] * y[None]


def forward(config: dict, weights: dict, tokens, per_layer: bool = False):
    """Logits [T, vocab] of one whole sequence (and the sum of the streams after every layer)."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    e = embed(list(tokens), w, config["embedding"])
    S = int(config.get("streams", 1))
    X = e[None].repeat(S, 1, 1)
    sums = []
    for i, layer in enumerate(config["layers"]):
        lw = sub(w, f"l{i}")
        mix = {"parallel": parallel, "latent_attention": latent_attention}[layer["type"]]
        X = streams_step(X, sub(lw, "hc1"), lw["norm1"], eps, lambda h: mix(h, sub(lw, "mix"), layer["mixer"], eps))
        if layer["mlp"] is not None:
            X = streams_step(X, sub(lw, "hc2"), lw["norm2"], eps, lambda h: experts(h, sub(lw, "mlp"), layer["mlp"]))
        sums.append(X.sum(0))
    logits = normed(X.sum(0), w["final.norm"], eps) @ w["head"].T
    if config.get("logit_softcap") is not None:
        cap = float(config["logit_softcap"])
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(sums)) if per_layer else logits


def load(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


class PlainTenalorn:
    def __init__(self, folder):
        self.cfg, self.weights = load(folder)


def logits_of(model: PlainTenalorn, tokens, layers: list | None = None):
    """Logits [T, vocab]; `layers`, if given, receives the sum of the streams after every layer."""
    out, sums = forward(model.cfg, model.weights, tokens, per_layer=True)
    if layers is not None:
        layers.extend(sums)
    return out


def greedy_generate(model: PlainTenalorn, prompt, n: int) -> list:
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(torch.argmax(logits_of(model, seq)[-1]))
        out.append(tok)
        seq.append(tok)
    return out
