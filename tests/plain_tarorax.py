"""Plain, slow Tarorax: whole sequences, dense masks, explicit loops over
tokens, no cache, float64, one function for each mechanism.  It shares no code
with ``airframe_b200`` (its own reading of config.json and of the tensors).

Notation: h is a sublayer's input [T, width]; W x means a weight stored
[out, in] applied to a vector; positions count from 0; X is the list of residual
streams, each [T, width].
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

from plain_gemma2 import read_safetensors

F64 = torch.float64


def read_model_folder(folder, dtype=F64):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    return cfg, read_safetensors(folder / "model.safetensors", dtype)


# ---------------------------------------------------------------- small pieces

def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def zero_centred_norm(x, w, eps):
    """RMS norm whose stored weight lies around zero: the factor is 1 + w."""
    return rms(x, eps) * (1.0 + w)


# ---------------------------------------------------------------- residual streams

def streams_read(X, w_in):
    """u = sum_s in[s] X[s]."""
    return sum(w_in[s] * X[s] for s in range(len(X)))


def streams_write(X, y, mix, w_out):
    """All streams at once from the old ones: X'[t] = sum_s mix[s, t] X[s] + out[t] y."""
    n = len(X)
    return [sum(mix[s, t] * X[s] for s in range(n)) + w_out[t] * y for t in range(n)]


# ---------------------------------------------------------------- gated linear attention

def channel_decay(h, w1, w2, b2, tau):
    """alpha = sigmoid(W2 (W1 h) + b2)^(1 / tau), one factor per key channel."""
    z = (h @ w1.T) @ w2.T + b2
    return torch.exp(torch.log(sigmoid(z)) / tau)


def decayed_outer_product_scan(q, k, v, alpha):
    """One head.  q, k, alpha [T, dk], v [T, dv].  S_t = diag(alpha_t) S_(t-1) + k_t v_t^T from S = 0,
    o_t = S_t^T q_t.  Returns o [T, dv]."""
    T, dk = k.shape
    S = torch.zeros(dk, v.shape[1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = alpha[t][:, None] * S + k[t][:, None] * v[t][None, :]
        out.append(S.T @ q[t])
    return torch.stack(out)


def gla_mixer(h, W, p, m, eps):
    heads, dk, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    T = h.shape[0]
    q = (h @ W[p + "q"].T) * dk ** -0.5
    k = h @ W[p + "k"].T
    v = h @ W[p + "v"].T
    alpha = channel_decay(h, W[p + "a1"], W[p + "a2"], W[p + "a2.b"], tau)
    outs = []
    for i in range(heads):
        kk = slice(i * dk, (i + 1) * dk)
        o = decayed_outer_product_scan(q[:, kk], k[:, kk], v[:, i * dv:(i + 1) * dv], alpha[:, kk])
        outs.append(rms(o, eps) * W[p + "norm"])
    o = torch.cat(outs, dim=1) * silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# ---------------------------------------------------------------- differential attention

def short_convolution(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                y[t] += w[:, j] * u[src]
    return y


def query_temperature(T, coef, every):
    """1 + coef ln(floor((p + 1) / every) + 1) for p = 0 .. T - 1."""
    return torch.tensor([1.0 + coef * math.log((p + 1) // every + 1) for p in range(T)], dtype=F64)


def capped_causal_softmax(q, k, scale, cap):
    """q [T, d], k [T, d] -> weights [T, T] over the keys j <= i."""
    s = (q @ k.T) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    T = q.shape[0]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    return torch.softmax(s, dim=-1)


def difference_factor(W, p, diff):
    return (math.exp(float((W[p + "lq1"] * W[p + "lk1"]).sum())) - math.exp(float((W[p + "lq2"] * W[p + "lk2"]).sum()))
            + diff)


def diff_attention_mixer(h, W, p, m, eps):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    diff = float(m["diff"])
    T = h.shape[0]
    q = h @ W[p + "q"].T + W[p + "q.b"]
    k = h @ W[p + "k"].T + W[p + "k.b"]
    v = h @ W[p + "v"].T + W[p + "v.b"]
    if m.get("conv"):
        q, k, v = (short_convolution(u, W[p + n + ".conv"]) for u, n in ((q, "q"), (k, "k"), (v, "v")))
    if m.get("q_temp"):
        q = q * query_temperature(T, float(m["q_temp"]["coef"]), int(m["q_temp"]["every"]))[:, None]
    lam = difference_factor(W, p, diff)
    cap = float(m.get("softcap") or 0.0)
    outs = []
    for i in range(H):
        g = i // (H // G)
        vv = v[:, g * dv:(g + 1) * dv]
        a = []
        for mp in range(2):
            qq = q[:, (2 * i + mp) * d:(2 * i + mp + 1) * d]
            kk = k[:, (2 * g + mp) * d:(2 * g + mp + 1) * d]
            a.append(capped_causal_softmax(qq, kk, float(m["scale"]), cap) @ vv)
        outs.append(rms(a[0] - lam * a[1], eps) * (1.0 - diff))
    o = torch.cat(outs, dim=1) * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T + W[p + "o.b"]


# ---------------------------------------------------------------- feed-forwards

def dense_ff(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, W, p, r):
    """Per token: the chosen experts and their weights.  Returns (ids [T, top], weights [T, top], margin [T]):
    margin is the smallest gap that decided a choice (between groups or between experts)."""
    E, top = r["experts"], r["top"]
    s = sigmoid(h @ W[p + "router"].T)
    choice = s + W[p + "correction"]
    T = h.shape[0]
    margin = torch.full((T,), float("inf"), dtype=F64)
    groups = r.get("groups")
    if groups:
        cnt, keep = groups["count"], groups["keep"]
        per = E // cnt
        gs = choice.view(T, cnt, per).topk(min(2, per), dim=-1).values.sum(-1)
        order = gs.sort(dim=-1, descending=True, stable=True)
        if keep < cnt:
            margin = torch.minimum(margin, order.values[:, keep - 1] - order.values[:, keep])
        kept = torch.zeros(T, cnt, dtype=torch.bool)
        kept.scatter_(1, order.indices[:, :keep], True)
        choice = choice.masked_fill(~kept.repeat_interleave(per, dim=1), float("-inf"))
    order = choice.sort(dim=-1, descending=True, stable=True)
    ids = order.indices[:, :top]
    if top < E:
        gap = order.values[:, top - 1] - order.values[:, top]
        margin = torch.minimum(margin, torch.where(torch.isfinite(gap), gap, torch.full_like(gap, float("inf"))))
    w = s.gather(1, ids)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * float(r["scale"])
    return ids, w, margin


def moe_ff(h, W, p, mlp, margins=None):
    ids, w, margin = route(h, W, p, mlp["router"])
    if margins is not None:
        margins.append(margin)
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            out[t] += w[t, j] * (W[f"{p}e{e}.down"] @ gelu_erf(W[f"{p}e{e}.up"] @ h[t]))
    return out


# ---------------------------------------------------------------- the model

def forward(cfg, W, tokens, layers_out=None, round_h=None, margins=None):
    """Logits [T, vocab] of one sequence.  ``layers_out`` (a list) receives the sum of the streams after every
    layer, ``margins`` (a list) every router's margins [T].  ``round_h``: a function applied to every sublayer's
    input (to model a 16-bit product input)."""
    eps = float(cfg["norm"]["eps"])
    rh = round_h or (lambda z: z)
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)]
    has_streams = "streams" in cfg
    S = int(cfg.get("streams", 1))
    X = [x.clone() for _ in range(S)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        subs = [(1, lambda h: (gla_mixer if layer["type"] == "gla" else diff_attention_mixer)(
            h, W, p + "mix.", layer["mixer"], eps))]
        if layer.get("mlp") is not None:
            mlp = layer["mlp"]
            subs.append((2, lambda h: dense_ff(h, W, p + "mlp.") if mlp["kind"] == "dense"
                         else moe_ff(h, W, p + "mlp.", mlp, margins)))
        for qn, fn in subs:
            if has_streams:
                u = streams_read(X, W[f"{p}hc{qn}.in"])
            else:
                u = X[0]
            y = fn(rh(zero_centred_norm(u, W[f"{p}norm{qn}"], eps))) * W[f"{p}ls{qn}"]
            if has_streams:
                X = streams_write(X, y, W[f"{p}hc{qn}.mix"], W[f"{p}hc{qn}.out"])
            else:
                X = [X[0] + y]
        if layers_out is not None:
            layers_out.append(sum(X))
    x = sum(X)
    return rh(zero_centred_norm(x, W["final.norm"], eps)) @ W["embed"].T


def logits(cfg, W, tokens):
    return forward(cfg, W, tokens)


def routing_margins(cfg, W, tokens):
    """Per position the smallest margin by which any router of the model chose (infinity without routers)."""
    m = []
    forward(cfg, W, tokens, margins=m)
    out = torch.full((len(tokens),), float("inf"), dtype=F64)
    for x in m:
        out = torch.minimum(out, x)
    return out


def generate_greedy(cfg, W, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(forward(cfg, W, ids)[-1].argmax()))
    return ids[len(prompt):]
