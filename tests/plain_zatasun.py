"""Plain, slow Zatasun: whole sequences, dense masks, explicit loops over
tokens, no cache, float64, one function for each mechanism.  It shares no code
with ``airframe_b200`` (its own reading of config.json and of the tensors).

Notation: h is a sublayer's input [T, width]; W x means a weight stored
[out, in] applied to a vector; positions count from 0.
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

def rms(x, eps, w=None):
    """x / sqrt(mean(x^2) + eps) over the last axis, times w when given."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + z.clamp_min(0.0)


# ---------------------------------------------------------------- rotation

def stretched_frequencies(base, dims, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2.  With ``scaling`` {factor, low, high, original}: a frequency whose
    wavelength 2 pi / f is shorter than original/high stays, one whose wavelength is longer than original/low
    is divided by factor, and in between the two are mixed: s = (original/wavelength - low) / (high - low),
    f <- (1 - s) f / factor + s f."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave < orig / high:
                pass
            elif wave > orig / low:
                f = f / factor
            else:
                s = (orig / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate_half(x, positions, freqs):
    """x [T, heads, d]: element i < n pairs with element i + n (n = number of frequencies); the pair (a, b)
    becomes (a cos - b sin, b cos + a sin) with the angle position * f_i; elements from 2n on pass."""
    n = freqs.numel()
    if n == 0:
        return x
    ang = positions.to(x.dtype)[:, None] * freqs.to(x.dtype)[None]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., :n], x[..., n:2 * n]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * n:]], dim=-1)


# ---------------------------------------------------------------- attention with a sink

def sink_attention(q, k, v, scale, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; head h reads group h // (H / G); position i sees every j <= i.
    The weights are exp(score) / (sum of exp(score) over the visible keys + exp(sink_h)): the sink adds to the
    denominator only."""
    T, H, d = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, h]) * scale
            m = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            out[i, h] = (e / (e.sum() + torch.exp(sink[h] - m))) @ v[: i + 1, g]
    return out


def whole_norm_attention(h, W, p, m, eps):
    """The left mixer: q and k are normed over their whole projection (all heads at once) with a weight of that
    size, then rotated; causal attention with a sink; output projection."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms(h @ W[p + "q"].T, eps, W[p + "q.norm"]).view(T, H, d)
    k = rms(h @ W[p + "k"].T, eps, W[p + "k.norm"]).view(T, G, d)
    v = (h @ W[p + "v"].T).view(T, G, dv)
    freqs = stretched_frequencies(m["rot"]["base"], m["rot"]["dims"], m["rot"].get("scaling"))
    pos = torch.arange(T)
    o = sink_attention(rotate_half(q, pos, freqs), rotate_half(k, pos, freqs), v, m["scale"], W[p + "sink"])
    return o.reshape(T, H * dv) @ W[p + "o"].T


# ---------------------------------------------------------------- the gated linear recurrence

def causal_conv(x, w, b):
    """x [T, C], w [C, taps] (the last column multiplies the current token, zeros before the start), b [C]."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x])
    out = torch.zeros_like(x)
    for t in range(T):
        out[t] = (padded[t: t + taps].T * w).sum(-1) + b
    return out


def gated_linear_recurrence(u, r, i, lam):
    """S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t from S = 0, with a_t = exp(-8 r_t softplus(lam))."""
    T, C = u.shape
    S = torch.zeros(C, dtype=u.dtype)
    out = torch.zeros_like(u)
    sp = softplus(lam)
    for t in range(T):
        a = torch.exp(-8.0 * r[t] * sp)
        S = a * S + torch.sqrt(1.0 - a * a) * i[t] * u[t]
        out[t] = S
    return out


def recurrent_block(h, W, p, m):
    """The right mixer: a gelu branch and a conv branch; the conv branch drives the recurrence whose gates come
    from block-diagonal matrices; the state times the gelu branch is projected out."""
    width, blocks = m["width"], m["blocks"]
    y = gelu_tanh(h @ W[p + "y"].T + W[p + "y.b"])
    u = causal_conv(h @ W[p + "x"].T + W[p + "x.b"], W[p + "conv"], W[p + "conv.b"])
    T = h.shape[0]
    ub = u.view(T, blocks, width // blocks)
    r = sigmoid(torch.einsum("boi,tbi->tbo", W[p + "ra"], ub) + W[p + "ra.b"]).reshape(T, width)
    i = sigmoid(torch.einsum("boi,tbi->tbo", W[p + "ri"], ub) + W[p + "ri.b"]).reshape(T, width)
    S = gated_linear_recurrence(u, r, i, W[p + "lam"])
    return (S * y) @ W[p + "o"].T


# ---------------------------------------------------------------- feed-forwards

def dense_ff(h, W, p):
    g = h @ W[p + "gate"].T
    return (g * sigmoid(g) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def clamped_expert(h, W, p, limit):
    g = (h @ W[p + "gate"].T).clamp(max=limit)
    u = (h @ W[p + "up"].T).clamp(-limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def routed_ff(h, W, p, mlp, margins=None):
    """Sigmoid scores from the router; the ``top`` largest choose the experts; a chosen expert's score multiplies
    its *input*; a shared expert runs for every token and is added times sigmoid(W_sg h).  ``margins`` (a list)
    receives, per token, by how much the last chosen score exceeds the first one left out."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = sigmoid(h @ W[p + "router"].T)
    out = torch.zeros_like(h)
    if margins is not None:
        ranked = s.sort(dim=-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top] if top < E else torch.full_like(s[:, 0], float("inf")))
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(s[t, e]), e))[:top]
        for e in order:
            out[t] += clamped_expert((s[t, e] * h[t])[None], W, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        gate = sigmoid(h @ W[p + "shared.sg"].T)
        out = out + gate * clamped_expert(h, W, p + "shared.", mlp["shared"]["limit"])
    return out


# ---------------------------------------------------------------- the model

def layer(x, W, i, spec, eps, margins=None):
    p = f"l{i}."
    m = spec["mixer"]
    mixed = (m["left_scale"] * whole_norm_attention(x, W, p + "mix.left.", m["left"], eps)
             + m["right_scale"] * recurrent_block(x, W, p + "mix.right.", m["right"]))
    x = x + rms(mixed, eps, W[p + "norm1"])
    mlp = spec["mlp"]
    if mlp is None:
        return x
    f = dense_ff(x, W, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(x, W, p + "mlp.", mlp, margins)
    return x + rms(f, eps, W[p + "norm2"])


def forward(cfg, W, tokens, return_layers=False, margins=None):
    """Logits [T, vocab] of one sequence (float64), and with ``return_layers`` the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = rms(W["embed"][torch.as_tensor(tokens, dtype=torch.long)], eps, W["embed.norm"])
    seen = []
    for i, spec in enumerate(cfg["layers"]):
        x = layer(x, W, i, spec, eps, margins)
        seen.append(x.clone())
    logits = (rms(x, eps, W["final.norm"]) @ W["embed"].T) * cfg["logit_scale"]
    return (logits, torch.stack(seen)) if return_layers else logits


def logits(cfg, W, tokens):
    return forward(cfg, W, tokens)


def routing_margins(cfg, W, tokens):
    """Per token, the smallest margin by which any of its routers chose (infinite without a choice to make):
    where it is tiny, a computation in fewer bits may choose otherwise and still be right."""
    seen = []
    forward(cfg, W, tokens, margins=seen)
    return torch.stack(seen).min(0).values if seen else torch.full((len(tokens),), float("inf"), dtype=F64)


def hidden_states(cfg, W, tokens, per_layer):
    """Appends the residual stream after every layer to ``per_layer``."""
    _, seen = forward(cfg, W, tokens, return_layers=True)
    per_layer.extend(seen)


def generate_greedy(cfg, W, prompt, n):
    ids = list(prompt)
    out = []
    for _ in range(n):
        nxt = int(forward(cfg, W, ids)[-1].argmax())
        out.append(nxt)
        ids.append(nxt)
    return out
