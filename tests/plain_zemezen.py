"""Plain, slow Zemezen decoder: whole sequences, no cache, one function per mechanism.

The oracle that the engine's Zemezen model is compared with.  It shares no code with the package:
the configuration is a plain dict, the weights a dict of name -> tensor, and every mechanism is
written out with elementary torch operations on the CPU in float64 (stored bfloat16 weights are
exact there).

Notation.  x: the residual stream [T, W].  rms(x) = x / sqrt(mean(x^2) + eps).  A layer reads the
stream once: h = rms(x) * w1, then x += mixer(h) + ff(h).  A layer entry with ``weights_of`` j runs
with layer j's tensors.  Three mixers: a gated delta rule whose state decays per key channel
(``channel_delta``), attention over one latent per token (``latent_attention``), and attention whose
values are its unnormed, unrotated keys, under a sliding window that also keeps the sequence's first
tokens, with a learned sink in the softmax's denominator (``attention``).
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gain_norm(x, w, eps):
    return rms(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def embed(w, tokens):
    return w["embed"].to(F)[torch.as_tensor(tokens, dtype=torch.long)]


# ------------------------------------------------------------------------------- channel_delta
def short_convolution(x, taps, history=None):
    """y[t, c] = sum_i taps[c, i] * x[t - (K - 1) + i, c]; the last column meets the current token; what lies before the
    start is zero (or ``history``, the K - 1 inputs before x).  x [T, C], taps [C, K]."""
    T, C = x.shape
    K = taps.shape[1]
    before = torch.zeros(K - 1, C, dtype=x.dtype) if history is None else history
    padded = torch.cat([before, x], dim=0)
    y = torch.zeros_like(x)
    for i in range(K):
        y = y + padded[i:i + T] * taps[:, i]
    return y


def unit(x):
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def channel_decay(h, w, pre, heads, dim):
    """g = exp(-exp(A_log_h) * softplus(A2 (A1 h) + dt_bias)): [T, heads, dim], one per head and key channel."""
    z = (h @ w[pre + "a1"].to(F).T) @ w[pre + "a2"].to(F).T + w[pre + "dt_bias"].to(F)
    rate = torch.exp(w[pre + "A_log"].to(F))[None, :, None]
    return torch.exp(-rate * softplus(z).view(h.shape[0], heads, dim))


def delta_recurrence(q, k, v, g, beta, state=None):
    """Per head, token by token: S <- g * S (rows = key channels); u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
    q, k, g [T, H, d]; v [T, H, dv]; beta [T, H]; state [H, d, dv] or None.  Returns (o [T, H, dv], state)."""
    T, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=q.dtype) if state is None else state.clone()
    out = []
    for t in range(T):
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return (torch.stack(out) if out else torch.zeros(0, H, dv, dtype=q.dtype)), S


def channel_delta(h, w, pre, m, eps):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(short_convolution(h @ w[pre + "q"].to(F).T, w[pre + "q.conv"].to(F)))
    k = silu(short_convolution(h @ w[pre + "k"].to(F).T, w[pre + "k.conv"].to(F)))
    v = silu(short_convolution(h @ w[pre + "v"].to(F).T, w[pre + "v.conv"].to(F)))
    q = unit(q.view(T, G, d)) * d ** -0.5
    k = unit(k.view(T, G, d))
    share = H // G
    q = q.repeat_interleave(share, dim=1)              # head h reads q/k head h // share
    k = k.repeat_interleave(share, dim=1)
    beta = torch.sigmoid(h @ w[pre + "b"].to(F).T)
    g = channel_decay(h, w, pre, H, d)
    o, _ = delta_recurrence(q, k, v.view(T, H, dv), g, beta)
    o = rms(o, eps) * w[pre + "norm"].to(F)
    gate = torch.sigmoid((h @ w[pre + "g1"].to(F).T) @ w[pre + "g2"].to(F).T).view(T, H, dv)
    return (o * gate).reshape(T, H * dv) @ w[pre + "o"].to(F).T


# ---------------------------------------------------------------------------- latent attention
def masked_softmax_attention(q, k, v, scale, seen, sink=None):
    """q, k [T, H, d], v [T, H, dv], seen [T, T] bool (query i, key j) -> [T, H, dv].  ``sink`` [H]: the
    denominator also holds exp(sink_h), which has no value."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~seen, float("-inf"))
    if sink is None:
        p = torch.softmax(s, dim=-1)
    else:
        top = torch.maximum(s.max(dim=-1, keepdim=True).values, sink[:, None, None])
        e = torch.exp(s - top)
        p = e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink[:, None, None] - top))
    return torch.einsum("hij,jhd->ihd", p, v)


def causal(T):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return j <= i


def latent_attention(h, w, pre, m, eps):
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w[pre + "q"].to(F).T).view(T, H, d)
    c = gain_norm(h @ w[pre + "dkv"].to(F).T, w[pre + "dkv.norm"].to(F), eps)
    k = (c @ w[pre + "uk"].to(F).T).view(T, H, d)
    v = (c @ w[pre + "uv"].to(F).T).view(T, H, dv)
    o = masked_softmax_attention(q, k, v, m["scale"], causal(T))
    return o.reshape(T, H * dv) @ w[pre + "o"].to(F).T


# ------------------------------------------------------------------------------------ attention
def rotate_half(x, positions, dims, base):
    """x [T, H, d]: channel i < dims/2 is paired with i + dims/2; the pair (a, b) at position p becomes
    (a cos - b sin, b cos + a sin) with angle p * base^(-2i/dims).  Channels from ``dims`` on pass."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    angle = torch.as_tensor(positions, dtype=F)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def window_with_first(T, size, keep_first):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def attention(h, w, pre, m, eps):
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = (h @ w[pre + "q"].to(F).T).view(T, H, d)
    k = (h @ w[pre + "k"].to(F).T).view(T, G, d)
    v = k                                               # the values are the keys as projected
    q = gain_norm(q, w[pre + "q.norm"].to(F), eps)
    k = gain_norm(k, w[pre + "k.norm"].to(F), eps)
    pos = list(range(T))
    q = rotate_half(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half(k, pos, m["rot"]["dims"], m["rot"]["base"])
    share = H // G
    k = k.repeat_interleave(share, dim=1)
    v = v.repeat_interleave(share, dim=1)
    seen = window_with_first(T, m["mask"]["size"], m["mask"]["keep_first"])
    o = masked_softmax_attention(q, k, v, m["scale"], seen, sink=w[pre + "sink"].to(F))
    return o.reshape(T, H * d) @ w[pre + "o"].to(F).T


# --------------------------------------------------------------------------------- feed-forward
def gated_expert(h, w, pre):
    return (silu(h @ w[pre + "gate"].to(F).T) * (h @ w[pre + "up"].to(F).T)) @ w[pre + "down"].to(F).T


def route(h, w, pre, router):
    """Scores = softmax over all experts; experts lie in ``groups.count`` equal runs of neighbours, a run scores its
    best expert, only the ``groups.keep`` best runs stay eligible; of those the ``top`` largest scores are chosen and
    weigh their experts as they are."""
    E, top = router["experts"], router["top"]
    s = torch.softmax(h @ w[pre + "router"].to(F).T, dim=-1)
    groups = router.get("groups")
    eligible = torch.ones_like(s, dtype=torch.bool)
    if groups:
        n, keep = groups["count"], groups["keep"]
        best = s.view(-1, n, E // n).max(dim=-1).values
        kept = torch.topk(best, keep, dim=-1).indices
        mask = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        eligible = mask[:, :, None].expand(-1, -1, E // n).reshape(-1, E)
    chosen = torch.topk(s.masked_fill(~eligible, -1.0), top, dim=-1).indices
    return chosen, torch.gather(s, 1, chosen)


def moe_ff(h, w, pre, mlp):
    chosen, weight = route(h, w, pre, mlp["router"])
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            out[t] += g * gated_expert(h[t:t + 1], w, f"{pre}e{e}.")[0]
    return out


# --------------------------------------------------------------------------------------- model
MIXERS = {"channel_delta": channel_delta, "latent_attention": latent_attention, "attention": attention}


def layer(x, w, i, cfg):
    spec = cfg["layers"][i]
    owner = spec.get("weights_of", i)
    eps = cfg["norm"]["eps"]
    p = f"l{owner}."
    h = gain_norm(x, w[p + "norm1"].to(F), eps)
    branch = MIXERS[spec["type"]](h, w, p + "mix.", spec["mixer"], eps)
    mlp = spec.get("mlp")
    if mlp:
        branch = branch + (gated_expert(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp))
    return x + branch


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (float64)."""
    x = embed(w, tokens)
    after = []
    for i in range(len(cfg["layers"])):
        x = layer(x, w, i, cfg)
        after.append(x)
    logits = gain_norm(x, w["final.norm"].to(F), cfg["norm"]["eps"]) @ w["head"].to(F).T
    return (logits, torch.stack(after)) if return_layers else logits
