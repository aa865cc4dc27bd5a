"""A plain, slow implementation of the Sopalorn decoder in float64 numpy: one function per mechanism, whole
sequences, token by token where a recurrence runs.  It shares no code with the package; the tests hold the package
to it.  ``cfg`` is the model's config.json as a dict, ``w`` maps tensor names to float64 arrays."""
from __future__ import annotations

import math

import numpy as np


# ------------------------------------------------------------------ small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def layer_norm(x, gain, bias, eps):
    mean = np.mean(x, axis=-1, keepdims=True)
    dev = x - mean
    return dev / np.sqrt(np.mean(dev * dev, axis=-1, keepdims=True) + eps) * gain + bias


# ------------------------------------------------------------------ positions
def rotary_frequencies(rot):
    """Frequencies of the rotated pairs, with the blend over a ramp of pair indices where ``scaling`` is given."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    grow = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])
        index = lambda turns: dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(index(float(sc["fast"]))), 0)
        hi = min(math.ceil(index(float(sc["slow"]))), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        grow = 0.1 * math.log(factor) + 1.0
    return f, grow


def rotate_interleaved(x, positions, rot):
    """x [T, heads, dim]: channels 2i and 2i+1 of a head's first ``dims`` channels turn by position * f_i."""
    if not rot:
        return x
    dims = int(rot["dims"])
    f, grow = rotary_frequencies(rot)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(angle) * grow)[:, None, :], (np.sin(angle) * grow)[:, None, :]
    out = x.copy()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ------------------------------------------------------------------ attention
def softmax_attention(q, k, v, scale, window=None, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, vd] of one sequence from position 0.  Query i sees key j <= i, and with a
    window only i - j < window.  ``sink`` [H]: one more term exp(sink_h) in head h's denominator, without a value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = s.max() if sink is None else max(s.max(), sink[h])
            e = np.exp(s - m)
            den = e.sum() + (0.0 if sink is None else math.exp(sink[h] - m))
            out[i, h] = (e / den) @ v[lo:i + 1, g]
    return out


def attention_keys_values(m, w, p, h, positions, eps):
    """The keys (normed and rotated, as a cache would hold them) and values of an attention layer with projections."""
    G, d, vd = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    k = h @ w[p + "k"].T
    k = rms(k, eps) * w[p + "k.norm"]
    k = rotate_interleaved(k.reshape(-1, G, d), positions, m.get("rot"))
    return k, (h @ w[p + "v"].T).reshape(-1, G, vd)


def attention_mixer(m, w, p, h, positions, eps, shared=None):
    """``shared``: (keys, values) of the layer that ``kv_from`` names, instead of projections of its own."""
    H, d = int(m["heads"]), int(m["dim"])
    q = h @ w[p + "q"].T
    q = rms(q, eps) * w[p + "q.norm"]
    q = rotate_interleaved(q.reshape(-1, H, d), positions, m.get("rot"))
    k, v = shared if shared is not None else attention_keys_values(m, w, p, h, positions, eps)
    o = softmax_attention(q, k, v, float(m["scale"]), None, np.zeros(H))        # a sink of score 0: one in the denominator
    return o.reshape(len(h), -1) @ w[p + "o"].T, (k, v)


def windowed_sink_attention(m, w, p, h):
    H, G, d, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T).reshape(-1, H, d)
    k = (h @ w[p + "k"].T).reshape(-1, G, d)
    v = (h @ w[p + "v"].T).reshape(-1, G, vd)
    window = int(m["mask"]["size"]) if m.get("mask") else None
    o = softmax_attention(q, k, v, float(m["scale"]), window, w[p + "sink"])
    return o.reshape(len(h), -1) @ w[p + "o"].T


# ------------------------------------------------------------------ recurrences
def lightning_mixer(m, w, p, h, eps):
    H, d, vd = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    T = len(h)
    q = silu(h @ w[p + "q"].T).reshape(T, H, d)
    k = silu(h @ w[p + "k"].T).reshape(T, H, d)
    v = silu(h @ w[p + "v"].T).reshape(T, H, vd)
    decay = np.asarray(m["decay"], dtype=np.float64)
    S = np.zeros((H, d, vd))
    o = np.zeros((T, H, vd))
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    y = rms(o.reshape(T, H * vd), eps) * w[p + "norm"] * sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def short_convolution(x, taps):
    """x [T, C], taps [C, K] with the last column the current token's; zeros before the sequence's start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C)), x], axis=0)
    out = np.zeros((T, C))
    for i in range(K):
        out += padded[i:i + T] * taps[:, i][None, :]
    return out


def gated_delta_rule(m, w, p, h, eps):
    H, G, d, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = len(h)
    q = silu(short_convolution(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, d)
    k = silu(short_convolution(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, d)
    v = silu(short_convolution(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, vd)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[p + "b"].T)                                           # [T, H]
    g = np.exp(-np.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    S = np.zeros((H, d, vd))
    o = np.zeros((T, H, vd))
    for t in range(T):
        for hh in range(H):
            kk, qq = k[t, hh // (H // G)], q[t, hh // (H // G)]
            S[hh] *= g[t, hh]
            u = beta[t, hh] * (v[t, hh] - S[hh].T @ kk)
            S[hh] += np.outer(kk, u)
            o[t, hh] = S[hh].T @ qq
    y = rms(o, eps) * w[p + "norm"] * silu(h @ w[p + "g"].T).reshape(T, H, vd)
    return y.reshape(T, H * vd) @ w[p + "o"].T


def parallel_mixer(m, w, p, h, eps):
    left = windowed_sink_attention(m["left"], w, p + "left.", h)
    right = gated_delta_rule(m["right"], w, p + "right.", h, eps)
    return 0.5 * (rms(left, eps) * w[p + "left.out"] + rms(right, eps) * w[p + "right.out"])


# ------------------------------------------------------------------ feed-forward
def dense_feed_forward(mlp, w, p, h):
    limit = float(mlp["limit"])
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(r, z, correction):
    """z [T, experts + identity] -> (chosen [T, top], weights [T, top])."""
    top = int(r["top"])
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    s = e / e.sum(axis=-1, keepdims=True)
    chosen = np.argsort(-(s + correction), axis=-1, kind="stable")[:, :top]
    ws = np.take_along_axis(s, chosen, axis=-1)
    return chosen, ws / (ws.sum(axis=-1, keepdims=True) + 1e-20) * float(r["scale"])


def expert_feed_forward(mlp, w, p, h):
    r = mlp["router"]
    real = int(r["experts"])
    chosen, weights = route(r, h @ w[p + "router"].T, w[p + "correction"])
    out = np.zeros_like(h)
    for t in range(len(h)):
        for e, wt in zip(chosen[t], weights[t]):
            if e >= real:
                out[t] += wt * h[t]                                             # an identity expert
            else:
                q = f"{p}e{e}."
                out[t] += wt * ((silu(w[q + "gate"] @ h[t]) * (w[q + "up"] @ h[t])) @ w[q + "down"].T)
    return out


# ------------------------------------------------------------------ the model
def forward(cfg, w, tokens):
    """Logits [T, vocab] and the stream (the sum of the copies) after every layer [layers, T, width] of one sequence."""
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    positions = np.arange(T)
    x0 = w["embed"][np.asarray(tokens)] * float(cfg["embedding"]["scale"])
    copies = cfg.get("streams")                      # absent: one stream and the plain residual sum
    n_streams = int(copies or 1)
    xs = [x0.copy() for _ in range(n_streams)]
    after, caches = [], {}

    def sublayer(i, which, fn):
        nonlocal xs
        p = f"l{i}."
        hc = f"{p}hc{which}."
        if copies is None:
            xs = [xs[0] + fn(layer_norm(xs[0], w[f"{p}norm{which}"], w[f"{p}norm{which}.b"], eps)) * w[f"{p}ls{which}"]]
            return
        u = sum(w[hc + "in"][s] * xs[s] for s in range(n_streams))
        y = fn(layer_norm(u, w[f"{p}norm{which}"], w[f"{p}norm{which}.b"], eps)) * w[f"{p}ls{which}"]
        xs = [sum(w[hc + "mix"][s, t] * xs[s] for s in range(n_streams)) + w[hc + "out"][t] * y for t in range(n_streams)]

    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "attention":
            def mix(h, i=i, m=m, p=p):
                shared = caches[m["kv_from"]] if m.get("kv_from") is not None else None
                y, caches[i] = attention_mixer(m, w, p, h, positions, eps, shared)
                return y
        elif layer["type"] == "lightning":
            mix = lambda h, m=m, p=p: lightning_mixer(m, w, p, h, eps)
        elif layer["type"] == "parallel":
            mix = lambda h, m=m, p=p: parallel_mixer(m, w, p, h, eps)
        else:
            raise ValueError(layer["type"])
        sublayer(i, 1, mix)
        mlp = layer.get("mlp")
        if mlp is not None:
            ff = dense_feed_forward if mlp["kind"] == "dense" else expert_feed_forward
            sublayer(i, 2, lambda h, mlp=mlp, ff=ff: ff(mlp, w, f"l{i}.mlp.", h))
        after.append(sum(xs))
    x = layer_norm(sum(xs), w["final.norm"], w["final.norm.b"], eps)
    return (x @ w["head"].T) * float(cfg["logit_scale"]), np.stack(after)
