"""Plain torch references of every kernel wrapper in ``dotllm_b200.kernels.ops``, with the same
signatures, on whatever device the tensors live on.

Two uses: each CUDA kernel is compared with its function here, alone and at sizes the engine
does not use; and the CPU tests swap these in for the CUDA wrappers to exercise the engine's
host logic.  Arithmetic is float32 (float64 where it is free); results are rounded to the dtype
the kernel writes.  Formulas as in tests/plain_llama.py, which cites the reference.
"""
from __future__ import annotations

import torch

import plain_llama

PAGE = 64


def gather_rows(table, ids, out=None, out_dtype=torch.float32):
    res = table[ids.long()].to(out_dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def add_rmsnorm(residual, delta, gain, eps, out_dtype, lazy=False):
    if hasattr(delta, "gain") and hasattr(delta, "extra"):          # a branch with a norm of its own
        return add_normed_branch(residual, delta, gain, eps, out_dtype)
    if hasattr(delta, "tensor"):
        delta = delta.tensor()
    if delta is not None:
        residual += delta.to(torch.float32)
    return plain_llama.rms_norm(residual, gain, eps).to(out_dtype)


def _rms(x, eps):
    x = x.to(torch.float32)
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def add_normed_branch(residual, branch, gain=None, eps=0.0, out_dtype=None):
    data = branch.data.tensor() if hasattr(branch.data, "tensor") else branch.data
    residual += _rms(data, branch.eps) * branch.gain
    if branch.extra is not None:
        residual += branch.extra
    return None if gain is None else (_rms(residual, eps) * gain).to(out_dtype)


def add_rows(residual, other):
    residual += other
    return residual


def embed_positions(table, pos_table, ids, positions):
    return table[ids.long()].to(torch.float32) + pos_table[positions.long()].to(torch.float32)


def gated_activation(gate_up, kind, limit=0.0, alpha=1.0):
    i = gate_up.shape[1] // 2
    g, u = gate_up[:, :i].to(torch.float32), gate_up[:, i:].to(torch.float32)
    if kind == "silu":
        y = g * torch.sigmoid(g) * u
    elif kind == "gelu_tanh":
        y = 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3))) * u
    else:
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
        y = g * torch.sigmoid(alpha * g) * (u + 1.0)
    return y.to(gate_up.dtype)


def gla_scan(q, k, v, z, z_bias, cu_new, slots, state, n_heads, dim, vdim, q_scale, tau=1.0):
    T = q.shape[0]
    out = torch.zeros((T, n_heads * vdim), dtype=torch.float32, device=q.device)
    qf, kf, vf = q.to(torch.float32), k.to(torch.float32), v.to(torch.float32)
    if z is None:                                           # one constant decay per head; silu on the way in
        alpha = z_bias.view(1, n_heads, 1).expand(T, n_heads, dim)
        qf, kf, vf = (t * torch.sigmoid(t) for t in (qf, kf, vf))
    else:
        alpha = torch.exp(torch.nn.functional.logsigmoid(z.to(torch.float32) + z_bias) / tau).view(T, n_heads, dim)
    qf = qf.reshape(T, n_heads, dim) * q_scale
    kf, vf = kf.reshape(T, n_heads, dim), vf.reshape(T, n_heads, vdim)
    for b in range(slots.numel()):
        S = state[int(slots[b])]
        for t in range(int(cu_new[b]), int(cu_new[b + 1])):
            S.mul_(alpha[t][:, :, None]).add_(kf[t][:, :, None] * vf[t][:, None, :])
            out[t] = torch.einsum("hdv,hd->hv", S, qf[t]).reshape(-1)
    return out


def head_norm_gate(o, g, gain, n_heads, vdim, eps, out_dtype, gate="silu"):
    T = o.shape[0]
    y = _rms(o.view(T, n_heads, vdim), eps) * gain
    gf = g.to(torch.float32).reshape(T, n_heads, vdim)
    act = torch.sigmoid(gf) if gate == "sigmoid" else gf * torch.sigmoid(gf)
    return (y * act).reshape(T, n_heads * vdim).to(out_dtype)


def head_rmsnorm(x, gain_a, heads_a, dim, eps, gain_b=None, heads_b=0):
    T = x.shape[0]
    xf = x.to(torch.float32).reshape(T, heads_a + heads_b, dim)
    y = _rms(xf, eps)
    y = torch.cat([y[:, :heads_a] * gain_a] + ([y[:, heads_a:] * gain_b] if heads_b else []), dim=1)
    return y.reshape(T, -1).to(x.dtype)


def delta_rule(x, taps, b_logit, z, dt_bias, a_log, token_seq, cu_new, slots, memory, n_heads, n_kv_heads, dim, vdim,
               q_scale, unit_eps, head_decay=False):
    """Sequence by sequence, token by token, from and into the slot's memory (states, then the convolution's history)."""
    T, H, G = x.shape[0], n_heads, n_kv_heads
    C, K = taps.shape
    n_state = H * dim * vdim
    out = torch.zeros((T, H * vdim), dtype=torch.float32, device=x.device)
    tf = taps.to(torch.float32)
    for b in range(slots.numel()):
        mem = memory[int(slots[b])]
        S = mem[:n_state].view(H, dim, vdim)
        hist = mem[n_state:].view(K - 1, C)
        for t in range(int(cu_new[b]), int(cu_new[b + 1])):
            now = x[t, :C].to(torch.float32)
            window = torch.cat([hist, now[None]], dim=0)                    # the K inputs the taps meet, oldest first
            y = (window * tf.T).sum(dim=0)
            y = y * torch.sigmoid(y)
            if K > 1:
                hist.copy_(window[1:].clone())
            q = y[:G * dim].view(G, dim)
            k = y[G * dim:2 * G * dim].view(G, dim)
            v = y[2 * G * dim:].view(H, vdim)
            q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + unit_eps) * q_scale
            k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
            q, k = q.repeat_interleave(H // G, dim=0), k.repeat_interleave(H // G, dim=0)
            beta = torch.sigmoid(b_logit[t].to(torch.float32))
            zt = (z[t] + dt_bias).view(H, 1).expand(H, dim) if head_decay else (z[t] + dt_bias).view(H, dim)
            g = torch.exp(-torch.exp(a_log)[:, None] * torch.nn.functional.softplus(zt))
            S.mul_(g[:, :, None])
            u = beta[:, None] * (v - torch.einsum("hdv,hd->hv", S, k))
            S.add_(k[:, :, None] * u[:, None, :])
            out[t] = torch.einsum("hdv,hd->hv", S, q).reshape(-1)
    return out


class StreamWrite:
    def __init__(self, data, scale, mix, out):
        self.data, self.scale, self.mix, self.out = data, scale, mix, out
        self.shape = tuple(data.shape)

    def narrowed(self, ids):
        return StreamWrite(self.data[ids.long()], self.scale, self.mix, self.out)


def stream_norm(x, copies, write, read, gain, bias, eps, out_dtype, kind="layernorm", summed=False):
    T, S = x.shape[0], int(copies)
    xs = x.view(T, S, -1)
    if write is not None:
        y = write.data.to(torch.float32) * (write.scale if write.scale is not None else 1.0)
        xs.copy_(torch.einsum("sr,tsh->trh", write.mix, xs.clone()) + write.out[None, :, None] * y[:, None, :])
    u = xs.sum(dim=1) if read is None else torch.einsum("s,tsh->th", read, xs)
    normed = None
    if gain is not None:
        if kind == "layernorm":
            d = u - u.mean(dim=-1, keepdim=True)
            normed = d / torch.sqrt((d * d).mean(dim=-1, keepdim=True) + eps) * gain + (bias if bias is not None else 0.0)
        else:
            normed = _rms(u, eps) * gain
        normed = normed.to(out_dtype)
    return (normed, u) if summed else normed


def stream_copies(x, copies, factor=1.0):
    return (x * factor).repeat(1, int(copies))


def embed_copies(table, ids, copies, factor=1.0):
    return (table[ids.long()].to(torch.float32) * factor).repeat(1, int(copies))


def group_rmsnorm(x, gain, width_a, width_b, eps):
    xf = x.to(torch.float32)
    parts = [_rms(xf[:, :width_a], eps)] + ([_rms(xf[:, width_a:width_a + width_b], eps)] if width_b else [])
    return (torch.cat(parts, dim=1) * gain).to(x.dtype)


def pair_norm_sum(a, b, gain_a, gain_b, eps, weight_a=0.5, weight_b=0.5):
    return weight_a * _rms(a, eps) * gain_a + weight_b * _rms(b, eps) * gain_b


def scale_values(values, factor):
    return values.mul_(factor)


def unary_activation(x, kind):
    assert kind == "relu2"
    return (torch.relu(x.to(torch.float32)) ** 2).to(x.dtype)


def activated_linear(x, w, kind, resident=False):
    return unary_activation(linear(x, w, torch.float32), kind).to(x.dtype)


def softcap(values, cap):
    values.copy_(cap * torch.tanh(values / cap))
    return values


def head_gate(o, gate, n_heads, width):
    g = torch.sigmoid(gate.to(torch.float32))
    o.copy_((o.to(torch.float32).reshape(o.shape[0], n_heads, width) * g[:, :, None]).reshape(o.shape).to(o.dtype))
    return o


def route_topk(x, w_router, bias, top, scoring="softmax_chosen", experts=None, with_logits=False, groups=None,
               correction=None, normalise=False, weight_scale=1.0):
    logits = x.to(torch.float32) @ w_router.to(torch.float32).T
    z = logits[:, :experts] if experts is not None else logits
    if bias is not None:
        z = z + bias
    share = torch.softmax(z, dim=-1)                        # over every expert, before any is ruled out
    if correction is not None:                              # the choice goes by share + correction
        z = share + correction
    if groups:
        count, keep = groups
        left = z.reshape(z.shape[0], count, -1).max(dim=-1).values
        kept = torch.zeros_like(left, dtype=torch.bool)
        for _ in range(keep):                               # the best runs one by one, ties to the lower index
            best = left.max(dim=-1).values
            at = (left == best[:, None]).to(torch.int32).argmax(dim=-1)
            kept = kept.scatter(1, at[:, None], True)
            left = left.scatter(1, at[:, None], float("-inf"))
        out_of_reach = (~kept).repeat_interleave(z.shape[1] // count, dim=1)
        z = z.masked_fill(out_of_reach, float("-inf"))
    ids = torch.empty((x.shape[0], top), dtype=torch.int32, device=x.device)
    vals = torch.empty((x.shape[0], top), dtype=torch.float32, device=x.device)
    for j in range(top):                                   # ties go to the lower index
        best = z.max(dim=-1).values
        at = (z == best[:, None]).to(torch.int32).argmax(dim=-1)
        ids[:, j], vals[:, j] = at, best
        z = z.scatter(1, at[:, None], float("-inf"))
    if scoring == "softmax_all":
        weights = torch.gather(share, 1, ids.long())
        if normalise:
            weights = weights / (weights.sum(dim=-1, keepdim=True) + 1e-20)
        weights = weights * weight_scale
    else:
        weights = torch.sigmoid(vals) if scoring == "sigmoid" else torch.softmax(vals, dim=-1)
    return (ids, weights, logits) if with_logits else (ids, weights)


def expert_gate_up(x, ids, w_gate_up, kind, limit=0.0, alpha=1.0, row_scale=None):
    T, top = ids.shape
    act = (lambda y: unary_activation(y, kind)) if kind == "relu2" else (lambda y: gated_activation(y, kind, limit, alpha))
    scale = (lambda t, j: float(row_scale[t, j])) if row_scale is not None else (lambda t, j: 1.0)
    E = w_gate_up.shape[0]                                  # an id beyond the matrices (an identity expert) gives zeros here
    rows = [act((x[t:t + 1].to(torch.float32) * scale(t, j)) @ w_gate_up[int(ids[t, j]) % E].to(torch.float32).T)[0] * (int(ids[t, j]) < E)
            for t in range(T) for j in range(top)]
    width = w_gate_up.shape[1] if kind == "relu2" else w_gate_up.shape[1] // 2
    return torch.stack(rows).to(x.dtype) if rows else torch.zeros((0, width), dtype=x.dtype)


def expert_down(h, ids, weights, w_down, addend=None, addend_gate=None, identity=None):
    T, top = ids.shape
    E = w_down.shape[0]
    out = torch.zeros((T, w_down.shape[1]), dtype=torch.float32, device=h.device)
    for t in range(T):
        for j in range(top):
            w = 1.0 if weights is None else weights[t, j]
            e = int(ids[t, j])
            if e < E:
                out[t] += w * (w_down[e].to(torch.float32) @ h[t * top + j].to(torch.float32))
            elif identity is not None and e < E + identity[1]:
                out[t] += w * identity[0][t].to(torch.float32)
    if addend is None:
        return out
    return out + (addend if addend_gate is None else addend * torch.sigmoid(addend_gate[:, :1]))


def linear_per_head(x, w):
    H, b, a = w.shape
    T = x.shape[0]
    y = torch.einsum("tha,hba->thb", x.to(torch.float32).reshape(T, H, a), w.to(torch.float32))
    return y.reshape(T, H * b).to(x.dtype)


def _rotate(x, cos, sin, positions, n_heads, head_dim, rotary_dim):
    t = x.shape[0]
    xf = x.to(torch.float32).reshape(t, n_heads, head_dim)
    c, s = cos[positions.long()], sin[positions.long()]
    if rotary_dim == head_dim:
        return plain_llama.apply_rope(xf, c, s).reshape(t, n_heads * head_dim)
    half = rotary_dim // 2                          # the first rotary_dim channels in pairs (i, i + half), the rest as they are
    u, v = xf[..., :half], xf[..., half:rotary_dim]
    c, s = c[:, None, :], s[:, None, :]
    return torch.cat([u * c - v * s, u * s + v * c, xf[..., rotary_dim:]], dim=-1).reshape(t, n_heads * head_dim)


def rope_cache_write(q, k, v, cos, sin, rotary_dim, token_seq, token_pos, block_table,
                     k_pool, v_pool, n_heads, n_kv_heads, head_dim, write_cache=True, value_dim=None, biases=None):
    vd = value_dim or head_dim
    qb, kb, vb = biases if biases is not None else (None, None, None)
    if qb is not None:
        q.copy_((q.to(torch.float32) + qb).to(q.dtype))
    if rotary_dim:
        q.copy_(_rotate(q, cos, sin, token_pos, n_heads, head_dim, rotary_dim).to(q.dtype))
    if not write_cache:
        return
    kf = k.to(torch.float32) + kb if kb is not None else k
    vf = (v.to(torch.float32) + vb).to(v.dtype) if vb is not None else v
    kr = _rotate(kf, cos, sin, token_pos, n_kv_heads, head_dim, rotary_dim).to(k.dtype) if rotary_dim else kf.to(k.dtype)
    for t in range(q.shape[0]):
        pos = int(token_pos[t])
        page = int(block_table[int(token_seq[t]), pos // PAGE])
        assert page >= 0
        k_pool[page, :, pos % PAGE, :] = kr[t].reshape(n_kv_heads, head_dim)
        v_pool[page, :, :, pos % PAGE] = vf[t].reshape(n_kv_heads, vd)


def gather_kv(k_pool, v_pool, pages, length):
    """Keys and values [length, nkv, hd] of one sequence from its pages (float32)."""
    ks, vs = [], []
    for j in range(length):
        page = int(pages[j // PAGE])
        ks.append(k_pool[page, :, j % PAGE, :])
        vs.append(v_pool[page, :, :, j % PAGE])
    return torch.stack(ks).to(torch.float32), torch.stack(vs).to(torch.float32)


def _gather_some(k_pool, v_pool, pages, positions):
    """Keys and values of the listed positions only (a page that a window gave back is never touched)."""
    ks = [k_pool[int(pages[j // PAGE]), :, j % PAGE, :] for j in positions]
    vs = [v_pool[int(pages[j // PAGE]), :, :, j % PAGE] for j in positions]
    return torch.stack(ks).to(torch.float32), torch.stack(vs).to(torch.float32)


def attention(q, k_pool, v_pool, token_seq, token_pos, block_table, n_heads, n_kv_heads,
              head_dim, scale, window=0, plan=None, score_hook=None, value_dim=None, gate=None, keep_first=0, sinks=None):
    vd = value_dim or head_dim
    if score_hook or vd != head_dim or gate is not None or keep_first or sinks is not None:
        return _attention_general(q, k_pool, v_pool, token_seq, token_pos, block_table, n_heads, n_kv_heads, head_dim,
                                  scale, window, score_hook, vd, gate, keep_first, sinks)
    T = q.shape[0]
    out = torch.empty((T, n_heads * head_dim), dtype=torch.float32, device=q.device)
    for t in range(T):
        pos = int(token_pos[t])
        first = max(0, pos - window + 1) if window else 0
        pages = block_table[int(token_seq[t])]
        ks, vs = [], []
        for j in range(first, pos + 1):
            page = int(pages[j // PAGE])
            ks.append(k_pool[page, :, j % PAGE, :])
            vs.append(v_pool[page, :, :, j % PAGE])
        k = torch.stack(ks).to(torch.float32).reshape(len(ks), n_kv_heads * head_dim)
        v = torch.stack(vs).to(torch.float32).reshape(len(vs), n_kv_heads * head_dim)
        # one query at the last of these keys: the causal mask hides nothing
        out[t] = plain_llama.causal_attention(q[t:t + 1].to(torch.float32), k, v, n_heads, n_kv_heads,
                                              scale, position_offset=len(ks) - 1)[0]
    return out.to(q.dtype)


def _attention_general(q, k_pool, v_pool, token_seq, token_pos, block_table, n_heads, n_kv_heads, head_dim, scale,
                       window, hook, vd, gate, keep_first=0, sinks=None):
    """Scores capped (softcap * tanh(s / softcap)) and then biased by slope * (key - query position); values of
    their own width; a head's output times sigmoid of its gate logit; a sequence's first ``keep_first`` keys visible
    beyond the window; a sink per head in the denominator."""
    T = q.shape[0]
    out = torch.empty((T, n_heads * vd), dtype=torch.float32, device=q.device)
    group = n_heads // n_kv_heads
    for t in range(T):
        pos = int(token_pos[t])
        first = max(0, pos - window + 1) if window else 0
        seen = list(range(min(keep_first, first))) + list(range(first, pos + 1))
        k, v = _gather_some(k_pool, v_pool, block_table[int(token_seq[t])], seen)
        for h in range(n_heads):
            qh = q[t, h * head_dim:(h + 1) * head_dim].to(torch.float32)
            s = (k[:, h // group] @ qh) * scale
            if hook and hook.softcap > 0:
                s = hook.softcap * torch.tanh(s / hook.softcap)
            if hook and hook.slopes is not None:
                s = s + float(hook.slopes[h]) * (torch.tensor(seen, dtype=torch.float32) - pos)
            if sinks is None:
                w = torch.softmax(s, dim=0)
            else:                                           # one more term in the denominator, nothing in the numerator
                w = torch.softmax(torch.cat([s, sinks[h:h + 1].to(torch.float32)]), dim=0)[:-1]
            o = w @ v[:, h // group]
            out[t, h * vd:(h + 1) * vd] = o if gate is None else o * torch.sigmoid(gate[t, h].to(torch.float32))
    return out.to(q.dtype)


def swiglu(gate_up):
    i = gate_up.shape[1] // 2
    g, u = gate_up[:, :i].to(torch.float32), gate_up[:, i:].to(torch.float32)
    return plain_llama.swiglu(g, u).to(gate_up.dtype)


def linear(x, w, out_dtype=None, resident=False, lazy=False):
    y = x.to(torch.float32) @ w.to(torch.float32).T
    return y.to(out_dtype or x.dtype)


def gated_linear(x, w_gate_up, resident=False, kind="silu", limit=0.0, alpha=1.0):
    if kind != "silu":
        return gated_activation(linear(x, w_gate_up, torch.float32), kind, limit, alpha).to(x.dtype)
    return swiglu(linear(x, w_gate_up, torch.float32)).to(x.dtype)


def repetition_penalty(logits, prev, prev_len, penalty, window, row_map=None, append=None):
    for r in range(logits.shape[0]):
        h = int(row_map[r]) if row_map is not None else r
        if append is not None and int(append[0][r]) >= 0:
            prev[h, int(append[0][r])] = int(append[1][r])
        previous = prev[h, :int(prev_len[r])].tolist()
        logits[r] = plain_llama.apply_repetition_penalty(logits[r].cpu(), previous, float(penalty[r]),
                                                         int(window[r])).to(logits.device)
    return logits


def sample(logits, temperature=None, top_k=None, top_p=None, min_p=None, uniform=None, out=None, split=None):
    out = []
    for r in range(logits.shape[0]):
        row = logits[r].detach().cpu()
        t = float(temperature[r]) if temperature is not None else 0.0
        out.append(plain_llama.sample(
            row, [], temperature=t, top_k=int(top_k[r]) if top_k is not None else 0,
            top_p=float(top_p[r]) if top_p is not None else 1.0,
            min_p=float(min_p[r]) if min_p is not None else 0.0,
            r=float(uniform[r]) if uniform is not None else None))
    return torch.tensor(out, dtype=torch.int32, device=logits.device)
