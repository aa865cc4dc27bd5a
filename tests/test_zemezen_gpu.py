"""Zemezen on the GPU against the plain implementation: each mechanism's kernel alone, whole prompts, portions,
token-by-token decoding, unequal batches, slots, states and pages that are used again, keys just inside and just outside
the window and the kept first tokens, long decoding over page borders, generation through the entry point, the replay
program, the command line."""
import copy
import json
import os
import random
import subprocess

import numpy as np
import pytest
import torch

import kernel_refs
import plain_zemezen as pz
import tiny_zemezen as tz
from dotllm_b200.kernels import ops

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]
# A row's rms error over the row's rms.  float32: summation order only, every row is held to the bound.
# bfloat16: both sides read the same bfloat16 weights; the engine rounds activations to bfloat16 between parts.  A router
# whose best scores nearly tie may choose the other expert in bfloat16, which changes that token's row and no other; so
# nine rows in ten are held to HALF the bound, all but 3 % to the bound, and none may exceed LOOSE.
REL = {torch.float32: 3e-5, torch.bfloat16: 4e-2}
LOOSE = 0.6


def row_errors(got, want):
    g, w = got.double().cpu().reshape(-1, got.shape[-1]), want.double().cpu().reshape(-1, want.shape[-1])
    return (g - w).pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-30)


def rel_err(got, want):
    return float(row_errors(got, want).max())


def assert_rows(got, want, dtype, what="", loose=LOOSE):
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    err = row_errors(got, want)
    if dtype == torch.float32:
        assert float(err.max()) <= REL[dtype], f"{what}: a row's rms error is {float(err.max()):.3e} of its rms > {REL[dtype]:.1e}"
        return
    over = int((err > REL[dtype]).sum())
    assert float(err.max()) <= loose and over <= max(1, int(0.03 * err.numel())), \
        f"{what}: {over} of {err.numel()} rows beyond {REL[dtype]:.1e}, the worst {float(err.max()):.3e}"
    if err.numel() >= 10:
        assert float(err.quantile(0.9)) <= REL[dtype] / 2, f"{what}: nine rows in ten should be within {REL[dtype] / 2:.1e}"


@pytest.fixture(scope="module")
def tmp(tmp_path_factory):
    return tmp_path_factory.mktemp("zemezen")


_loaded = {}


def load_pair(tmp, which, dtype, seed=0):
    from dotllm_b200 import Model
    key = (which, dtype, seed)
    if key not in _loaded:
        folder = tz.sharp_folder(tmp, dtype=dtype, seed=seed, sink=20.0) if which == "sharp" else \
            tz.sharp_folder(tmp, dtype=dtype, seed=seed, sink=2.0, gains=0.25) if which == "soft" else \
            tz.make_folder(tmp, which, seed=seed, dtype=dtype)
        cfg, weights = tz.read_folder(folder)
        _loaded[key] = (Model.load(folder, dtype=dtype), cfg, weights, folder)
    return _loaded[key]


def g64(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64) * scale


def close(got, want, dtype, tol32=2e-5, tol16=2e-2):
    scale = float(want.double().abs().max().clamp_min(1e-6))
    err = float((got.double().cpu() - want.double().cpu()).abs().max()) / scale
    assert err <= (tol32 if dtype == torch.float32 else tol16), err


def run_cuts(model, tokens, cuts):
    """Feed ``tokens`` to a fresh sequence in portions of the given sizes, the rest one by one; the logits of every token."""
    from dotllm_b200.engine import StepEntry
    cache = model.new_cache(64 * ((len(tokens) + 63) // 64 + 1))
    cache.fill_free_pages(float("nan"))
    seq = cache.open_sequence()
    outs, at = [], 0
    sizes = list(cuts)
    while at < len(tokens):
        n = min(sizes.pop(0) if sizes else 1, len(tokens) - at)
        outs.append(model.step(cache, [StepEntry(seq, tokens[at:at + n], list(range(n)))]).clone())
        at += n
    cache.close_sequence(seq)
    cache.check()
    return torch.cat(outs)


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dim,vdim,K", [(4, 2, 24, 20, 3), (2, 2, 64, 64, 4), (3, 3, 10, 7, 1), (6, 2, 16, 24, 5), (2, 1, 128, 128, 4),
                                           (1, 1, 200, 33, 2), (2, 1, 512, 16, 2), (8, 8, 8, 130, 4), (2, 1, 16, 12, 7), (1, 1, 8, 8, 11), (2, 2, 8, 4, 20)])
def test_delta_rule_kernels_alone(H, G, dim, vdim, K, dtype):
    """Convolutions with their history, unit lengths, step sizes, decays and the recurrence: a step of three unequal
    prompts (one of a single token, one shorter than the taps), a step of portions of two, one and eight tokens, then
    three steps of one token each; slots that are not neighbours; the memory around the used slots stays as it was."""
    C = 2 * G * dim + H * vdim
    n_state = H * dim * vdim
    taps = g64(C, K, seed=1, scale=0.5).to(dtype)
    dt_bias, a_log = g64(H * dim, seed=2).float(), g64(H, seed=3, scale=0.5).float()
    memory = torch.zeros(7, n_state + (K - 1) * C)
    memory[[0, 3, 6]] = 7.0                                                   # slots that no sequence of the step owns
    slots = torch.tensor([4, 1, 5], dtype=torch.int32)
    want_mem, got_mem = memory.clone(), memory.clone().to(DEV)
    dev = lambda t: t.to(DEV)
    for round_, news in enumerate(([37, 1, 2], [2, 1, 8], [1, 1, 1], [1, 1, 1], [1, 1, 1])):
        T = sum(news)
        x = g64(T, C + 5 + H + 3, seed=10 + round_).to(dtype)                 # the channels, other columns, the step sizes, padding
        b = x[:, C + 5:C + 5 + H]
        z = g64(T, H * dim, seed=20 + round_).float()
        seq = torch.tensor([i for i, n in enumerate(news) for _ in range(n)], dtype=torch.int32)
        cu = torch.tensor([0] + list(np.cumsum(news)), dtype=torch.int32)
        want = kernel_refs.delta_rule(x, taps, b, z, dt_bias, a_log, seq, cu, slots, want_mem, H, G, dim, vdim, dim ** -0.5, 1e-6)
        gx = dev(x)
        got = ops.delta_rule(gx, dev(taps), gx[:, C + 5:C + 5 + H], dev(z), dev(dt_bias), dev(a_log), dev(seq), dev(cu), dev(slots),
                             got_mem, H, G, dim, vdim, dim ** -0.5, 1e-6)
        close(got, want, dtype, 3e-5, 3e-5)                                   # float32 from the convolution on in either run
        close(got_mem, want_mem, dtype, 3e-5, 3e-5)
    assert torch.equal(got_mem.cpu()[[0, 3, 6]], memory[[0, 3, 6]]) and float(got_mem[2].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("K", [4, 6])
def test_delta_rule_long_steps_of_several_sequences(K, dtype):
    """Steps long enough that a block of the convolution's kernel walks a run of tokens: sequences begin and end inside
    runs, one is a single token between two long ones, one is shorter than the taps; then the same sequences go on."""
    H, G, dim, vdim = 8, 4, 8, 16
    C = 2 * G * dim + H * vdim
    n_state = H * dim * vdim
    taps = g64(C, K, seed=1, scale=0.5).to(dtype)
    dt_bias, a_log = g64(H * dim, seed=2).float(), g64(H, seed=3, scale=0.5).float()
    memory = torch.zeros(6, n_state + (K - 1) * C)
    slots = torch.tensor([4, 1, 5, 2], dtype=torch.int32)
    want_mem, got_mem = memory.clone(), memory.clone().to(DEV)
    dev = lambda t: t.to(DEV)
    for round_, news in enumerate(([301, 1, 212, 2], [3, 170, 1, 401], [1, 1, 1, 1])):
        T = sum(news)
        x = g64(T, C + H, seed=30 + round_).to(dtype)
        z = g64(T, H * dim, seed=40 + round_).float()
        seq = torch.tensor([i for i, n in enumerate(news) for _ in range(n)], dtype=torch.int32)
        cu = torch.tensor([0] + list(np.cumsum(news)), dtype=torch.int32)
        want = kernel_refs.delta_rule(x, taps, x[:, C:], z, dt_bias, a_log, seq, cu, slots, want_mem, H, G, dim, vdim, dim ** -0.5, 1e-6)
        gx = dev(x)
        got = ops.delta_rule(gx, dev(taps), gx[:, C:], dev(z), dev(dt_bias), dev(a_log), dev(seq), dev(cu), dev(slots), got_mem,
                             H, G, dim, vdim, dim ** -0.5, 1e-6)
        close(got, want, dtype, 1e-4, 1e-4)
        close(got_mem, want_mem, dtype, 1e-4, 1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
def test_delta_rule_does_not_depend_on_the_cut(dtype):
    """The same tokens as one step, as portions, and one by one give the same bits (every sum runs in an order that the
    position fixes), also with a neighbour in the batch."""
    H, G, dim, vdim, K, T = 3, 1, 40, 24, 4, 50
    C = 2 * G * dim + H * vdim
    x, taps = g64(T, C + H, seed=1).to(dtype).to(DEV), g64(C, K, seed=2, scale=0.5).to(dtype).to(DEV)
    z, dt_bias, a_log = g64(T, H * dim, seed=3).float().to(DEV), g64(H * dim, seed=4).float().to(DEV), g64(H, seed=5).float().to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)

    def run(cuts, neighbour=False):
        memory = torch.zeros(3, H * dim * vdim + (K - 1) * C, device=DEV)
        out, at = [], 0
        for n in cuts:
            xs, zs = x[at:at + n], z[at:at + n]
            seq, cu, slots = [0] * n, [0, n], [2]
            if neighbour:                                                     # another sequence's token rides in front
                xs, zs = torch.cat([x[7:8], xs]), torch.cat([z[7:8], zs])
                seq, cu, slots = [0] + [1] * n, [0, 1, n + 1], [0, 2]
            o = ops.delta_rule(xs, taps, xs[:, C:], zs, dt_bias, a_log, i32(seq), i32(cu), i32(slots), memory, H, G, dim, vdim, 0.2, 1e-6)
            out.append(o[1:] if neighbour else o)
            at += n
        return torch.cat(out), memory[2].clone()

    whole, mem = run([T])
    for cuts, neighbour in (([17, 2, 31], False), ([1] * T, False), ([30] + [1] * 20, True)):
        got, m = run(cuts, neighbour)
        assert torch.equal(got, whole) and torch.equal(m, mem), cuts


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_norms_alone(dtype):
    x = g64(9, (5 + 2) * 24 + 8, seed=1).to(dtype)
    ga, gb = g64(24, seed=2).float(), g64(24, seed=3).float()
    want = kernel_refs.head_rmsnorm(x[:, :7 * 24], ga, 5, 24, 1e-5, gb, 2)
    got = ops.head_rmsnorm(x.to(DEV)[:, :7 * 24], ga.to(DEV), 5, 24, 1e-5, gb.to(DEV), 2)
    close(got, want, dtype, 2e-6, 1e-2)
    close(ops.head_rmsnorm(x.to(DEV)[:, 24:4 * 24], gb.to(DEV), 3, 24, 1e-3), kernel_refs.head_rmsnorm(x[:, 24:4 * 24], gb, 3, 24, 1e-3),
          dtype, 2e-6, 1e-2)
    o, g, gain = g64(6, 3 * 20, seed=4).float(), g64(6, 3 * 20, seed=5).to(dtype), g64(20, seed=6).float()
    for gate in ("silu", "sigmoid"):
        close(ops.head_norm_gate(o.to(DEV), g.to(DEV), gain.to(DEV), 3, 20, 1e-5, dtype, gate=gate),
              kernel_refs.head_norm_gate(o, g, gain, 3, 20, 1e-5, dtype, gate=gate), dtype, 2e-6, 1e-2)


def test_router_with_groups_alone():
    """Softmax over all experts, the best groups by their best expert, the largest scores among those; ties go to the
    lower index; groups of one expert, one group, every group kept."""
    for E, top, groups, seed in ((8, 4, (4, 3), 1), (6, 3, (3, 2), 2), (12, 2, (12, 5), 3), (9, 4, None, 4), (10, 5, (1, 1), 5),
                                 (64, 8, (8, 4), 6), (6, 6, (2, 2), 7)):
        x, wr = g64(40, 24, seed=seed).float(), g64(E, 24, seed=seed + 50).float()
        spec = {"experts": E, "top": top, **({"groups": {"count": groups[0], "keep": groups[1]}} if groups else {})}
        pid, pw = pz.route(x.double(), {"r.router": wr.double()}, "r.", spec)
        for tie in (False, True):
            if tie:
                wr[E - 1] = wr[0]                                             # the first and the last expert score alike
            ids, wts = ops.route_topk(x.to(DEV), wr.to(DEV), None, top, scoring="softmax_all", groups=groups)
            rid, rw = kernel_refs.route_topk(x, wr, None, top, scoring="softmax_all", groups=groups)
            assert torch.equal(ids.cpu(), rid), (E, top, groups)
            assert torch.allclose(wts.cpu(), rw, rtol=1e-5, atol=1e-7)
            if not tie:
                assert torch.equal(pid.sort(-1).values, rid.long().sort(-1).values)
                assert torch.allclose(pw.float().sort(-1).values, rw.sort(-1).values, rtol=1e-5)


def paged(lens, nkv, hd, dtype, seed):
    """Pools of NaN with room for sequences of the given lengths on shuffled pages; the block table."""
    pages = [(n + 63) // 64 for n in lens]
    total = sum(pages) + 3
    order = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).tolist()
    table = torch.full((len(lens), max(pages)), -1, dtype=torch.int32)
    k_pool = torch.full((total, nkv, 64, hd), float("nan"), dtype=dtype)
    v_pool = torch.full((total, nkv, hd, 64), float("nan"), dtype=dtype)
    at = 0
    for b, n in enumerate(pages):
        for p in range(n):
            table[b, p] = order[at]
            at += 1
    return k_pool, v_pool, table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,window,keep", [(6, 2, 24, 37, 3), (8, 2, 64, 70, 5), (4, 1, 128, 130, 70), (3, 1, 10, 1, 2),
                                                  (2, 2, 96, 6, 11), (4, 4, 32, 64, 64), (8, 2, 64, 5000, 0), (16, 1, 64, 33, 1)])
def test_windowed_attention_with_kept_tokens_and_sinks_alone(nh, nkv, hd, window, keep, dtype):
    """Attention over pages with a window, kept first tokens and a sink per head: prompts that cross pages, portions that
    start inside a page, one token each; the step's plan is given, so the bfloat16 run takes whichever kernel serves
    these sizes.  Pages that the window has passed (and that hold no kept token) are NaN."""
    from dotllm_b200.engine.step import AttentionPlan
    lens = [300, 80, 131]
    k_pool, v_pool, table = paged(lens, nkv, hd, dtype, 3)
    for b, n in enumerate(lens):
        for j in range(n):
            page = int(table[b, j // 64])
            k_pool[page, :, j % 64, :] = g64(nkv, hd, seed=1000 * b + j).to(dtype)
            v_pool[page, :, :, j % 64] = g64(nkv, hd, seed=5000 * b + j).to(dtype)
    sinks = g64(nh, seed=9, scale=2.0).float()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    gk, gv = k_pool.to(DEV), v_pool.to(DEV)
    for starts, news in (([0, 0, 0], [280, 70, 129]), ([280, 70, 129], [19, 9, 1]), ([299, 79, 130], [1, 1, 1])):
        T = sum(news)
        seq = torch.tensor([b for b, n in enumerate(news) for _ in range(n)], dtype=torch.int32)
        pos = torch.tensor([s + i for s, n in zip(starts, news) for i in range(n)], dtype=torch.int32)
        q = g64(T, nh * hd, seed=T).to(dtype)
        want = kernel_refs.attention(q, k_pool, v_pool, seq, pos, table, nh, nkv, hd, 0.3, window, keep_first=keep, sinks=sinks)
        totals = [s + n for s, n in zip(starts, news)]
        plan = AttentionPlan(3, max(news), max(totals), all(n == 1 for n in news), i32(starts), i32(news),
                             i32([0] + list(np.cumsum(news))), i32(totals), list(starts), list(news))
        # what a windowed cache has given back by now holds anything
        hidden_k, hidden_v = gk.clone(), gv.clone()
        for b in range(3):
            for p in range((keep + 63) // 64, max(0, (starts[b] - window + 1)) // 64):
                hidden_k[int(table[b, p])] = float("nan")
                hidden_v[int(table[b, p])] = float("nan")
        got = ops.attention(q.to(DEV), hidden_k, hidden_v, seq.to(DEV), pos.to(DEV), table.to(DEV), nh, nkv, hd, 0.3, window,
                            plan=plan, keep_first=keep, sinks=sinks.to(DEV))
        close(got, want, dtype, 2e-5, 2e-2)
        if dtype == torch.float32:
            no_sink = ops.attention(q.to(DEV), hidden_k, hidden_v, seq.to(DEV), pos.to(DEV), table.to(DEV), nh, nkv, hd, 0.3, window,
                                    keep_first=keep)
            assert float((no_sink.cpu() - want).abs().max()) > 1e-3


@pytest.mark.parametrize("nh,nkv,hd,window,keep", [(4, 2, 64, 200, 4), (4, 1, 128, 130, 70), (2, 2, 128, 64, 64), (4, 4, 64, 300, 129),
                                                  (2, 1, 128, 1, 1), (2, 2, 64, 1000, 200)])
def test_long_prompts_with_kept_tokens_and_sinks_on_both_prompt_kernels(nh, nkv, hd, window, keep, monkeypatch):
    """Prompts and portions of several hundred tokens in bfloat16, so that the window's first page lies well behind the kept
    pages and the two tiles of a block start on different pages: the tcgen05 kernel and the mma.sync kernel against the plain
    attention and against each other.  Pages between the kept ones and the step's first window are NaN."""
    from dotllm_b200.engine.step import AttentionPlan
    from dotllm_b200.kernels import attention_fast
    dtype = torch.bfloat16
    lens = [900, 333, 64, 700]
    k_pool, v_pool, table = paged(lens, nkv, hd, dtype, 11)
    gen = torch.Generator().manual_seed(3)
    for b, n in enumerate(lens):
        for p in range((n + 63) // 64):
            page = int(table[b, p])
            k_pool[page] = torch.randn(nkv, 64, hd, generator=gen).to(dtype)
            v_pool[page] = torch.randn(nkv, hd, 64, generator=gen).to(dtype)
    sinks = g64(nh, seed=9, scale=2.0).float()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    for starts, news in (([0, 0, 0, 0], [900, 333, 64, 700]), ([500, 300, 63, 1], [400, 33, 1, 699]), ([640, 0, 0, 448], [257, 2, 1, 129])):
        T = sum(news)
        seq = torch.tensor([b for b, n in enumerate(news) for _ in range(n)], dtype=torch.int32)
        pos = torch.tensor([s + i for s, n in zip(starts, news) for i in range(n)], dtype=torch.int32)
        q = (torch.randn(T, nh * hd, generator=gen) * 0.5).to(dtype)
        want = kernel_refs.attention(q, k_pool, v_pool, seq, pos, table, nh, nkv, hd, 0.2, window, keep_first=keep, sinks=sinks)
        totals = [s + n for s, n in zip(starts, news)]
        hidden_k, hidden_v = k_pool.clone().to(DEV), v_pool.clone().to(DEV)
        for b in range(len(lens)):
            for p in range((keep + 63) // 64, max(0, (starts[b] - window + 1)) // 64):
                hidden_k[int(table[b, p])] = float("nan")
                hidden_v[int(table[b, p])] = float("nan")
        outs = []
        for special in (True, False):
            monkeypatch.setattr(attention_fast, "PREFILL_TC_SPECIAL", special)
            plan = AttentionPlan(len(lens), max(news), max(totals), False, i32(starts), i32(news),
                                 i32([0] + list(np.cumsum(news))), i32(totals), list(starts), list(news))
            got = ops.attention(q.to(DEV), hidden_k, hidden_v, seq.to(DEV), pos.to(DEV), table.to(DEV), nh, nkv, hd, 0.2, window,
                                plan=plan, keep_first=keep, sinks=sinks.to(DEV))
            assert torch.isfinite(got.float()).all()
            close(got, want, dtype, 2e-5, 2e-2)
            outs.append(got.float().cpu())
        assert float((outs[0] - outs[1]).abs().max()) <= 2e-2
        no_sink = ops.attention(q.to(DEV), hidden_k, hidden_v, seq.to(DEV), pos.to(DEV), table.to(DEV), nh, nkv, hd, 0.2, window,
                                plan=AttentionPlan(len(lens), max(news), max(totals), False, i32(starts), i32(news),
                                                   i32([0] + list(np.cumsum(news))), i32(totals), list(starts), list(news)),
                                keep_first=keep)
        assert float((no_sink.float().cpu() - want).abs().max()) > 1e-3


@pytest.mark.parametrize("blocks", [0, 1, 3, 7])
@pytest.mark.parametrize("nh,nkv,hd,window,keep", [(8, 2, 64, 100, 3), (4, 4, 128, 64, 64), (12, 1, 32, 70, 130), (6, 2, 96, 129, 65),
                                                  (4, 2, 64, 1, 1), (2, 1, 64, 640, 200)])
def test_decode_steps_with_kept_tokens_and_sinks_over_cut_pages(nh, nkv, hd, window, keep, blocks, monkeypatch):
    """One new token per sequence, in bfloat16, through the decode kernel that shares the step's pages out to its blocks:
    sequences that end on a page's first and last place, shorter than the window, shorter than the kept tokens, and long
    ones whose kept pages and window pages land in different blocks (few blocks make every pair a cut one).  The pages
    between the kept ones and the window's are NaN.  The packed prompt kernel with tiles of one row gives the same."""
    from dotllm_b200.engine.step import AttentionPlan
    from dotllm_b200.kernels import attention_fast
    dtype = torch.bfloat16
    lens = [1000, 64, 65, 200, 129, 1, 3, 449]
    k_pool, v_pool, table = paged(lens, nkv, hd, dtype, 5)
    gen = torch.Generator().manual_seed(7)
    for b, n in enumerate(lens):
        for p in range((n + 63) // 64):
            page = int(table[b, p])
            k_pool[page] = torch.randn(nkv, 64, hd, generator=gen).to(dtype)
            v_pool[page] = torch.randn(nkv, hd, 64, generator=gen).to(dtype)
            first = max(0, n - window)
            if (p + 1) * 64 <= first and p * 64 >= keep:              # wholly hidden: between the kept tokens and the window
                k_pool[page], v_pool[page] = float("nan"), float("nan")
            if (p + 1) * 64 > n:                                      # places that no token has reached yet
                k_pool[page, :, n - p * 64:, :] = float("nan")
                v_pool[page, :, :, n - p * 64:] = float("nan")
    sinks = g64(nh, seed=11, scale=2.0).float()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    B = len(lens)
    starts, news = [n - 1 for n in lens], [1] * B
    seq, pos = torch.arange(B, dtype=torch.int32), torch.tensor(starts, dtype=torch.int32)
    q = g64(B, nh * hd, seed=13).to(dtype)
    scale = 0.2
    clean_k, clean_v = torch.nan_to_num(k_pool.float(), nan=0.0).to(dtype), torch.nan_to_num(v_pool.float(), nan=0.0).to(dtype)
    want = kernel_refs.attention(q, clean_k, clean_v, seq, pos, table, nh, nkv, hd, scale, window, keep_first=keep, sinks=sinks)
    make_plan = lambda: AttentionPlan(B, 1, max(lens), True, i32(starts), i32(news), i32(list(range(B + 1))), i32(lens), list(starts), list(news))
    args = (q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), seq.to(DEV), pos.to(DEV), table.to(DEV), nh, nkv, hd, scale, window)
    monkeypatch.setattr(attention_fast, "DECODE_BLOCKS", blocks)
    got = ops.attention(*args, plan=make_plan(), keep_first=keep, sinks=sinks.to(DEV))
    close(got, want, dtype)
    if blocks == 0:
        monkeypatch.setattr(attention_fast, "DECODE_SPECIAL", False)
        other = ops.attention(*args, plan=make_plan(), keep_first=keep, sinks=sinks.to(DEV))
        close(other, want, dtype)
        close(got, other.float(), dtype, tol16=1e-2)
        no_keep = ops.attention(*args, plan=make_plan(), sinks=sinks.to(DEV))
        assert float((no_keep.float().cpu() - want).abs().max()) > 1e-3


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
def test_whole_portions_and_decoding(tmp, which, dtype):
    model, cfg, w, _ = load_pair(tmp, which, dtype)
    tokens = tz.random_tokens(150, cfg["vocab"], 7)
    ref = pz.forward(cfg, w, tokens)
    whole = run_cuts(model, tokens, [150])
    assert_rows(whole, ref, dtype, "whole prompt")
    for cuts in ([100, 50], [64, 64, 2, 20], [63, 3, 2, 2, 70], [1, 2, 129, 5], [130], [2]):
        got = run_cuts(model, tokens, cuts)
        assert_rows(got, ref, dtype, f"cuts {cuts}")
        if dtype == torch.float32:
            assert rel_err(got, whole) < 1e-5, cuts


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["A", "B", "D"])
def test_unequal_batches_slots_and_pages_used_again(tmp, which, dtype):
    from dotllm_b200.engine import StepEntry
    model, cfg, w, _ = load_pair(tmp, which, dtype)
    lens = [1, 70, 23, 131]
    prompts = [tz.random_tokens(n + 12, cfg["vocab"], 20 + n) for n in lens]
    refs = [pz.forward(cfg, w, p) for p in prompts]
    cache = model.new_cache(64 * 8)
    for round_ in range(2):                                          # the second time every slot, state and page has been used before
        cache.fill_free_pages(float("nan"))
        seqs = [cache.open_sequence() for _ in prompts]
        order = list(range(len(prompts))) if round_ == 0 else [2, 0, 3, 1]
        out = model.step(cache, [StepEntry(seqs[i], prompts[i][:lens[i]], [0, lens[i] - 1]) for i in order])
        want = torch.cat([refs[i][[0, lens[i] - 1]] for i in order])
        assert_rows(out, want, dtype, "a batch of unequal prompts")
        live = list(order)
        for t in range(12):
            if t == 5:
                gone = live.pop(1)                                   # a request ends early; its slot and pages go back ...
                cache.close_sequence(seqs[gone])
                cache.fill_free_pages(float("nan"))
            out = model.step(cache, [StepEntry(seqs[i], [prompts[i][lens[i] + t]]) for i in live])
            assert_rows(out, torch.stack([refs[i][lens[i] + t] for i in live]), dtype, f"decoding together, step {t}")
        for i in live:
            cache.close_sequence(seqs[i])
        cache.check()
    assert not cache.live


@pytest.mark.parametrize("dtype", DTYPES)
def test_layers_at_a_real_models_widths(tmp, dtype):
    """Width 1,024, heads and latents of 128 channels, experts of 512: the sizes at which the bfloat16 run takes the
    tensor-core kernels and the sorted experts."""
    model, cfg, w, _ = load_pair(tmp, "wide", dtype)
    tokens = tz.random_tokens(330, cfg["vocab"], 11)
    ref = pz.forward(cfg, w, tokens)
    assert_rows(run_cuts(model, tokens, [300]), ref, dtype, "a prompt of 300 tokens and 30 decoded", loose=2.0)
    assert_rows(run_cuts(model, tokens[:200], [130, 70]), ref[:200], dtype, "two portions", loose=2.0)


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Configurations that nobody chose (`tiny_zemezen.random_config`): a prompt and twenty decoded tokens, then a batch of
    three unequal prompts (one of a single token) decoded together, eager and through captured steps, in both dtypes."""
    from dotllm_b200 import Model
    from dotllm_b200.engine import StepEntry
    rng = random.Random(100 + seed)
    cfg_dict = tz.random_config(rng)
    n = rng.randrange(140, 330)
    lens = [1, rng.randrange(2, 80), rng.randrange(80, 200)]
    for dtype in DTYPES:
        folder = tz.make_folder(tmp_path, f"random{seed}", dtype=dtype, cfg=cfg_dict)
        cfg, w = tz.read_folder(folder)
        model = Model.load(folder, dtype=dtype)
        tokens = tz.random_tokens(n, cfg["vocab"], seed)
        prompts = [tz.random_tokens(L + 8, cfg["vocab"], seed * 7 + L) for L in lens]
        ref, refs = pz.forward(cfg, w, tokens), [pz.forward(cfg, w, p) for p in prompts]
        got = [run_cuts(model, tokens, [n - 20])]
        want = [ref]
        cache = model.new_cache(64 * 12)
        cache.fill_free_pages(float("nan"))
        seqs = [cache.open_sequence() for _ in prompts]
        got.append(model.step(cache, [StepEntry(q, p[:L], [L - 1]) for q, p, L in zip(seqs, prompts, lens)]).clone())
        want.append(torch.stack([r[L - 1] for r, L in zip(refs, lens)]))
        for t in range(8):
            got.append(model.step(cache, [StepEntry(q, [p[L + t]]) for q, p, L in zip(seqs, prompts, lens)], graphs=t >= 4).clone())
            want.append(torch.stack([r[L + t] for r, L in zip(refs, lens)]))
        err = row_errors(torch.cat(got), torch.cat(want))
        assert torch.isfinite(err).all()
        if dtype == torch.float32:
            assert float(err.max()) <= REL[dtype], (seed, float(err.max()), cfg_dict)
        else:
            assert float(err.median()) <= REL[dtype] / 2 and float(err.max()) <= LOOSE and \
                int((err > REL[dtype]).sum()) <= max(1, int(0.03 * err.numel())), (seed, float(err.median()), float(err.max()), cfg_dict)


def test_keys_at_the_windows_edges_decide_whole_rows(tmp):
    """One attention layer whose scores are scaled until the softmax all but picks a single key.  The plain implementation
    must differ visibly when the window is one token longer or shorter, when one first token more or fewer is kept, and
    when the sink is taken away; the engine must agree with the right one: in a prompt that crosses pages, across a
    portion's start, and when decoding goes on over page borders while the window gives pages back."""
    dtype = torch.float32
    tokens = tz.random_tokens(330, 120, 3)
    for which in ("sharp", "soft"):
        model, cfg, w, _ = load_pair(tmp, which, dtype)
        ref = pz.forward(cfg, w, tokens)
        rms = ref.pow(2).mean(-1).sqrt()

        def changed(**mask):
            other = copy.deepcopy(cfg)
            other["layers"][0]["mixer"]["mask"].update(mask)
            return pz.forward(other, w, tokens)

        controls = [changed(size=22), changed(size=24), changed(keep_first=2), changed(keep_first=4)] if which == "sharp" else \
            [pz.forward(cfg, dict(w, **{"l0.mix.sink": w["l0.mix.sink"] - 30.0}), tokens)]       # with scores of order one the sink shows
        for wrong in controls:
            assert int(((wrong - ref).pow(2).mean(-1).sqrt() / rms > 1e-2).sum()) >= 20
        for cuts in ([330], [63, 1, 1, 200], [128, 64, 2], [290], [20]):
            got = run_cuts(model, tokens, cuts)
            assert rel_err(got, ref) < 1e-4, cuts
        bf = load_pair(tmp, which, torch.bfloat16)
        ref16 = pz.forward(bf[1], bf[2], tokens)
        for cuts in ([300], [100]):
            row_err = row_errors(run_cuts(bf[0], tokens, cuts), ref16)
            assert float(row_err.median()) < 4e-2 and int((row_err > 0.3).sum()) <= 6, (which, cuts, float(row_err.median()), int((row_err > 0.3).sum()))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_over_page_borders(tmp, dtype):
    model, cfg, w, _ = load_pair(tmp, "A", dtype)
    tokens = tz.random_tokens(330, cfg["vocab"], 5)
    ref = pz.forward(cfg, w, tokens)
    got = run_cuts(model, tokens, [30])                              # 300 tokens one by one, over five page borders
    assert_rows(got, ref, dtype, "300 decoded tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["A", "B"])
def test_greedy_generation_through_the_entry_point(tmp, which, dtype):
    from dotllm_b200 import InferenceOptions
    model, cfg, w, _ = load_pair(tmp, which, dtype)
    prompts = [tz.random_tokens(n, cfg["vocab"], 60 + n) for n in (1, 9, 40, 70)]
    n_new = 24
    outs = model.generate(prompts, InferenceOptions(temperature=0.0, max_tokens=n_new, stop_token_ids=[]))
    for p, o in zip(prompts, outs):
        assert o.finish_reason.value == "length" and o.generated_token_count == n_new
        ref = pz.forward(cfg, w, p + o.generated_token_ids)
        spread = float(ref.std())
        for i, tok in enumerate(o.generated_token_ids):              # teacher-forced: the plain arg-max, or within rounding of it
            row = ref[len(p) - 1 + i]
            assert int(row.argmax()) == tok or float(row.max() - row[tok]) <= (1e-4 if dtype == torch.float32 else 0.1) * spread, \
                (i, tok, int(row.argmax()))
    again = model.generate(prompts, InferenceOptions(temperature=0.0, max_tokens=n_new, stop_token_ids=[]))      # through captured steps now
    alone = model.generate(prompts[2], InferenceOptions(temperature=0.0, max_tokens=n_new, stop_token_ids=[]))
    if dtype == torch.float32:
        assert [o.generated_token_ids for o in again] == [o.generated_token_ids for o in outs]
        assert alone.generated_token_ids == outs[2].generated_token_ids


def test_decode_steps_replayed_from_graphs(tmp):
    """Steps captured as graphs (exact batch size and the shared widths with idle rows) give the eager steps' logits."""
    from dotllm_b200.engine import StepEntry
    dtype = torch.float32
    model, cfg, w, _ = load_pair(tmp, "A", dtype)
    prompts = [tz.random_tokens(n + 10, cfg["vocab"], 80 + n) for n in (5, 66, 30)]
    refs = [pz.forward(cfg, w, p) for p in prompts]
    for graphs in (True, "lazy"):
        cache = model.new_cache(64 * 6)
        seqs = [cache.open_sequence() for _ in prompts]
        model.step(cache, [StepEntry(s, p[:-10], []) for s, p in zip(seqs, prompts)])
        for t in range(10):
            out = model.step(cache, [StepEntry(s, [p[len(p) - 10 + t]]) for s, p in zip(seqs, prompts)], graphs=graphs)
            assert_rows(out, torch.stack([r[len(r) - 10 + t] for r in refs]), dtype, f"graphs={graphs} step {t}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program_on_a_zemezen_folder(tmp_path, dtype):
    tdtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    folder = tz.make_folder(tmp_path, "D", seed=2, dtype=tdtype)
    cfg, w = tz.read_folder(folder)
    a, b = tz.random_tokens(90, cfg["vocab"], 1), tz.random_tokens(30, cfg["vocab"], 2)
    ra, rb = pz.forward(cfg, w, a), pz.forward(cfg, w, b)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:80], "want": [0, 79]}, {"id": "b", "tokens": b[:20], "want": []}], "end": []}]
    for t in range(10):
        steps.append({"step": t + 1, "entries": [{"id": "a", "tokens": [a[80 + t]], "want": [0]},
                                                 {"id": "b", "tokens": [b[20 + t]], "want": [0] if t % 2 else []}],
                      "end": ["a", "b"] if t == 9 else []})
    out_dir = tmp_path / "out"
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out_dir),
                           "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [x for s in steps for x in ("done", str(s["step"]))]
    read = lambda n: torch.from_numpy(np.fromfile(out_dir / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"]).copy())
    assert_rows(read(0), ra[[0, 79]], tdtype, "prompt step")
    for t in range(10):
        want = [ra[80 + t]] + ([rb[20 + t]] if t % 2 else [])
        assert_rows(read(t + 1), torch.stack(want), tdtype, f"decode step {t}")


def test_command_line_makes_and_runs_a_zemezen_folder(tmp_path):
    """`random` writes a folder from a configuration file, `run` generates from it: greedy tokens are the plain
    implementation's, a seeded sampled request gives the same tokens twice."""
    import sys
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(tz.CONFIGS["C"]))
    folder = tmp_path / "model"
    made = subprocess.run([sys.executable, "-m", "dotllm_b200", "random", str(cfg_path), str(folder), "--seed", "3", "--dtype", "float32"],
                          cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert made.returncode == 0, made.stderr[-2000:]
    cfg, w = tz.read_folder(folder)
    prompt = tz.random_tokens(11, cfg["vocab"], 9)
    run = lambda *extra: subprocess.run([sys.executable, "-m", "dotllm_b200", "run", str(folder), "-p", ",".join(map(str, prompt)),
                                         "-n", "6", "--dtype", "float32", "--json", *extra], cwd=ROOT, capture_output=True, text=True,
                                        timeout=600)
    proc = run("-t", "0", "--stop-ids", "")
    assert proc.returncode == 0, proc.stderr[-2000:]
    tokens = json.loads(proc.stdout)["results"][0]["generated_token_ids"]
    ref = pz.forward(cfg, w, prompt + tokens)
    assert tokens == [int(ref[len(prompt) - 1 + i].argmax()) for i in range(6)]
    a, b = run("-t", "0.9", "--top-k", "30", "-s", "5"), run("-t", "0.9", "--top-k", "30", "-s", "5")
    assert a.returncode == 0 and json.loads(a.stdout)["results"][0]["generated_token_ids"] == \
        json.loads(b.stdout)["results"][0]["generated_token_ids"]
