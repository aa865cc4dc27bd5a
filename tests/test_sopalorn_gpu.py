"""Sopalorn on the GPU against the plain implementation: each new kernel alone, whole prompts, portions, token-by-token
decoding, unequal batches, slots, states and pages that are used again, keys just inside and just outside the window, far
keys, the first tokens, long decoding over page borders, generation through the entry point, the replay program, the
command line."""
import copy
import json
import os
import random
import subprocess

import numpy as np
import pytest
import torch

import kernel_refs
import tiny_sopalorn as ts
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
    return tmp_path_factory.mktemp("sopalorn")


_loaded = {}


def load_pair(tmp, which, dtype, seed=0, change=None, tag=""):
    from dotllm_b200 import Model
    key = (which, dtype, seed, tag)
    if key not in _loaded:
        folder = ts.make_folder(tmp / tag if tag else tmp, which, seed=seed, dtype=dtype)
        if change is not None:
            ts.rewrite(folder, change)
        cfg, weights = ts.read_folder(folder)
        _loaded[key] = (Model.load(folder, dtype=dtype), cfg, weights, folder)
    return _loaded[key]


def g32(*shape, seed=0, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float32) * scale).to(DEV)


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


# ------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("S,H,kind", [(1, 52, "layernorm"), (2, 264, "layernorm"), (3, 96, "rmsnorm"), (4, 1000, "layernorm"),
                                      (8, 40, "layernorm"), (2, 5000, "rmsnorm")])
def test_stream_of_copies_write_read_and_norm_alone(S, H, kind, dtype):
    T = 7
    x = g32(T, S * H, seed=1, scale=3.0) + 5.0                    # a mean far from zero: the variance must come from the deviations
    y = g32(T, H, seed=2).to(dtype)
    scale, mix, out, read = g32(H, seed=3), g32(S, S, seed=4), g32(S, seed=5), g32(S, seed=6)
    gain, bias = g32(H, seed=7), (g32(H, seed=8) if kind == "layernorm" else None)
    for write in (None, ops.StreamWrite(y, scale, mix, out), ops.StreamWrite(y, None, mix, out)):
        for rd in (read, None):
            xa, xb = x.clone(), x.clone().cpu()
            wb = None if write is None else kernel_refs.StreamWrite(write.data.cpu(), None if write.scale is None else write.scale.cpu(),
                                                                    mix.cpu(), out.cpu())
            got, u = ops.stream_norm(xa, S, write, rd, gain, bias, 1e-5, dtype, kind=kind, summed=True)
            want, wu = kernel_refs.stream_norm(xb, S, wb, None if rd is None else rd.cpu(), gain.cpu(), None if bias is None else bias.cpu(),
                                               1e-5, dtype, kind=kind, summed=True)
            close(got, want, dtype)
            close(u, wu, torch.float32)
            close(xa, xb, torch.float32)
    copies = ops.stream_copies(x[:, :H].contiguous(), S, 0.7)
    assert torch.equal(copies.cpu(), kernel_refs.stream_copies(x[:, :H].cpu(), S, 0.7))
    table, ids = g32(11, H + 4, seed=9).to(dtype)[:, :H], torch.tensor([3, 0, 10, 3], dtype=torch.int32, device=DEV)
    assert torch.equal(ops.embed_copies(table, ids, S, 0.7).cpu(), kernel_refs.embed_copies(table.cpu(), ids.cpu(), S, 0.7))


@pytest.mark.parametrize("dtype", DTYPES)
def test_norms_over_groups_of_columns_and_pairs_of_branches_alone(dtype):
    for wa, wb in ((320, 160), (30, 14), (4096, 1024), (48, 0)):
        x = g32(9, wa + wb + 8, seed=wa).to(dtype)
        gain = g32(wa + wb, seed=1)
        got = ops.group_rmsnorm(x[:, :wa + wb], gain, wa, wb, 1e-6)
        close(got, kernel_refs.group_rmsnorm(x[:, :wa + wb].cpu(), gain.cpu(), wa, wb, 1e-6), dtype)
    for H in (52, 256, 1000):
        a, b, ga, gb = g32(5, H, seed=1, scale=4.0), g32(5, H, seed=2, scale=0.01), g32(H, seed=3), g32(H, seed=4)
        close(ops.pair_norm_sum(a, b, ga, gb, 1e-6, 0.5, 0.5), kernel_refs.pair_norm_sum(a.cpu(), b.cpu(), ga.cpu(), gb.cpu(), 1e-6),
              torch.float32)
    v = g32(3, 77, seed=9)
    assert torch.equal(ops.scale_values(v.clone(), 0.3).cpu(), v.cpu() * 0.3)
    # a norm over all heads' outputs at once is one head as wide as all: widths on both sides of the kernel's wide form
    for H, vdim in ((1, 1024), (1, 4096), (1, 1000), (1, 520), (2, 2048), (1, 8192)):
        o, g, gain = g32(6, H * vdim, seed=5, scale=3.0), g32(6, H * vdim + 8, seed=6).to(dtype)[:, :H * vdim], g32(vdim, seed=7)
        for gate in ("sigmoid", "silu"):
            close(ops.head_norm_gate(o, g, gain, H, vdim, 1e-6, dtype, gate=gate),
                  kernel_refs.head_norm_gate(o.cpu(), g.cpu(), gain.cpu(), H, vdim, 1e-6, dtype, gate=gate), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dim,vdim", [(7, 40, 48), (3, 16, 24), (5, 6, 9), (2, 64, 64), (8, 128, 128), (1, 200, 40)])
def test_linear_attention_with_constant_decays_alone(H, dim, vdim, dtype):
    """Unequal prompts, then portions and single tokens from the states they left, in slots that are not neighbours."""
    lens = [1, 37, 70]
    T = sum(lens)
    width = 2 * H * dim + H * vdim
    decay = torch.tensor([0.3, 0.9, 0.999, 1.0, 0.6, 0.97, 0.5, 0.99][:H], dtype=torch.float32, device=DEV)
    state = torch.zeros((6, H, dim, vdim), dtype=torch.float32, device=DEV)
    ref_state = state.cpu().clone()
    slots = torch.tensor([4, 0, 2], dtype=torch.int32, device=DEV)
    for round_, sizes in enumerate((lens, [5, 1, 2], [1, 1, 1])):
        n = sum(sizes)
        proj = g32(n, width + 8, seed=10 + round_).to(dtype)
        q, k, v = proj[:, :H * dim], proj[:, H * dim:2 * H * dim], proj[:, 2 * H * dim:width]
        cu = torch.tensor([0] + list(np.cumsum(sizes)), dtype=torch.int32, device=DEV)
        got = ops.gla_scan(q, k, v, None, decay, cu, slots, state, H, dim, vdim, 1.0)
        want = kernel_refs.gla_scan(q.cpu(), k.cpu(), v.cpu(), None, decay.cpu(), cu.cpu(), slots.cpu(), ref_state, H, dim, vdim, 1.0)
        close(got, want, dtype, tol16=2e-5)                         # the inputs are the same bfloat16 numbers: float32 from there on
        close(state, ref_state, dtype, tol16=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dim,vdim,K", [(4, 2, 40, 48, 4), (4, 2, 24, 20, 3), (3, 3, 10, 7, 1), (6, 2, 16, 24, 5), (2, 1, 128, 128, 4)])
def test_delta_rule_with_a_decay_per_head_alone(H, G, dim, vdim, K, dtype):
    C = 2 * G * dim + H * vdim
    taps = g32(C, K, seed=1, scale=0.5).to(dtype)
    dt, a_log = g32(H, seed=2), g32(H, seed=3, scale=0.5)
    memory = torch.zeros((5, H * dim * vdim + (K - 1) * C), dtype=torch.float32, device=DEV)
    ref_memory = memory.cpu().clone()
    slots = torch.tensor([3, 1], dtype=torch.int32, device=DEV)
    for round_, sizes in enumerate(([40, 3], [2, 70], [1, 1])):
        n = sum(sizes)
        x = g32(n, C + 16, seed=20 + round_).to(dtype)
        b = g32(n, H, seed=30 + round_).to(dtype)
        z = g32(n, 8, seed=40 + round_)[:, :H]                     # a column view, as the mixer's padded product gives it
        cu = torch.tensor([0] + list(np.cumsum(sizes)), dtype=torch.int32, device=DEV)
        seq = torch.repeat_interleave(torch.arange(len(sizes)), torch.tensor(sizes)).to(torch.int32).to(DEV)
        got = ops.delta_rule(x, taps, b, z, dt, a_log, seq, cu, slots, memory, H, G, dim, vdim, dim ** -0.5, 1e-6, head_decay=True)
        want = kernel_refs.delta_rule(x.cpu(), taps.cpu(), b.cpu(), z.cpu(), dt.cpu(), a_log.cpu(), seq.cpu(), cu.cpu(), slots.cpu(), ref_memory,
                                      H, G, dim, vdim, dim ** -0.5, 1e-6, head_decay=True)
        close(got, want, dtype, tol16=5e-5)
        close(memory, ref_memory, dtype, tol16=5e-5)


def test_router_with_corrections_alone():
    """The choice goes by share + correction, the weights by the shares: a correction that lifts a poor expert above a good
    one must change the choice and leave the weights the shares'; ties go to the lower index."""
    dtype = torch.float32
    T, K, E, top = 50, 32, 11, 4
    x, w = g32(T, K, seed=1), g32(16, K, seed=2)                    # rows beyond E ride the product and are ignored
    corr = g32(E, seed=3, scale=0.2)
    for normalise, scale in ((True, 2.0), (False, 1.0), (True, 1.0)):
        ids, wts = ops.route_topk(x, w, None, top, scoring="softmax_all", experts=E, correction=corr, normalise=normalise, weight_scale=scale)
        rids, rw = kernel_refs.route_topk(x.cpu(), w.cpu(), None, top, scoring="softmax_all", experts=E, correction=corr.cpu(),
                                          normalise=normalise, weight_scale=scale)
        assert torch.equal(ids.cpu(), rids)
        close(wts, rw, dtype)
        if normalise:
            assert float((wts.sum(-1) - scale).abs().max()) < 1e-5
    plain_ids, _ = ops.route_topk(x, w, None, top, scoring="softmax_all", experts=E)
    assert not torch.equal(plain_ids, ids)                          # the correction decided somewhere
    big = torch.zeros(E, device=DEV)
    big[7] = 5.0                                                    # lifts expert 7 to the top everywhere, with its own small share as weight
    ids, wts = ops.route_topk(x, w, None, 1, scoring="softmax_all", experts=E, correction=big)
    share = torch.softmax(x @ w[:E].T, dim=-1)
    assert bool((ids == 7).all()) and float((wts[:, 0] - share[:, 7]).abs().max()) < 1e-6
    same = torch.zeros((3, K), device=DEV)                          # equal logits: equal shares, the lowest indices win
    ids, wts = ops.route_topk(same, w, None, 3, scoring="softmax_all", experts=E, correction=torch.zeros(E, device=DEV), normalise=True)
    assert ids.cpu().tolist() == [[0, 1, 2]] * 3


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [3, 70])
def test_identity_experts_alone(T, dtype):
    """Experts without matrices give back their input: row by row (few rows) and sorted by expert on the tensor cores (many)."""
    K, ff, E, n_id, top = 64, 32, 5, 3, 4
    x = g32(T, K, seed=1).to(dtype)
    wgu, wd = g32(E, 2 * ff, K, seed=2, scale=0.2).to(dtype), g32(E, K, ff, seed=3, scale=0.2).to(dtype)
    gen = torch.Generator().manual_seed(4)
    ids = torch.stack([torch.randperm(E + n_id, generator=gen)[:top] for _ in range(T)]).to(torch.int32).to(DEV)
    ids[0] = torch.tensor([E, E + 1, E + 2, 0])                     # a token that uses every identity expert
    wts = torch.rand((T, top), generator=gen).to(DEV)
    h = ops.expert_gate_up(x, ids, wgu, "silu")
    got = ops.expert_down(h, ids, wts, wd, identity=(x, n_id))
    rh = kernel_refs.expert_gate_up(x.cpu(), ids.cpu(), wgu.cpu(), "silu")
    want = kernel_refs.expert_down(rh, ids.cpu(), wts.cpu(), wd.cpu(), identity=(x.cpu(), n_id))
    close(got, want, dtype)
    none = kernel_refs.expert_down(rh, ids.cpu(), wts.cpu(), wd.cpu())
    assert float((want - none).abs().max()) > 0.1                   # the identity experts' share shows
    if ops.experts_grouped_takes(x, ids, wgu, wd):
        close(ops.experts_grouped(x, ids, wts, wgu, wd, "silu", identity=(x, n_id)), want, dtype)
    else:
        assert dtype == torch.float32 or T * top < ops.GROUPED_MIN_ROWS


# ------------------------------------------------------------------ the model
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["A", "B", "C", "D", "E"])
def test_whole_portions_and_decoding(tmp, which, dtype):
    model, cfg, w, _ = load_pair(tmp, which, dtype)
    tokens = ts.random_tokens(150, cfg["vocab"], 7)
    ref = ts.plain_logits(cfg, w, tokens)
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
    prompts = [ts.random_tokens(n + 12, cfg["vocab"], 20 + n) for n in lens]
    refs = [ts.plain_logits(cfg, w, p) for p in prompts]
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
    """Width 1,024, heads of 128 channels, experts of 512: the sizes at which the bfloat16 run takes the tensor-core kernels
    and the sorted experts."""
    model, cfg, w, _ = load_pair(tmp, "wide", dtype)
    tokens = ts.random_tokens(230, cfg["vocab"], 11)
    ref = ts.plain_logits(cfg, w, tokens)
    assert_rows(run_cuts(model, tokens, [200]), ref, dtype, "a prompt of 200 tokens and 30 decoded", loose=2.0)
    assert_rows(run_cuts(model, tokens[:200], [130, 70]), ref[:200], dtype, "two portions", loose=2.0)


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Configurations that nobody chose (`tiny_sopalorn.random_config`): a prompt and twenty decoded tokens, then a batch of
    three unequal prompts (one of a single token) decoded together, eager and through captured steps, in both dtypes."""
    from dotllm_b200 import Model
    from dotllm_b200.engine import StepEntry
    rng = random.Random(300 + seed)
    cfg_dict = ts.random_config(rng)
    n = rng.randrange(100, 200)
    lens = [1, rng.randrange(2, 80), rng.randrange(80, 150)]
    for dtype in DTYPES:
        folder = ts.make_folder(tmp_path, f"random{seed}", dtype=dtype, cfg=cfg_dict)
        cfg, w = ts.read_folder(folder)
        model = Model.load(folder, dtype=dtype)
        tokens = ts.random_tokens(n, cfg["vocab"], seed)
        prompts = [ts.random_tokens(L + 8, cfg["vocab"], seed * 7 + L) for L in lens]
        ref, refs = ts.plain_logits(cfg, w, tokens), [ts.plain_logits(cfg, w, p) for p in prompts]
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


def _sharpen_window(tensors):
    # the attention's side outweighs the delta rule's and the embedding, and its sinks stay small beside the sharp scores
    tensors["l0.mix.left.q"] *= 4.0
    tensors["l0.mix.left.out"] *= 8.0
    tensors["l0.mix.right.out"] *= 0.25
    tensors["l0.ls1"] *= 8.0


def test_keys_at_the_windows_edges_decide_whole_rows(tmp):
    """One parallel layer whose attention's scores are scaled until the softmax all but picks a single key.  The plain
    implementation must differ visibly when the window is one token longer or shorter and when the sinks are taken away;
    the engine must agree with the right one: in a prompt that crosses pages, across a portion's start, and when decoding
    goes on over page borders while the window gives pages back."""
    dtype = torch.float32
    tokens = ts.random_tokens(330, 120, 3)
    model, cfg, w, _ = load_pair(tmp, "sharp_window", dtype, change=_sharpen_window, tag="sharp")
    ref = ts.plain_logits(cfg, w, tokens)
    rms = ref.pow(2).mean(-1).sqrt()

    def changed(size):
        other = copy.deepcopy(cfg)
        other["layers"][0]["mixer"]["left"]["mask"]["size"] = size
        return ts.plain_logits(other, w, tokens)

    controls = [changed(22), changed(24), ts.plain_logits(cfg, dict(w, **{"l0.mix.left.sink": w["l0.mix.left.sink"] + 12.0}), tokens)]
    for wrong in controls:
        assert int(((wrong - ref).pow(2).mean(-1).sqrt() / rms > 1e-2).sum()) >= 20
    for cuts in ([330], [63, 1, 1, 200], [128, 64, 2], [290], [20]):
        got = run_cuts(model, tokens, cuts)
        assert rel_err(got, ref) < 1e-4, cuts
    bf = load_pair(tmp, "sharp_window", torch.bfloat16, change=_sharpen_window, tag="sharp")
    ref16 = ts.plain_logits(bf[1], bf[2], tokens)
    for cuts in ([300], [100]):
        row_err = row_errors(run_cuts(bf[0], tokens, cuts), ref16)
        assert float(row_err.median()) < 4e-2 and int((row_err > 0.3).sum()) <= 6, (cuts, float(row_err.median()), int((row_err > 0.3).sum()))


def _sharpen_far(tensors):
    tensors["l0.mix.q.norm"] *= 2.0
    tensors["l0.mix.k.norm"] *= 2.0
    tensors["l0.mix.o"] *= 16.0
    tensors["l0.ls1"] *= 4.0


def _soften_far(tensors):
    tensors["l0.mix.q.norm"] *= 0.125
    tensors["l0.mix.o"] *= 16.0
    tensors["l0.ls1"] *= 4.0


def test_far_keys_rotation_and_the_added_one_decide_whole_rows(tmp):
    """One attention layer over every earlier key, sharpened the same way: dropping the keys beyond the last hundred, pairing
    the rotated channels the other way, leaving the frequencies unblended and leaving the one out of the denominator must
    each change many rows of the plain result; the engine agrees with the design over prompts, portions and decoding."""
    import plain_sopalorn as ps
    dtype = torch.float32
    tokens = ts.random_tokens(400, 120, 5)
    model, cfg, w, _ = load_pair(tmp, "sharp_far", dtype, change=_sharpen_far, tag="far")
    ref = ts.plain_logits(cfg, w, tokens)
    rms = ref.pow(2).mean(-1).sqrt()
    differs = lambda other: int(((other - ref).pow(2).mean(-1).sqrt() / rms > 1e-2).sum())
    no_scaling = copy.deepcopy(cfg)
    del no_scaling["layers"][0]["mixer"]["rot"]["scaling"]
    assert differs(ts.plain_logits(no_scaling, w, tokens)) >= 20
    saved = ps.softmax_attention, ps.rotate_interleaved
    try:
        ps.softmax_attention = lambda q, k, v, scale, window=None, sink=None: saved[0](q, k, v, scale, 100, sink)
        assert differs(ts.plain_logits(cfg, w, tokens)) >= 20       # without the far keys
        ps.softmax_attention = saved[0]

        def half_pairs(x, positions, rot):                          # channel i with i + dims/2 instead of 2i with 2i + 1
            dims = int(rot["dims"])
            order = list(range(0, dims, 2)) + list(range(1, dims, 2))
            back = np.argsort(order)
            y = x.copy()
            y[..., :dims] = saved[1](x[..., :dims][..., back], positions, rot)[..., order]
            return y
        ps.rotate_interleaved = half_pairs
        assert differs(ts.plain_logits(cfg, w, tokens)) >= 20
    finally:
        ps.softmax_attention, ps.rotate_interleaved = saved
    for cuts in ([400], [63, 1, 1, 200], [128, 64, 2], [350], [20]):
        assert rel_err(run_cuts(model, tokens, cuts), ref) < 1e-4, cuts
    # with scores of order one the added one takes a visible share of every row's softmax
    soft_model, soft_cfg, soft_w, _ = load_pair(tmp, "sharp_far", dtype, change=_soften_far, tag="soft")
    soft_ref = ts.plain_logits(soft_cfg, soft_w, tokens[:150])
    try:
        ps.softmax_attention = lambda q, k, v, scale, window=None, sink=None: saved[0](q, k, v, scale, window, None)
        without = ts.plain_logits(soft_cfg, soft_w, tokens[:150])
    finally:
        ps.softmax_attention = saved[0]
    # (where the keys are few: the first tokens of a sequence, whose sum of weights is of the order of the one)
    assert int(((without - soft_ref).pow(2).mean(-1).sqrt() / soft_ref.pow(2).mean(-1).sqrt() > 1e-2)[:12].sum()) >= 6
    for cuts in ([150], [70, 2], [3]):
        assert rel_err(run_cuts(soft_model, tokens[:150], cuts), soft_ref) < 1e-4, cuts
    bf = load_pair(tmp, "sharp_far", torch.bfloat16, change=_sharpen_far, tag="far")
    ref16 = ts.plain_logits(bf[1], bf[2], tokens)
    for cuts in ([380], [100]):
        row_err = row_errors(run_cuts(bf[0], tokens, cuts), ref16)
        assert float(row_err.median()) < 4e-2 and int((row_err > 0.3).sum()) <= 8, (cuts, float(row_err.median()), int((row_err > 0.3).sum()))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_over_page_borders(tmp, dtype):
    model, cfg, w, _ = load_pair(tmp, "A", dtype)
    tokens = ts.random_tokens(330, cfg["vocab"], 5)
    ref = ts.plain_logits(cfg, w, tokens)
    got = run_cuts(model, tokens, [30])                              # 300 tokens one by one, over five page borders
    assert_rows(got, ref, dtype, "300 decoded tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["A", "B"])
def test_greedy_generation_through_the_entry_point(tmp, which, dtype):
    from dotllm_b200 import InferenceOptions
    model, cfg, w, _ = load_pair(tmp, which, dtype)
    prompts = [ts.random_tokens(n, cfg["vocab"], 60 + n) for n in (1, 9, 40, 70)]
    n_new = 24
    outs = model.generate(prompts, InferenceOptions(temperature=0.0, max_tokens=n_new, stop_token_ids=[]))
    for p, o in zip(prompts, outs):
        assert o.finish_reason.value == "length" and o.generated_token_count == n_new
        ref = ts.plain_logits(cfg, w, p + o.generated_token_ids)
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
    prompts = [ts.random_tokens(n + 10, cfg["vocab"], 80 + n) for n in (5, 66, 30)]
    refs = [ts.plain_logits(cfg, w, p) for p in prompts]
    for graphs in (True, "lazy"):
        cache = model.new_cache(64 * 6)
        seqs = [cache.open_sequence() for _ in prompts]
        model.step(cache, [StepEntry(s, p[:-10], []) for s, p in zip(seqs, prompts)])
        for t in range(10):
            out = model.step(cache, [StepEntry(s, [p[len(p) - 10 + t]]) for s, p in zip(seqs, prompts)], graphs=graphs)
            assert_rows(out, torch.stack([r[len(r) - 10 + t] for r in refs]), dtype, f"graphs={graphs} step {t}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program_on_a_sopalorn_folder(tmp_path, dtype):
    tdtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    folder = ts.make_folder(tmp_path, "D", seed=2, dtype=tdtype)
    cfg, w = ts.read_folder(folder)
    a, b = ts.random_tokens(90, cfg["vocab"], 1), ts.random_tokens(30, cfg["vocab"], 2)
    ra, rb = ts.plain_logits(cfg, w, a), ts.plain_logits(cfg, w, b)
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


def test_command_line_makes_and_runs_a_sopalorn_folder(tmp_path):
    """`random` writes a folder from a configuration file, `run` generates from it: greedy tokens are the plain
    implementation's, a seeded sampled request gives the same tokens twice."""
    import sys
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(ts.CONFIGS["C"]))
    folder = tmp_path / "model"
    made = subprocess.run([sys.executable, "-m", "dotllm_b200", "random", str(cfg_path), str(folder), "--seed", "3", "--dtype", "float32"],
                          cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert made.returncode == 0, made.stderr[-2000:]
    cfg, w = ts.read_folder(folder)
    prompt = ts.random_tokens(11, cfg["vocab"], 9)
    run = lambda *extra: subprocess.run([sys.executable, "-m", "dotllm_b200", "run", str(folder), "-p", ",".join(map(str, prompt)),
                                         "-n", "6", "--dtype", "float32", "--json", *extra], cwd=ROOT, capture_output=True, text=True,
                                        timeout=600)
    proc = run("-t", "0", "--stop-ids", "")
    assert proc.returncode == 0, proc.stderr[-2000:]
    tokens = json.loads(proc.stdout)["results"][0]["generated_token_ids"]
    ref = ts.plain_logits(cfg, w, prompt + tokens)
    assert tokens == [int(ref[len(prompt) - 1 + i].argmax()) for i in range(6)]
    a, b = run("-t", "0.9", "--top-k", "30", "-s", "5"), run("-t", "0.9", "--top-k", "30", "-s", "5")
    assert a.returncode == 0 and json.loads(a.stdout)["results"][0]["generated_token_ids"] == \
        json.loads(b.stdout)["results"][0]["generated_token_ids"]
