"""Sopalorn without a GPU: configuration, model description, tensor names, cache needs of a layer that keeps two things,
the plain implementation's own mechanisms, and the engine's host logic (steps, cache, schedule) with the plain kernel
references."""
import copy
import json
import random

import numpy as np
import pytest
import torch

import plain_sopalorn as ps
import tiny_sopalorn as ts
from dotllm_b200.config import build_spec, config_from_dict, load_config
from dotllm_b200.engine import StepEntry, run_step
from dotllm_b200.errors import ConfigError
from dotllm_b200.models.decoder import DecoderModel
from dotllm_b200.parts.base import Runtime
from dotllm_b200.weights import load_into

CPU = Runtime(torch.float32, torch.device("cpu"))


def test_configuration_reads_every_key_and_writes_it_back():
    for name in ("A", "B", "C", "D", "E", "wide", "sharp_window", "sharp_far"):
        cfg = config_from_dict(copy.deepcopy(ts.CONFIGS[name]))
        assert cfg.to_dict() == ts.CONFIGS[name], name
        assert type(cfg).__name__ == "SopalornConfig"
    assert config_from_dict(copy.deepcopy(ts.CONFIGS["D"])).streams is None
    for broken, match in ((lambda c: c.pop("width"), "width"), (lambda c: c["layers"][1]["mixer"]["right"].pop("conv"), "conv"),
                          (lambda c: c["layers"][1].update(type="gla"), "type"),
                          (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
                          (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
                          (lambda c: c["layers"][3]["mixer"].update(dim=32), "differ"),
                          (lambda c: c["layers"][3]["mixer"]["rot"].update(base=7.0), "differ"),
                          (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "router"),
                          (lambda c: c["layers"][2]["mixer"].update(decay=[0.5, 0.9]), "decay"),
                          (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "rot"),
                          (lambda c: c["layers"][1]["mixer"]["left"]["mask"].update(size=0), "mask"),
                          (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "kv_heads"),
                          (lambda c: c["layers"][0]["mlp"].update(limit=-1.0), "limit"),
                          (lambda c: c.update(streams=0), "streams"),
                          (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind")):
        bad = copy.deepcopy(ts.CONFIGS["A"])
        broken(bad)
        with pytest.raises(ConfigError, match=match):
            config_from_dict(bad)


def test_description_schedule_tensor_names_and_cache_needs():
    spec = build_spec(config_from_dict(copy.deepcopy(ts.CONFIGS["A"])))
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3] and [e.cache_of for e in spec.schedule] == [None, None, None, 0]
    model = DecoderModel(spec, CPU)
    expected, _ = model.expected_weights()
    names = set(expected)
    assert {"embed", "head", "final.norm", "final.norm.b", "l0.norm1", "l0.norm1.b", "l0.norm2.b", "l0.ls1", "l0.ls2", "l0.hc1.in",
            "l0.hc1.out", "l0.hc1.mix", "l0.hc2.mix", "l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.o",
            "l0.mlp.gate", "l1.mix.left.q", "l1.mix.left.sink", "l1.mix.left.out", "l1.mix.right.out", "l1.mix.right.q.conv",
            "l1.mix.right.b", "l1.mix.right.a", "l1.mix.right.A_log", "l1.mix.right.dt_bias", "l1.mix.right.g", "l1.mix.right.norm",
            "l1.mlp.router", "l1.mlp.correction", "l1.mlp.e5.down", "l2.mix.norm", "l2.mix.g", "l3.mix.q", "l3.mix.q.norm"} <= names
    assert not any(n.startswith(("l3.mix.k", "l3.mix.v", "l2.mlp", "l2.norm2", "l2.ls2", "l2.hc2", "l1.mlp.e6", "l0.mix.sink")) for n in names)
    assert tuple(expected["l0.mix.q.norm"].shape) == (6 * 24,) and tuple(expected["l0.mix.k.norm"].shape) == (2 * 24,)
    assert tuple(expected["l0.mix.v"].shape) == (2 * 20, 96) and tuple(expected["l0.mix.o"].shape) == (96, 6 * 20)
    assert tuple(expected["l1.mlp.router"].shape) == (8, 96) and tuple(expected["l1.mlp.correction"].shape) == (8,)
    assert tuple(expected["l1.mix.right.a"].shape) == (4, 96) and tuple(expected["l1.mix.right.dt_bias"].shape) == (4,)
    assert tuple(expected["l1.hc2.mix"].shape) == (3, 3) and tuple(expected["l2.mix.norm"].shape) == (3 * 24,)
    needs = model.cache_needs()
    assert needs[0].kind == "kv" and (needs[0].key_width(), needs[0].value_width(), needs[0].window) == (24, 20, None)
    assert isinstance(needs[1], tuple) and [n.kind for n in needs[1]] == ["kv", "state"] and needs[1][0].window == 37
    assert needs[1][1].state_shape == (4 * 24 * 20 + 2 * (2 * 48 + 80),)          # the states, then two inputs of every channel
    assert needs[2].kind == "state" and needs[2].state_shape == (3, 16, 24)
    # without the key "streams": no weights of copies, one stream
    plain = DecoderModel(build_spec(config_from_dict(copy.deepcopy(ts.CONFIGS["D"]))), CPU)
    assert not any(".hc" in n for n in plain.expected_weights()[0]) and "l0.ls1" in plain.expected_weights()[0]


def test_a_layer_that_keeps_two_things_gets_two_views():
    from dotllm_b200.cache.model_cache import ModelCache
    from dotllm_b200.parts.base import CacheNeed
    kv, state = CacheNeed("kv", n_kv_heads=1, head_dim=4, window=10), CacheNeed("state", state_shape=(5,))
    needs = [(kv, state), CacheNeed("kv", n_kv_heads=1, head_dim=4, window=10), (kv, state), CacheNeed("state", state_shape=(5,)), None]
    cache = ModelCache(needs, [None, None, None, None, None], CPU, 64 * 6)
    assert len(cache.groups) == 2 and sorted(len(g.entries) for g in cache.groups) == [3, 3]
    seq = cache.open_sequence()
    cache.reserve([(seq, 70)])
    tables = {g.index: torch.zeros((1, 2), dtype=torch.int32) for g in cache.kv_groups}
    slots = torch.zeros(1, dtype=torch.int32)
    pair = cache.view(0, tables, slots)
    assert isinstance(pair, tuple) and [v.kind for v in pair] == ["kv", "state"] and all(v.writes for v in pair)
    other = cache.view(2, tables, slots)
    assert other[0].k.data_ptr() != pair[0].k.data_ptr() and other[1].state.data_ptr() != pair[1].state.data_ptr()
    assert cache.view(1, tables, slots).kind == "kv" and cache.view(3, tables, slots).kind == "state" and cache.view(4, tables, slots) is None
    cache.commit(seq, 70)
    cache.close_sequence(seq)
    cache.check()
    # an execution that reads a pair's storage gets both, and writes neither
    shared = ModelCache([(kv, state), (kv, state)], [None, 0], CPU, 64 * 2)
    got = shared.view(1, {g.index: torch.zeros((1, 1), dtype=torch.int32) for g in shared.kv_groups}, slots)
    assert [v.writes for v in got] == [False, False]


# ------------------------------------------------------------------ the plain implementation's own mechanisms
def test_plain_lightning_attention_alone():
    rng = np.random.default_rng(0)
    m = {"heads": 2, "dim": 3, "vdim": 4, "decay": [0.5, 1.0]}
    w = {"q": rng.normal(size=(6, 5)), "k": rng.normal(size=(6, 5)), "v": rng.normal(size=(8, 5)), "g": rng.normal(size=(8, 5)),
         "o": np.eye(8), "norm": np.ones(8)}
    h = rng.normal(size=(7, 5))
    y = ps.lightning_mixer(m, w, "", h, 1e-6)
    q, k, v = (ps.silu(h @ w[n].T) for n in "qkv")
    # closed form: o_t = sum_{j<=t} decay^(t-j) (q_t . k_j) v_j per head
    o = np.zeros((7, 2, 4))
    for t in range(7):
        for hh, d in enumerate(m["decay"]):
            for j in range(t + 1):
                o[t, hh] += d ** (t - j) * (q[t, 3 * hh:3 * hh + 3] @ k[j, 3 * hh:3 * hh + 3]) * v[j, 4 * hh:4 * hh + 4]
    want = ps.rms(o.reshape(7, 8), 1e-6) * ps.sigmoid(h @ w["g"].T)
    assert np.allclose(y, want)


def test_plain_delta_rule_convolution_and_router_alone():
    rng = np.random.default_rng(1)
    x, taps = rng.normal(size=(12, 3)), rng.normal(size=(3, 4))
    y = ps.short_convolution(x, taps)
    assert np.allclose(y[0], taps[:, 3] * x[0])                     # the last column meets the current token, zeros before it
    assert np.allclose(y[5], (taps.T * x[2:6]).sum(0))
    assert np.allclose(ps.short_convolution(x, taps[:, 3:]), taps[:, 3] * x)       # one tap: a scale per channel
    # the first token of a delta rule: the state is zero, so u = beta v and o = (q . k) beta v before the norm; with one
    # value channel the per-head norm leaves only the sign, times the gate
    m = {"heads": 2, "kv_heads": 1, "dim": 3, "vdim": 1, "conv": 1}
    w = {n: rng.normal(size=s) for n, s in (("q", (3, 5)), ("k", (3, 5)), ("v", (2, 5)), ("b", (2, 5)), ("a", (2, 5)), ("g", (2, 5)))}
    w.update({"q.conv": np.ones((3, 1)), "k.conv": np.ones((3, 1)), "v.conv": np.ones((2, 1)), "A_log": np.zeros(2), "dt_bias": np.zeros(2),
              "norm": np.ones(1), "o": np.eye(2)})
    h = rng.normal(size=(1, 5))
    out = ps.gated_delta_rule(m, w, "", h, 1e-12)
    q, k, v = ps.silu(h @ w["q"].T)[0], ps.silu(h @ w["k"].T)[0], ps.silu(h @ w["v"].T)[0]
    sign = np.sign((q @ k) * v)
    assert np.allclose(out[0], sign * ps.silu(h @ w["g"].T)[0], atol=1e-5)
    # router: shares of the softmax over all, the correction decides the choice only, weights normalised and scaled
    r = {"experts": 3, "identity": 2, "top": 2, "scale": 3.0}
    z = np.array([[2.0, 1.0, 0.0, 1.5, -1.0]])
    s = np.exp(z) / np.exp(z).sum()
    chosen, weights = ps.route(r, z, np.zeros(5))
    assert chosen.tolist() == [[0, 3]] and np.allclose(weights, s[0, [0, 3]] / s[0, [0, 3]].sum() * 3.0)
    chosen, weights = ps.route(r, z, np.array([0.0, 0.0, 10.0, 0.0, 0.0]))
    assert chosen.tolist() == [[2, 0]] and np.allclose(weights, s[0, [2, 0]] / s[0, [2, 0]].sum() * 3.0)
    # an identity expert gives back its input: with every choice an identity the feed-forward is scale * h
    mlp = {"expert": {"ff": 2}, "router": {"experts": 1, "identity": 2, "top": 2, "scale": 3.0}}
    ww = {"router": np.array([[0.0] * 4, [1.0] * 4, [2.0] * 4]), "correction": np.array([-10.0, 0.0, 0.0]), "e0.gate": np.ones((2, 4)),
          "e0.up": np.ones((2, 4)), "e0.down": np.ones((4, 2))}
    hh = np.abs(rng.normal(size=(3, 4)))
    assert np.allclose(ps.expert_feed_forward(mlp, ww, "", hh), 3.0 * hh)


def test_plain_rotation_and_frequencies_against_the_packages_tables():
    from dotllm_b200.parts.rotary import rotary_frequencies, rotary_magnitude
    rng = np.random.default_rng(3)
    rot = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    x = rng.normal(size=(5, 3, 12))
    y = ps.rotate_interleaved(x, list(range(5)), rot)
    f, grow = ps.rotary_frequencies(rot)
    assert np.array_equal(y[..., 8:], x[..., 8:]) and np.allclose(y[0], x[0] * np.r_[np.full(8, grow), np.ones(4)])
    assert np.allclose(y[..., 0:8:2] ** 2 + y[..., 1:8:2] ** 2, grow ** 2 * (x[..., 0:8:2] ** 2 + x[..., 1:8:2] ** 2))
    q, k = x[:1, :1], x[1:2, :1]
    dot = lambda a, b: float((ps.rotate_interleaved(q, [a], rot) * ps.rotate_interleaved(k, [b], rot)).sum())
    assert dot(7, 3) == pytest.approx(dot(104, 100), rel=1e-9) and abs(dot(7, 3) - dot(7, 4)) > 1e-6
    # the package's tables hold the same frequencies and the same factor on cos and sin
    scaling = {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64, "fast_turns": 8.0, "slow_turns": 1.0}
    assert np.allclose(rotary_frequencies(8, 100.0, scaling), f, rtol=1e-12) and rotary_magnitude(scaling) == pytest.approx(grow)
    plain = ps.rotary_frequencies({"dims": 8, "base": 100.0})[0]
    assert np.allclose(plain, 100.0 ** (-np.arange(4) / 4.0)) and not np.allclose(plain, f)


def test_plain_copies_of_the_stream():
    """One copy with unit weights is the plain residual sum; copies that only pass through leave the sum of the copies
    equal to copies x the single stream when nothing is written."""
    rng = np.random.default_rng(5)
    cfg = copy.deepcopy(ts.CONFIGS["D"])
    cfg["layers"] = cfg["layers"][:1]
    folder_w = {}
    spec = DecoderModel(build_spec(config_from_dict(copy.deepcopy(cfg))), CPU).expected_weights()[0]
    for name, s in spec.items():
        folder_w[name] = rng.normal(size=tuple(s.shape)) * 0.3
    tokens = [3, 9, 27, 81, 2]
    base = ps.forward(cfg, folder_w, tokens)[0]
    one = dict(cfg, streams=1)
    for which in (1, 2):
        folder_w[f"l0.hc{which}.in"], folder_w[f"l0.hc{which}.out"], folder_w[f"l0.hc{which}.mix"] = np.ones(1), np.ones(1), np.ones((1, 1))
    assert np.allclose(ps.forward(one, folder_w, tokens)[0], base)
    two = dict(cfg, streams=2)
    for which in (1, 2):                                            # read the first copy, write it back, never touch the second
        folder_w[f"l0.hc{which}.in"], folder_w[f"l0.hc{which}.out"] = np.array([1.0, 0.0]), np.array([1.0, 0.0])
        folder_w[f"l0.hc{which}.mix"] = np.eye(2)
    logits, after = ps.forward(two, folder_w, tokens)
    x0 = folder_w["embed"][tokens] * cfg["embedding"]["scale"]
    assert np.allclose(after[0], ps.forward(cfg, folder_w, tokens)[1][0] + x0)      # the untouched copy is still the embedding


# ------------------------------------------------------------------ the engine's host logic
def load(tmp_path, which, cfg=None, change=None):
    folder = ts.make_folder(tmp_path, which, cfg=cfg)
    if change is not None:
        ts.rewrite(folder, change)
    cfg, weights = ts.read_folder(folder)
    return load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder), cfg, weights


@pytest.mark.parametrize("which", ["A", "C", "D", "E"])
def test_steps_cuts_and_batches_agree_with_the_plain_implementation(cpu_kernels, tmp_path, which):
    model, cfg, w = load(tmp_path, which)
    a, b = ts.random_tokens(83, cfg["vocab"], 1), ts.random_tokens(21, cfg["vocab"], 2)
    ra, rb = ts.plain_logits(cfg, w, a).float(), ts.plain_logits(cfg, w, b).float()
    cache = model.new_cache(64 * 4)
    cache.fill_free_pages(float("nan"))
    sa, sb = cache.open_sequence(), cache.open_sequence()
    out = run_step(model, cache, [StepEntry(sa, a[:66], [0, 1, 65]), StepEntry(sb, b[:5], [4])])
    assert torch.allclose(out, torch.cat([ra[[0, 1, 65]], rb[[4]]]), atol=2e-4)
    out = run_step(model, cache, [StepEntry(sa, a[66:68], [0, 1]), StepEntry(sb, b[5:19], [13])])       # portions of 2 and 14
    assert torch.allclose(out, torch.cat([ra[[66, 67]], rb[[18]]]), atol=2e-4)
    for t in range(68, 83):
        entries = [StepEntry(sa, [a[t]])] + ([StepEntry(sb, [b[t - 49]])] if t - 49 < 21 else [])
        out = run_step(model, cache, entries)
        assert torch.allclose(out[0], ra[t], atol=2e-4)
        if len(entries) == 2:
            assert torch.allclose(out[1], rb[t - 49], atol=2e-4)
    cache.close_sequence(sa)
    cache.fill_free_pages(float("nan"))
    sc = cache.open_sequence()                           # takes the slot, the states and the pages that a gave back
    out = run_step(model, cache, [StepEntry(sc, b, None)])
    assert torch.allclose(out[0], rb[-1], atol=2e-4)
    cache.check()


def test_configurations_drawn_at_random(cpu_kernels, tmp_path):
    rng = random.Random(12)
    for n in range(3):
        model, cfg, w = load(tmp_path, f"random{n}", cfg=ts.random_config(rng))
        a = ts.random_tokens(70, cfg["vocab"], n)
        ref = ts.plain_logits(cfg, w, a).float()
        cache = model.new_cache(256)
        s = cache.open_sequence()
        out = [run_step(model, cache, [StepEntry(s, a[:61], [60])]), run_step(model, cache, [StepEntry(s, a[61:68], [6])])]
        out += [run_step(model, cache, [StepEntry(s, [t])]) for t in a[68:]]
        assert torch.allclose(torch.cat(out), ref[[60, 67, 68, 69]], atol=3e-4), cfg


def test_a_window_that_is_one_token_off_would_show(cpu_kernels, tmp_path):
    """One parallel layer whose attention is sharpened until single keys decide rows: the plain implementation with a window
    one token longer or shorter differs visibly, and so does the one with other sinks.  The engine agrees with the right
    one across a cut and through decoded tokens."""
    def sharpen(tensors):
        tensors["l0.mix.left.q"] *= 4.0
        tensors["l0.mix.left.out"] *= 8.0
        tensors["l0.mix.right.out"] *= 0.25
        tensors["l0.ls1"] *= 8.0
    model, cfg, w = load(tmp_path, "sharp_window", change=sharpen)
    tokens = ts.random_tokens(90, cfg["vocab"], 4)
    ref = ts.plain_logits(cfg, w, tokens).float()
    rms = ref.pow(2).mean(-1).sqrt()

    def changed(size):
        other = copy.deepcopy(cfg)
        other["layers"][0]["mixer"]["left"]["mask"]["size"] = size
        return ts.plain_logits(other, w, tokens).float()

    for wrong in (changed(22), changed(24), ts.plain_logits(cfg, dict(w, **{"l0.mix.left.sink": w["l0.mix.left.sink"] + 12.0}), tokens).float()):
        assert int(((wrong - ref).pow(2).mean(-1).sqrt() / rms > 1e-2).sum()) >= 5
    cache = model.new_cache(256)
    s = cache.open_sequence()
    out = [run_step(model, cache, [StepEntry(s, tokens[:70], list(range(70)))])]
    out += [run_step(model, cache, [StepEntry(s, [t])]) for t in tokens[70:]]
    assert float(((torch.cat(out) - ref).pow(2).mean(-1).sqrt() / rms).max()) < 1e-4


def test_trace_replay_of_a_sopalorn_folder(cpu_kernels, tmp_path):
    import io
    from dotllm_b200.engine.trace import TraceReplayer
    model, cfg, w = load(tmp_path, "C")

    class Wrapped:                                        # what the replayer needs of a Model
        def new_cache(self, n):
            return model.new_cache(n)

        def step(self, cache, entries):
            return run_step(model, cache, entries)

    a = ts.random_tokens(12, cfg["vocab"], 3)
    ref = ts.plain_logits(cfg, w, a).float()
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:9], "want": [0, 8]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[9:10], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": a[10:], "want": [1]}], "end": ["x"]}]
    out = io.StringIO()
    replayer = TraceReplayer(Wrapped(), 128, tmp_path / "out")
    replayer.check_kernels = lambda: None
    replayer.run([json.dumps(s) for s in steps], out)
    assert out.getvalue().split() == ["done", "0", "done", "1", "done", "2"]
    got0 = torch.from_numpy(np.fromfile(tmp_path / "out" / "0.f32", dtype="<f4").reshape(-1, cfg["vocab"]).copy())
    got2 = torch.from_numpy(np.fromfile(tmp_path / "out" / "2.f32", dtype="<f4").reshape(-1, cfg["vocab"]).copy())
    assert not (tmp_path / "out" / "1.f32").exists()
    assert torch.allclose(got0, ref[[0, 8]], atol=2e-4) and torch.allclose(got2, ref[[11]], atol=2e-4)
    assert not replayer.sequences and not replayer.cache.live
