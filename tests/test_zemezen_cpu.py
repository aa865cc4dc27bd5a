"""Zemezen without a GPU: configuration, model description, tensor names, the plain implementation's own
mechanisms, and the engine's host logic (steps, cache, schedule) with the plain kernel references."""
import copy
import json
import random

import pytest
import torch

import plain_zemezen as pz
import tiny_zemezen as tz
from dotllm_b200.config import build_spec, config_from_dict, load_config
from dotllm_b200.engine import StepEntry, run_step
from dotllm_b200.errors import ConfigError, WeightsError
from dotllm_b200.models.decoder import DecoderModel
from dotllm_b200.parts.base import Runtime
from dotllm_b200.weights import load_into

CPU = Runtime(torch.float32, torch.device("cpu"))


def test_configuration_reads_every_key_and_writes_it_back():
    for name in ("A", "B", "C", "D", "wide", "sharp"):
        cfg = config_from_dict(copy.deepcopy(tz.CONFIGS[name]))
        assert cfg.to_dict() == tz.CONFIGS[name]
        assert type(cfg).__name__ == "ZemezenConfig"
    for broken, match in ((lambda c: c.pop("width"), "width"), (lambda c: c["layers"][0]["mixer"].pop("conv"), "conv"),
                          (lambda c: c["layers"][1].update(type="gla"), "type"),
                          (lambda c: c["layers"][4].update(weights_of=4), "weights_of"),
                          (lambda c: c["layers"][4].update(weights_of=5), "weights_of"),
                          (lambda c: c["layers"][4]["mixer"].update(dim=8), "differs"),
                          (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "groups"),
                          (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
                          (lambda c: c["layers"][2]["mixer"].update(vdim=8), "vdim"),
                          (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=26), "rot"),
                          (lambda c: c["layers"][2]["mixer"]["mask"].update(size=0), "mask"),
                          (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
                          (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind")):
        bad = copy.deepcopy(tz.CONFIGS["A"])
        broken(bad)
        with pytest.raises(ConfigError, match=match):
            config_from_dict(bad)


def test_sizes_beyond_the_delta_rules_kernels_are_refused_when_the_model_is_made():
    for layer in (tz.delta(2, 2, 16, 8, 65), tz.delta(1, 1, 520, 8, 2)):
        spec = build_spec(config_from_dict(tz.config(64, 100, 1e-5, [layer])))
        with pytest.raises(ConfigError, match="channel delta"):
            DecoderModel(spec, CPU)
    DecoderModel(build_spec(config_from_dict(tz.config(64, 100, 1e-5, [tz.delta(1, 1, 512, 8, 64)]))), CPU)


def test_description_schedule_tensor_names_and_cache_needs():
    spec = build_spec(config_from_dict(copy.deepcopy(tz.CONFIGS["A"])))
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3, 0, 2] and len(spec.layers) == 4
    assert all(e.cache_of is None for e in spec.schedule)          # every run keeps a cache or state of its own
    model = DecoderModel(spec, CPU)
    expected, optional = model.expected_weights()
    names = set(expected)
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.mix.q", "l0.mix.q.conv", "l0.mix.k.conv", "l0.mix.v.conv", "l0.mix.b",
            "l0.mix.A_log", "l0.mix.norm", "l0.mix.a1", "l0.mix.a2", "l0.mix.dt_bias", "l0.mix.g1", "l0.mix.g2", "l0.mix.o",
            "l0.mlp.gate", "l1.mix.q", "l1.mix.dkv", "l1.mix.dkv.norm", "l1.mix.uk", "l1.mix.uv", "l1.mlp.router", "l1.mlp.e5.down",
            "l2.mix.q", "l2.mix.k", "l2.mix.q.norm", "l2.mix.k.norm", "l2.mix.sink", "l2.mix.o", "l3.norm1"} <= names
    assert not any(n.startswith(("l4.", "l5.", "l3.mlp", "l2.mix.v")) or n.endswith(("norm2", "router.b")) for n in names)
    assert tuple(expected["l0.mix.q"].shape) == (2 * 24, 96) and tuple(expected["l0.mix.v"].shape) == (4 * 20, 96)
    assert tuple(expected["l0.mix.a2"].shape)[0] == 4 * 24 and tuple(expected["l0.mix.g2"].shape)[0] == 4 * 20
    assert tuple(expected["l0.mix.v.conv"].shape) == (80, 3) and tuple(expected["l2.mix.sink"].shape) == (6,)
    assert tuple(expected["l2.mix.o"].shape) == (96, 6 * 24) and tuple(expected["l1.mix.uv"].shape) == (3 * 24, 40)
    needs = model.cache_needs()
    assert [n.kind for n in needs] == ["state", "kv", "kv", "kv", "state", "kv"]
    assert needs[0].state_shape == (4 * 24 * 20 + 2 * (2 * 48 + 80),)          # the states, then two inputs of every channel
    assert (needs[1].n_kv_heads, needs[1].key_width(), needs[1].window) == (1, 40, None)
    assert (needs[2].window, needs[2].keep_first, needs[3].window, needs[3].keep_first) == (37, 3, 50, 0)
    cache = model.new_cache(256)
    state = [g for g in cache.groups if g.kind == "state"]
    assert len(state) == 1 and state[0].state.shape[0] == 2                       # both runs of layer 0, a state each
    windowed = [g for g in cache.groups if g.kind == "kv" and g.window == 37]
    assert len(windowed) == 1 and windowed[0].k.shape[0] == 2 and windowed[0].keep_first == 3


def test_ranks_that_only_the_tensors_give(tmp_path):
    folder = tz.make_folder(tmp_path, "D")
    cfg = json.loads((folder / "config.json").read_text())
    del cfg["layers"][0]["mixer"]["ranks"]                         # the stored factors are 4 and 9 wide, the defaults are not
    (folder / "config.json").write_text(json.dumps(cfg))
    model = load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder)
    assert (model.blocks[0].mixer.decay_rank, model.blocks[0].mixer.gate_rank) == (4, 9)
    cfg["layers"][0]["mixer"]["vdim"] = 12
    (folder / "config.json").write_text(json.dumps(cfg))
    with pytest.raises(WeightsError, match="wrong shapes"):
        load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder)


def test_kept_first_pages_stay_when_the_window_moves_on():
    from dotllm_b200.cache.model_cache import ModelCache
    from dotllm_b200.parts.base import CacheNeed
    needs = [CacheNeed("kv", n_kv_heads=1, head_dim=4, window=10, keep_first=70), CacheNeed("kv", n_kv_heads=1, head_dim=4, window=10)]
    cache = ModelCache(needs, [None, None], CPU, 64 * 12)
    seq = cache.open_sequence()
    for length in (60, 130, 300):
        cache.reserve([(seq, length)])
        cache.commit(seq, length)
    kept, plain = seq.pages[0], seq.pages[1]
    assert [p >= 0 for p in kept] == [True, True, False, False, True] and [p >= 0 for p in plain] == [False] * 4 + [True]
    cache.check()
    cache.close_sequence(seq)
    cache.check()
    assert all(g.pages.n_free == g.pages.count for g in cache.kv_groups)


# ------------------------------------------------------------------ the plain implementation's own mechanisms
def test_plain_delta_rule_alone():
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    q, k, v, dec, beta = r(30, 2, 6), r(30, 2, 6), r(30, 2, 5), torch.sigmoid(r(30, 2, 6)), torch.sigmoid(r(30, 2))
    whole, s_whole = pz.delta_recurrence(q, k, v, dec, beta)
    first, s = pz.delta_recurrence(q[:11], k[:11], v[:11], dec[:11], beta[:11])
    rest, s = pz.delta_recurrence(q[11:], k[11:], v[11:], dec[11:], beta[11:], s)
    assert torch.allclose(torch.cat([first, rest]), whole) and torch.allclose(s, s_whole)
    # the first token: the state is zero, so u = beta v and o = (q . k) beta v
    assert torch.allclose(whole[0], (q[0] * k[0]).sum(-1, keepdim=True) * beta[0][:, None] * v[0])
    # with beta 1, no decay and a unit key, the state returns the value just written along that key
    kk = pz.unit(k)
    o, S = pz.delta_recurrence(kk, kk, v, torch.ones_like(dec), torch.ones_like(beta))
    assert torch.allclose(o, v * (kk * kk).sum(-1, keepdim=True), atol=1e-5)
    # decays act on the rows of S that belong to key channels: a decay of zero in every channel but one forgets the rest
    only = torch.zeros_like(dec)
    only[:, :, 2] = 1.0
    _, S = pz.delta_recurrence(q[:5], k[:5], v[:5], only[:5], torch.zeros_like(beta[:5]), torch.ones(2, 6, 5, dtype=torch.float64))
    assert torch.equal(S[:, 2], torch.ones(2, 5, dtype=torch.float64)) and float(S[:, [0, 1, 3, 4, 5]].abs().max()) == 0.0


def test_plain_convolution_and_its_history():
    g = torch.Generator().manual_seed(1)
    x, taps = torch.randn(12, 3, generator=g, dtype=torch.float64), torch.randn(3, 4, generator=g, dtype=torch.float64)
    y = pz.short_convolution(x, taps)
    assert torch.allclose(y[0], taps[:, 3] * x[0])                  # the last column meets the current token, zeros before it
    assert torch.allclose(y[5], (taps.T * x[2:6]).sum(0))
    cut = pz.short_convolution(x[7:], taps, history=x[4:7])
    assert torch.allclose(cut, y[7:])
    assert torch.allclose(pz.short_convolution(x, taps[:, 3:]), taps[:, 3] * x)       # one tap: a scale per channel


def test_plain_window_sink_and_router():
    seen = pz.window_with_first(12, 4, 2)
    for i in range(12):
        assert [j for j in range(12) if seen[i, j]] == sorted(set(range(max(0, i - 3), i + 1)) | set(range(min(2, i + 1))))
    g = torch.Generator().manual_seed(2)
    q, k = torch.randn(9, 1, 4, generator=g, dtype=torch.float64), torch.randn(9, 1, 4, generator=g, dtype=torch.float64)
    v = torch.eye(9, dtype=torch.float64)[:, None, :]              # the output row is the attention weights themselves
    p = pz.masked_softmax_attention(q, k, v, 1.0, pz.window_with_first(9, 3, 1))[:, 0]
    sunk = pz.masked_softmax_attention(q, k, v, 1.0, pz.window_with_first(9, 3, 1), sink=torch.tensor([0.7], dtype=torch.float64))[:, 0]
    for i in range(9):
        assert abs(p[i].sum().item() - 1) < 1e-12 and sunk[i].sum().item() < 1 - 1e-3
        scores = (k[:, 0] @ q[i, 0])[pz.window_with_first(9, 3, 1)[i]]
        assert sunk[i].sum().item() == pytest.approx(float(torch.exp(scores).sum() / (torch.exp(scores).sum() + torch.exp(torch.tensor(0.7)))))
        assert torch.allclose(sunk[i] / sunk[i].sum(), p[i])
    # groups: experts 0-1, 2-3, 4-5; the two best groups by their best expert stay; scores are shares of the whole softmax
    w = {"r.router": torch.eye(6, dtype=torch.float64)}
    h = torch.tensor([[3.0, 0.0, 2.9, 2.8, 2.0, 2.95]], dtype=torch.float64)
    chosen, weight = pz.route(h, w, "r.", {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 2}})
    assert chosen.tolist() == [[0, 5, 4]]                          # group 1 (2.9, 2.8) loses to groups 0 (3.0) and 2 (2.95)
    assert torch.allclose(weight, torch.softmax(h, -1)[0, [0, 5, 4]][None]) and float(weight.sum()) < 1
    chosen, _ = pz.route(h, w, "r.", {"experts": 6, "top": 3})
    assert chosen.tolist() == [[0, 5, 2]]


def test_plain_rotation():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(5, 3, 12, generator=g, dtype=torch.float64)
    y = pz.rotate_half(x, list(range(5)), 8, 100.0)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])
    assert torch.allclose(y[..., :4] ** 2 + y[..., 4:8] ** 2, x[..., :4] ** 2 + x[..., 4:8] ** 2)
    q, k = x[:1, :1], x[1:2, :1]
    dot = lambda a, b: float((pz.rotate_half(q, [a], 8, 100.0) * pz.rotate_half(k, [b], 8, 100.0)).sum())
    assert dot(7, 3) == pytest.approx(dot(104, 100), rel=1e-9) and abs(dot(7, 3) - dot(7, 4)) > 1e-6


# ------------------------------------------------------------------ the engine's host logic
def load(tmp_path, which, cfg=None):
    folder = tz.make_folder(tmp_path, which, cfg=cfg)
    cfg, weights = tz.read_folder(folder)
    return load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder), cfg, weights


@pytest.mark.parametrize("which", ["A", "C", "D"])
def test_steps_cuts_and_batches_agree_with_the_plain_implementation(cpu_kernels, tmp_path, which):
    model, cfg, w = load(tmp_path, which)
    a, b = tz.random_tokens(83, cfg["vocab"], 1), tz.random_tokens(21, cfg["vocab"], 2)
    ra, rb = pz.forward(cfg, w, a).float(), pz.forward(cfg, w, b).float()
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
    sc = cache.open_sequence()                           # takes the slot, the state and the pages that a gave back
    out = run_step(model, cache, [StepEntry(sc, b, None)])
    assert torch.allclose(out[0], rb[-1], atol=2e-4)
    cache.check()


def test_configurations_drawn_at_random(cpu_kernels, tmp_path):
    rng = random.Random(11)
    for n in range(3):
        model, cfg, w = load(tmp_path, f"random{n}", cfg=tz.random_config(rng))
        a = tz.random_tokens(70, cfg["vocab"], n)
        ref = pz.forward(cfg, w, a).float()
        cache = model.new_cache(256)
        s = cache.open_sequence()
        out = [run_step(model, cache, [StepEntry(s, a[:61], [60])]), run_step(model, cache, [StepEntry(s, a[61:68], [6])])]
        out += [run_step(model, cache, [StepEntry(s, [t])]) for t in a[68:]]
        assert torch.allclose(torch.cat(out), ref[[60, 67, 68, 69]], atol=3e-4), cfg


def test_a_window_that_is_one_token_off_would_show(cpu_kernels, tmp_path):
    """One attention layer sharpened until single keys decide rows: the plain implementation with a window one token
    longer or shorter, or with one kept token more or fewer, differs visibly; with scores of order one, so does the one
    without the sink.  The engine agrees with the right one across a cut and through decoded tokens."""
    for sink, gains in ((20.0, 2.0), (2.0, 0.25)):
        folder = tz.sharp_folder(tmp_path, sink=sink, gains=gains)
        cfg, w = tz.read_folder(folder)
        model = load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder)
        tokens = tz.random_tokens(90, cfg["vocab"], 4)
        ref = pz.forward(cfg, w, tokens).float()
        rms = ref.pow(2).mean(-1).sqrt()

        def changed(**mask):
            other = copy.deepcopy(cfg)
            other["layers"][0]["mixer"]["mask"].update(mask)
            return pz.forward(other, w, tokens).float()

        controls = [changed(size=22), changed(size=24), changed(keep_first=2), changed(keep_first=4)] if gains > 1 else \
            [pz.forward(cfg, dict(w, **{"l0.mix.sink": w["l0.mix.sink"] - 30.0}), tokens).float()]
        for wrong in controls:
            assert int(((wrong - ref).pow(2).mean(-1).sqrt() / rms > 1e-2).sum()) >= 5
        cache = model.new_cache(256)
        s = cache.open_sequence()
        out = [run_step(model, cache, [StepEntry(s, tokens[:70], list(range(70)))])]
        out += [run_step(model, cache, [StepEntry(s, [t])]) for t in tokens[70:]]
        assert float(((torch.cat(out) - ref).pow(2).mean(-1).sqrt() / rms).max()) < 1e-4


def test_trace_replay_of_a_zemezen_folder(cpu_kernels, tmp_path):
    import io
    import numpy as np
    from dotllm_b200.engine.trace import TraceReplayer
    model, cfg, w = load(tmp_path, "C")

    class Wrapped:                                        # what the replayer needs of a Model
        def new_cache(self, n):
            return model.new_cache(n)

        def step(self, cache, entries):
            return run_step(model, cache, entries)

    a = tz.random_tokens(12, cfg["vocab"], 3)
    ref = pz.forward(cfg, w, a).float()
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
