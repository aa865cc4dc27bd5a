"""Decode and prefill throughput of the Llama-3.1-8B-shaped model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 8192] [--layers L]
                    [--dtype bfloat16|float32] [--shape 8b|1b|13b] [--repeats 5]
    python bench.py --shape 1b --workload unequal     # 64 prompts of 16..2048 tokens in one step, then 256 decode steps
    python bench.py --workload staggered              # Model.generate while 64 requests end one by one (also --shape 1b)
    python bench.py --workload short-prompts          # time to the first token of single short prompts, eager and captured
    python bench.py --workload kubedra [--shape 1b]   # the Kubedra design beside a Llama of equal width and depth, and its kernels
    python bench.py --workload komulorn [--shape 1b]  # the Komulorn design beside a Llama of equal width, heads and depth, and its kernels
    python bench.py --workload zemezen [--shape 1b]   # the Zemezen design beside a Kubedra of equal width and depth, and its kernels
    python bench.py --workload sopalorn [--shape 1b]  # the Sopalorn design beside a Zemezen of equal width and depth, and its kernels
    python bench.py --impl plain-cpu                  # the plain implementation under tests/, timed on the CPU

A "step" is one decode step: one new token for each of ``batch`` sequences that already hold
``context`` tokens.  ``value`` is decoded tokens per second, timed on the device with CUDA events
over K consecutive steps (every step reads all weights, far more than the L2 holds).  ``e2e`` is
the same through the public entry point with host token ids in and out every step.  The line also
carries a 2,048-token prefill, decode at batch 1 and 64, the decode step's HBM roofline, the share
of an eager step's kernel time per kernel family, and tokens per second of ``Model.generate`` itself
(the loop users call: prompts in, 256 new tokens each out, stop tokens off).  Every timed region is
repeated ``--repeats`` times; the best repetition is reported with the coefficient of variation over
all of them (the reference's protocol, benchmarks/DotLLM.Benchmarks/InferenceBenchmarks.cs:30).

The cache contents are random numbers written directly into the pages: a decode step's time does
not depend on the values it reads, and filling 64 x 8192 positions through the model would take
longer than the whole measurement.  Weights are random (seeded), token ids synthetic.

The reference (kkokosa/dotLLM) is a .NET 10 program that loads GGUF checkpoints; neither the SDK
nor a checkpoint can be had offline here, so ``--impl reference`` reports itself unavailable.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_31_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 131072,
    "hidden_act": "silu",
}
# The other two benchmark shapes of the same architecture (selected with --shape).
LLAMA_32_1B = dict(LLAMA_31_8B, num_hidden_layers=16, hidden_size=2048, num_attention_heads=32, num_key_value_heads=8,
                   head_dim=64, intermediate_size=8192, vocab_size=128256, tie_word_embeddings=True,
                   rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                 "original_max_position_embeddings": 8192})
LLAMA_2_13B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 40,
    "head_dim": 128, "intermediate_size": 13824, "vocab_size": 32000, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 4096, "hidden_act": "silu",
}
SHAPES = {"8b": ("Llama-3.1-8B-shaped", LLAMA_31_8B), "1b": ("Llama-3.2-1B-shaped", LLAMA_32_1B),
          "13b": ("Llama-2-13B-shaped", LLAMA_2_13B)}
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
FP32_TFLOPS_NOMINAL = 74.5      # 148 multiprocessors x 128 FMA a clock x 2 x 1.965 GHz: no measured float32 peak exists


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            data = json.load(open(path))
            return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]), "source": "measured"}
        except (OSError, ValueError, KeyError):
            pass
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples taken while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "plain-cpu"])
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--repeats", type=int, default=5, help="repetitions of every timed region (best and CV are reported)")
    ap.add_argument("--workload", default="steady", choices=["steady", "unequal", "staggered", "short-prompts", "kubedra", "komulorn", "zemezen", "sopalorn"],
                    help="unequal: 64 prompts of 16..2048 tokens in one prefill step, then 256 decode steps; "
                         "staggered: Model.generate on 64 prompts whose requests end five steps apart; "
                         "short-prompts: the time to the first token of single prompts of 20 to 1,024 tokens; "
                         "kubedra: prefill and decode of the Kubedra design at layer sizes of a real model beside a Llama of "
                         "equal width and depth, and each of its kernels against its roofline; "
                         "komulorn: the same for the Komulorn design beside a Llama of equal width, heads and depth; "
                         "zemezen: the same for the Zemezen design beside a Kubedra of equal width and depth; "
                         "sopalorn: the same for the Sopalorn design beside a Zemezen of equal width and depth")
    ap.add_argument("--no-generate", action="store_true", help="skip the Model.generate cells")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes: the 8B default, or 1b / 13b")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (0: all of them)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points and the prefill")
    ap.add_argument("--only-prefill", action="store_true", help="run only the 2,048-token prefill (for profiling)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="with --only-prefill: tokens of the one prompt (the line itself always reports 2,048)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference",
                          "unavailable": "kkokosa/dotLLM is a .NET 10 program reading GGUF checkpoints; no .NET SDK, "
                                         "no checkpoint and no network exist here, so it cannot be installed or run"}))
        return 0
    if args.impl == "plain-cpu":
        return plain_cpu_baseline()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU library: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from dotllm_b200 import InferenceOptions, Model, StepEntry
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.kernels import library, ops

    if args.workload == "kubedra":
        return kubedra_workload(args)
    if args.workload == "komulorn":
        return komulorn_workload(args)
    if args.workload == "zemezen":
        return zemezen_workload(args)
    if args.workload == "sopalorn":
        return sopalorn_workload(args)
    pk = peaks()
    shape_name, shape = SHAPES[args.shape]
    cfg_dict = dict(shape, num_hidden_layers=args.layers or shape["num_hidden_layers"])
    cfg = config_from_dict(cfg_dict)
    torch.cuda.set_device(0)
    t0 = time.time()
    model = Model.random(cfg, seed=0, dtype=args.dtype, device="cuda:0", on_device=True)
    esize = 2 if args.dtype == "bfloat16" else 4
    dtype_name = "bf16" if args.dtype == "bfloat16" else "fp32"
    compute_peak = pk["bf16_tflops"] if args.dtype == "bfloat16" else FP32_TFLOPS_NOMINAL
    torch.cuda.synchronize()
    print(f"[bench] model ready in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)

    steps, warmup, ctx = args.steps, args.warmup, args.context
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    reps = max(1, args.repeats)
    room = ctx + 2 * reps * steps + warmup + 128        # every timed step grows every sequence by one token
    # The cache must fit beside the weights: a batch whose sequences of `ctx` tokens would not fit
    # runs at the longest context that does (reported with its point).
    per_token = 2 * esize * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim
    free_bytes, _ = torch.cuda.mem_get_info()
    fit_tokens = int(0.85 * free_bytes) // per_token
    ctx_of = {b: min(ctx, max(256, fit_tokens // b - (room - ctx)) // 64 * 64) for b in batches}
    cache_tokens = max(b * ((ctx_of[b] + room - ctx + 63) // 64 * 64) for b in batches)
    cache = model.new_cache(max_tokens=cache_tokens, max_sequences=max(batches))
    for g in cache.kv_groups:                              # random cache contents (see the header)
        g.k.normal_(0.0, 0.5)
        g.v.normal_(0.0, 0.5)
    weight_bytes = model.decoder.weight_bytes_per_step()
    kv_bytes_per_token = cache.bytes_per_token()
    vocab = cfg.vocab_size
    gen = torch.Generator().manual_seed(1)

    # count this library's own kernel launches (the graph replays what was captured)
    launches = {"n": 0}
    real_call = library.call

    def counting_call(name, *a):
        launches["n"] += 1
        return real_call(name, *a)
    library.call = counting_call                           # every kernel module calls through library.call

    def spread(values):
        """Coefficient of variation of the repetitions (0 for a single one)."""
        return round(statistics.pstdev(values) / statistics.mean(values), 4) if len(values) > 1 else 0.0

    def decode_point(batch, measure_e2e):
        ctx = ctx_of[batch]
        seqs = [cache.open_sequence() for _ in range(batch)]
        cache.reserve([(s, ctx) for s in seqs])
        for s in seqs:
            cache.commit(s, ctx)
        tokens = torch.randint(0, vocab, (batch,), generator=gen).tolist()
        graphs = model.decode_graphs(cache)
        entries = [StepEntry(s, [t]) for s, t in zip(seqs, tokens)]
        launches["n"] = 0
        logits = graphs.run(entries)                         # captures; host tokens in
        per_replay = launches["n"] // 2                      # the eager run before capture + the capture itself
        tok_buf = graphs.token_buffer(batch)
        ops.sample(logits, out=tok_buf)
        for _ in range(warmup):
            ops.sample(graphs.run(entries, device_tokens=True), out=tok_buf)
        torch.cuda.synchronize()
        sampler = ClockSampler()
        times = []
        for _ in range(reps):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(steps):
                ops.sample(graphs.run(entries, device_tokens=True), out=tok_buf)
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) / steps)
        clocks = sampler.stop()
        ms = min(times)
        result = {"ms": ms, "tok_s": batch * 1000.0 / ms, "clocks": clocks, "launches": steps * (per_replay + 1),
                  "mean_len": sum(s.length for s in seqs) / batch, "cv": spread(times)}
        if measure_e2e:
            host_tokens = tok_buf.tolist()
            copied = graphs.captured[batch].h2d_bytes         # counted where the copies are issued
            e2e_times = []
            for _ in range(reps):
                torch.cuda.synchronize()
                t_a = time.perf_counter()
                for _ in range(steps):
                    lg = model.step(cache, [StepEntry(s, [t]) for s, t in zip(seqs, host_tokens)], graphs=True)
                    host_tokens = ops.sample(lg).tolist()        # device -> host read of the step's result
                torch.cuda.synchronize()
                e2e_times.append((time.perf_counter() - t_a) * 1e3 / steps)
            e2e_ms = min(e2e_times)
            result["e2e"] = {"value": batch * 1000.0 / e2e_ms, "unit": "tokens/s", "ms_per_step": e2e_ms,
                             "h2d_bytes_per_step": (graphs.captured[batch].h2d_bytes - copied) // (steps * reps),
                             "d2h_bytes_per_step": 4 * batch, "cv": spread(e2e_times)}
            result["shares"] = family_shares(seqs, host_tokens)
        for s in seqs:
            cache.close_sequence(s)
        return result

    FAMILIES = (("products", ("gemm", "swiglu")), ("attention", ("attention", "rope")),
                ("norm_embed_sample", ("rmsnorm", "gather", "sample", "penalty")))

    def family_shares(seqs, host_tokens):
        """One eager decode step with a CUDA event on either side of every kernel of this library: the
        share of the summed kernel time per family.  (Eager launches do not overlap as a replayed
        graph's do, so these are shares of kernel time, not of the step's wall time.)"""
        spans = []

        def timed_call(name, *a):
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            counting_call(name, *a)
            a1.record()
            spans.append((name, a0, a1))
        library.call = timed_call
        try:
            lg = model.step(cache, [StepEntry(s, [t]) for s, t in zip(seqs, host_tokens)])
            ops.sample(lg)
            torch.cuda.synchronize()
        finally:
            library.call = counting_call
        total = sum(a0.elapsed_time(a1) for _, a0, a1 in spans) or 1.0
        shares = {}
        for family, keys in FAMILIES:
            shares[family] = round(sum(a0.elapsed_time(a1) for n, a0, a1 in spans if any(k in n for k in keys)) / total, 3)
        shares["other"] = round(max(0.0, 1.0 - sum(shares.values())), 3)
        return shares

    def prefill_flops(T, rows_out):
        """The products the step runs: Q/K/V for every token in every layer; the output projection and
        the feed-forward for every token in all layers but the last, which runs them (and the head) for
        the ``rows_out`` rows whose logits are wanted only."""
        qkv = 2 * cfg.hidden_size * (cfg.q_dim + 2 * cfg.kv_dim)
        rest = 2 * (cfg.q_dim * cfg.hidden_size + 3 * cfg.hidden_size * cfg.intermediate_size)
        L = cfg.num_hidden_layers
        return T * (L * qkv + (L - 1) * rest) + rows_out * (rest + 2 * cfg.hidden_size * vocab)

    def prefill_point(tokens=PREFILL_TOKENS):
        """One prompt of ``tokens`` tokens through model.step: best of ``reps`` after three warm-ups
        (the first is eager, the second captures the step's graph, the rest replay it)."""
        import numpy as np
        prompt = np.asarray(torch.randint(0, vocab, (tokens,), generator=gen))
        times = []
        for it in range(3 + reps):
            s = cache.open_sequence()
            torch.cuda.synchronize()
            a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            model.step(cache, [StepEntry(s, prompt)], graphs=True)       # the step's shape repeats: replayed from its graph
            b_.record()
            torch.cuda.synchronize()
            if it >= 3:
                times.append(a.elapsed_time(b_))
            cache.close_sequence(s)
        p_ms = min(times)
        T = tokens
        flops = prefill_flops(T, 1) + cfg.num_hidden_layers * 2 * T * T * cfg.q_dim
        return {"value": round(T * 1000.0 / p_ms, 1), "tokens": T, "ms": round(p_ms, 3),
                "frac": round(flops / (p_ms * 1e-3) / (compute_peak * 1e12), 4),
                "peak": pk["source"] if args.dtype == "bfloat16" else "nominal fp32", "cv": spread(times)}

    def generate_point(batch, prompt_len=128, new_tokens=256, sampled=False):
        """Tokens per second of Model.generate itself: host prompts in, host tokens out, stop tokens off.
        ``sampled``: temperature 0.8, top-k 40, top-p 0.95 and a seed instead of greedy."""
        prompts = [torch.randint(0, vocab, (prompt_len,), generator=gen).tolist() for _ in range(batch)]
        need = batch * ((prompt_len + new_tokens + 63) // 64 * 64)
        if need > cache.max_tokens:
            return None
        generator = model.generator(cache=cache, max_batch=batch)
        if sampled:
            options = InferenceOptions(temperature=0.8, top_k=40, top_p=0.95, seed=7, max_tokens=new_tokens, stop_token_ids=[])
        else:
            options = InferenceOptions(temperature=0.0, max_tokens=new_tokens, stop_token_ids=[])
        generator.generate(prompts[:batch], options)          # warm-up: captures the graph of this batch size
        times = []
        for _ in range(min(reps, 3)):
            torch.cuda.synchronize()
            t_a = time.perf_counter()
            out = generator.generate(prompts, options)
            torch.cuda.synchronize()
            times.append(time.perf_counter() - t_a)
        assert all(o.generated_token_count == new_tokens for o in out)
        t = out[0].timings
        return {"value": round(batch * new_tokens / min(times), 1), "prompt_tokens": prompt_len, "new_tokens": new_tokens,
                "decode_tok_s": round(batch * t.decode_steps / (t.decode_ms / 1e3), 1), "prefill_ms": round(t.prefill_ms, 2),
                "sampling_ms": round(t.sampling_ms, 2), "cv": spread(times)}

    if args.workload == "short-prompts":
        return short_prompt_workload(args, model, cfg, gen, shape_name, dtype_name)
    if args.workload == "staggered":
        return staggered_workload(args, model, cfg, gen, shape_name, dtype_name)
    if args.workload == "unequal":
        return unequal_workload(args, model, cache, cfg, gen, pk, shape_name, dtype_name, compute_peak, weight_bytes, prefill_flops)

    if args.only_prefill:
        print(json.dumps({"prefill": prefill_point(args.prefill_tokens), "layers": cfg.num_hidden_layers}))
        return 0

    main_point = decode_point(args.batch, True)
    points = {}
    prefill = None
    generate = {}
    if not args.no_points:
        for b in batches:
            if b != args.batch:
                name = f"decode_b{b}" if ctx_of[b] == ctx else f"decode_b{b}_ctx{ctx_of[b]}"
                points[name] = round(decode_point(b, False)["tok_s"], 1)
        points[f"decode_b{args.batch}"] = round(main_point["tok_s"], 1)
        prefill = prefill_point()
        if not args.no_generate:
            for b in sorted({args.batch, 64}):
                g = generate_point(b)
                if g is not None:
                    generate[f"b{b}"] = g
            g = generate_point(64, sampled=True)
            if g is not None:
                generate["b64_sampled"] = g

    step_bytes = weight_bytes + args.batch * main_point["mean_len"] * kv_bytes_per_token
    achieved = step_bytes / (main_point["ms"] * 1e-3) / 1e9
    line = {
        "metric": "decode tokens/s", "value": round(main_point["tok_s"], 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(main_point["ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_name,
        "data": "synthetic: seeded random weights, random token ids, random cache contents",
        "config": {"model": shape_name, "layers": cfg.num_hidden_layers,
                   "layers_full": shape["num_hidden_layers"], "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": vocab,
                   "global_batch": args.batch, "seq_len": ctx_of[args.batch], "parallelism": "none (1 GPU)",
                   "weights": dtype_name, "cache": f"{dtype_name} pages of 64 tokens",
                   "l2": "inputs larger than L2 (all weights are read every step)",
                   "decode": "CUDA graph replay, one captured graph per batch size",
                   "prefill_tokens": PREFILL_TOKENS},
        "repeats": reps, "cv": main_point["cv"],
        "clocks": main_point["clocks"],
        "e2e": main_point.get("e2e"),
        "gpu_launches": main_point["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"],
                     "bytes_per_step": int(step_bytes)},
        "shares": main_point.get("shares"),
    }
    if prefill is not None:
        line["prefill"] = prefill
        line["points"] = points
    if generate:
        line["generate"] = generate
    print(json.dumps(line))
    return 0


KUBEDRA_SIZES = {
    # width, heads and feed-forward of the Llama shape of the same name; four layers, one of each pairing of mixer and feed-forward
    "1b": dict(width=2048, heads=16, key=64, value=128, q_rank=768, kv_rank=128, att_dim=128, window=1024, ff=8192,
               experts=16, top=2, expert_ff=2048, shared_ff=2048, llama=dict(heads=16, kv_heads=4, head_dim=128, ff=8192)),
    "8b": dict(width=4096, heads=32, key=64, value=128, q_rank=1536, kv_rank=128, att_dim=128, window=1024, ff=14336,
               experts=32, top=4, expert_ff=2048, shared_ff=2048, llama=dict(heads=32, kv_heads=8, head_dim=128, ff=14336)),
}


def design_bench_tools(args):
    """What the workloads that set a design beside a Llama of equal size share: the measured peaks, a timer of one call
    (median of the repetitions after three warm-ups, the L2 flushed before each unless told otherwise), and the three
    points of a model (a prompt of `prefill_tokens` through an eager step, decode steps of 8 and 64 sequences at a context
    of 2,048 tokens through captured steps)."""
    import types
    import numpy as np
    import torch
    from dotllm_b200 import StepEntry
    pk = peaks()
    hbm, tflops = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    gen = torch.Generator().manual_seed(1)
    reps, T, ctx = max(3, args.repeats), args.prefill_tokens, 2048
    sampler = ClockSampler()
    def timed(fn, n=None, flushed=True):
        n = n or reps
        out = []
        for it in range(3 + n):
            if flushed:
                flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if it >= 3:
                out.append(a.elapsed_time(b))
        return statistics.median(out)

    def model_points(model, vocab):
        res = {}
        prompt = np.asarray(torch.randint(0, vocab, (T,), generator=gen))
        cache = model.new_cache(max_tokens=64 * (ctx + 192), max_sequences=64)

        def prefill():
            s = cache.open_sequence()
            model.step(cache, [StepEntry(s, prompt)])
            cache.close_sequence(s)
        ms = timed(prefill, flushed=False)
        res["prefill_tok_s"] = round(T * 1000.0 / ms, 1)
        res["prefill_ms"] = round(ms, 3)
        for batch in (8, 64):
            seqs = [cache.open_sequence() for _ in range(batch)]
            for lo in range(0, batch, 8):                       # fill the contexts through the model, eight prompts a step
                model.step(cache, [StepEntry(s, np.asarray(torch.randint(0, vocab, (ctx,), generator=gen)), []) for s in seqs[lo:lo + 8]])
            ids = [[int(t)] for t in torch.randint(0, vocab, (batch,), generator=gen)]
            step = lambda: model.step(cache, [StepEntry(s, t) for s, t in zip(seqs, ids)], graphs=True)
            for _ in range(max(3, args.warmup)):
                step()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(args.steps):
                step()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / args.steps
            res[f"decode_b{batch}_tok_s"] = round(batch * 1000.0 / ms, 1)
            res[f"decode_b{batch}_ms"] = round(ms, 3)
            for s in seqs:
                cache.close_sequence(s)
        return res

    return types.SimpleNamespace(pk=pk, hbm=hbm, tflops=tflops, dev=dev, reps=reps, T=T, ctx=ctx, sampler=sampler, timed=timed,
                                 model_points=model_points)


def kubedra_workload(args):
    """Prefill (one prompt of 2,048 tokens) and decode (batch 8 and 64 at context 2,048) tokens per second of a four-layer
    Kubedra model at a real model's layer sizes, beside a four-layer Llama of the same width, head count and feed-forward
    width; then every kernel of the new design alone against its roofline (bytes it must move over the measured copy
    bandwidth, or arithmetic over the measured bf16 rate), beside the like kernel of the Llama path.  Random weights,
    synthetic tokens, bfloat16, CUDA events, an L2 flush between the timed launches of a kernel."""
    import torch
    from dotllm_b200 import Model
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.kernels import ops
    tools = design_bench_tools(args)
    pk, hbm, tflops, dev, T, ctx, sampler, timed, model_points = (tools.pk, tools.hbm, tools.tflops, tools.dev, tools.T, tools.ctx,
                                                                  tools.sampler, tools.timed, tools.model_points)
    sizes = ["1b", "8b"] if args.shape not in ("1b",) else ["1b"]

    def kernel_table(z):
        """Each kernel alone: (microseconds, fraction of its roofline) at prefill (T rows) and decode (64 rows) sizes."""
        W, H, dk, dv, r, E, top, ff = z["width"], z["heads"], z["key"], z["value"], z["kv_rank"], z["experts"], z["top"], z["expert_ff"]
        bf = torch.bfloat16
        rows = {}

        def row(name, fn, bytes_=0, flops=0):
            us = timed(fn) * 1000.0
            need = max(bytes_ / hbm, flops / tflops) * 1e6
            rows[name] = {"us": round(us, 1), "roofline_us": round(need, 2), "frac": round(need / us, 4)}
        for label, n, n_seqs in (("prefill", T, 1), ("decode", 64, 64)):
            x = torch.randn(n, W, device=dev).to(bf)
            stream, delta = torch.randn(n, W, device=dev), torch.randn(n, W, device=dev)
            gain = torch.ones(W, device=dev)
            # the norm between sublayers: new (branch normalised, added, sum normalised) and old (added, normalised)
            row(f"branch_norm_add {label}", lambda: ops.add_rmsnorm(stream, ops.NormedBranch(delta, gain, 1e-5), gain, 1e-5, bf),
                bytes_=n * W * (4 + 4 + 4 + 2))
            row(f"llama add_rmsnorm {label}", lambda: ops.add_rmsnorm(stream, delta, gain, 1e-5, bf), bytes_=n * W * (4 + 4 + 4 + 2))
            # gated linear attention: the scan and the per-head norm with its gate
            kw, vw = H * dk, H * dv
            proj = torch.randn(n, 2 * kw + 2 * vw, device=dev).to(bf)
            zz, zb = torch.randn(n, kw, device=dev), torch.zeros(kw, device=dev)
            state = torch.zeros(n_seqs + 1, H, dk, dv, device=dev)
            cu = torch.arange(0, n + 1, n // n_seqs, dtype=torch.int32, device=dev)
            slots = torch.arange(n_seqs, dtype=torch.int32, device=dev)
            scan = lambda: ops.gla_scan(proj[:, :kw], proj[:, kw:2 * kw], proj[:, 2 * kw:2 * kw + vw], zz, zb, cu, slots, state,
                                        H, dk, dv, dk ** -0.5, 16.0)
            io = n * (2 * kw * 2 + vw * 2 + kw * 4 + vw * 4) + 2 * n_seqs * H * dk * dv * 4
            row(f"gla_scan {label}", scan, bytes_=io, flops=4 * n * H * dk * dv)
            o = scan()
            row(f"head_norm_gate {label}", lambda: ops.head_norm_gate(o, proj[:, 2 * kw + vw:], torch.ones(dv, device=dev), H, dv, 1e-5, bf),
                bytes_=n * vw * (4 + 2 + 2))
            # experts
            wr, wgu = torch.randn(E, W, device=dev).to(bf), (torch.randn(E, 2 * ff, W, device=dev) * 0.02).to(bf)
            wd = (torch.randn(E, W, ff, device=dev) * 0.02).to(bf)
            ids, wts = ops.route_topk(x, wr, None, top)
            used = min(E, n * top)
            row(f"route_topk {label}", lambda: ops.route_topk(x, wr, None, top), bytes_=n * W * 2 + E * W * 2, flops=2 * n * E * W)
            row(f"expert_gate_up {label}", lambda: ops.expert_gate_up(x, ids, wgu, "clamped_sigmoid", 7.0, 1.702),
                bytes_=used * 2 * ff * W * 2 + n * W * 2 + n * top * ff * 2, flops=2 * n * top * 2 * ff * W)
            h = ops.expert_gate_up(x, ids, wgu, "clamped_sigmoid", 7.0, 1.702)
            row(f"expert_down {label}", lambda: ops.expert_down(h, ids, wts, wd), bytes_=used * ff * W * 2 + n * top * ff * 2 + n * W * 4,
                flops=2 * n * top * ff * W)
            if ops.experts_grouped_takes(x, ids, wgu, wd):
                # the path a step of this many rows takes: sort, gather, two tcgen05 products, weighted sum
                row(f"experts sorted on tensor cores {label}", lambda: ops.experts_grouped(x, ids, wts, wgu, wd, "clamped_sigmoid", 7.0, 1.702),
                    bytes_=used * 3 * ff * W * 2 + n * W * (2 + 4) + n * top * (W * 2 + ff * 4 + W * 8), flops=2 * n * top * 3 * ff * W)
            # the like kernel of the Llama path: the dense gated product of the same rows
            wl = (torch.randn(2 * z["ff"], W, device=dev) * 0.02).to(bf)
            row(f"llama gated product {label}", lambda: ops.gated_linear(x, wl, resident=True),
                bytes_=2 * z["ff"] * W * 2 + n * W * 2 + n * z["ff"] * 2, flops=2 * n * 2 * z["ff"] * W)
            del wgu, wd, wl
        return rows

    out = {}
    for name in sizes:
        z = KUBEDRA_SIZES[name]
        mix_g = {"heads": z["heads"], "dim": z["key"], "vdim": z["value"], "tau": 16.0, "decay_rank": 64}
        mix_l = {"heads": z["heads"], "dim": z["att_dim"], "vdim": z["att_dim"], "q_rank": z["q_rank"], "kv_rank": z["kv_rank"],
                 "mask": {"size": z["window"]}}
        moe = {"kind": "moe", "expert": {"ff": z["expert_ff"], "limit": 7.0}, "router": {"experts": z["experts"], "top": z["top"]},
               "shared": {"ff": z["shared_ff"], "limit": 7.0}}
        dense = {"kind": "dense", "ff": z["ff"]}
        vocab = 32000
        kcfg = {"architecture": "Kubedra", "vocab": vocab, "width": z["width"], "max_positions": 8192, "norm": {"eps": 1e-5},
                "layers": [{"type": "gla", "mixer": mix_g, "mlp": dense}, {"type": "gla", "mixer": mix_g, "mlp": moe},
                           {"type": "latent_attention", "mixer": mix_l, "mlp": moe},
                           {"type": "latent_attention", "mixer": mix_l, "mlp": dense}]}
        la = z["llama"]
        lcfg = dict(LLAMA_31_8B, num_hidden_layers=4, hidden_size=z["width"], num_attention_heads=la["heads"],
                    num_key_value_heads=la["kv_heads"], head_dim=la["head_dim"], intermediate_size=la["ff"], vocab_size=vocab,
                    max_position_embeddings=8192, tie_word_embeddings=True)
        point = {}
        for label, cfg_dict in (("kubedra", kcfg), ("llama", lcfg)):
            model = Model.random(config_from_dict(cfg_dict), seed=0, dtype="bfloat16", device="cuda:0", on_device=True)
            point[label] = model_points(model, vocab)
            print(f"[bench] {name} {label}: {point[label]}", file=sys.stderr, flush=True)
            del model
            torch.cuda.empty_cache()
        point["kernels"] = kernel_table(z)
        for k, v in point["kernels"].items():
            print(f"[bench] {name} {k}: {v}", file=sys.stderr, flush=True)
        out[name] = point
    first = out[sizes[0]]
    print(json.dumps({"metric": "kubedra_decode_tokens_per_second", "value": first["kubedra"]["decode_b8_tok_s"], "unit": "tokens/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "higher_is_better": True, "dtype": "bf16",
                      "data": "synthetic", "vs_baseline": None, "clocks": sampler.stop(),
                      "config": {"model": "Kubedra, four layers at the sizes named", "batch": 8, "context": ctx, "prefill_tokens": T,
                                 "l2": "flushed between a kernel's timed launches"},
                      "peaks": pk, "sizes": out}))
    return 0


KOMULORN_SIZES = {
    # width, heads, key/value heads and head size of the Llama shape of the same name; four layers, the second and the fourth
    # reading the keys and values of the layer before them; every layer with routed experts and a gated shared expert
    "1b": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, rot=64, experts=16, top=2, expert_ff=2048, shared_ff=2048, ff=8192),
    "8b": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, rot=64, experts=32, top=4, expert_ff=2048, shared_ff=2048, ff=14336),
    # keys narrower than values: every head laid out at the values' width (zeros behind the keys)
    "8b-96-128": dict(width=4096, heads=32, kv_heads=8, dim=96, vdim=128, rot=32, experts=32, top=4, expert_ff=2048, shared_ff=2048,
                      ff=14336),
}


def komulorn_workload(args):
    """Prefill (one prompt of 2,048 tokens) and decode (batch 8 and 64 at context 2,048) tokens per second of a four-layer
    Komulorn model at a real model's layer sizes, beside a four-layer Llama of the same width, heads and head size (its
    closest relative here: the same attention over the same paged cache, a dense feed-forward instead of experts); then the
    kernels that the design adds or changes, each alone against its roofline (bytes it must move over the measured copy
    bandwidth, or arithmetic over the measured bf16 rate), beside the like kernel of the Llama or the Kubedra path.  Random
    weights, synthetic tokens, bfloat16, CUDA events, an L2 flush between the timed launches of a kernel."""
    import torch
    from dotllm_b200 import Model
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.engine.step import AttentionPlan
    from dotllm_b200.kernels import ops
    tools = design_bench_tools(args)
    pk, hbm, tflops, dev, T, ctx, sampler, timed, model_points = (tools.pk, tools.hbm, tools.tflops, tools.dev, tools.T, tools.ctx,
                                                                  tools.sampler, tools.timed, tools.model_points)
    sizes = ["1b"] if args.shape == "1b" else ["1b", "8b", "8b-96-128"]
    bf = torch.bfloat16

    def kernel_table(z):
        W, H, G, hd, rd, E, top, ff = z["width"], z["heads"], z["kv_heads"], max(z["dim"], z["vdim"]), z["rot"], z["experts"], z["top"], z["expert_ff"]
        rows = {}

        def row(name, fn, bytes_=0, flops=0):
            us = timed(fn) * 1000.0
            need = max(bytes_ / hbm, flops / tflops) * 1e6
            rows[name] = {"us": round(us, 1), "roofline_us": round(need, 2), "frac": round(need / us, 4)}
        pos_table = torch.arange(ctx + T + 8, dtype=torch.float64)[:, None] * (1e4 ** (-torch.arange(hd // 2, dtype=torch.float64) / (hd // 2)))
        cos_full, sin_full = torch.cos(pos_table).float().to(dev), torch.sin(pos_table).float().to(dev)
        # the rotation of rd channels as the bfloat16 layout runs it: spread over the head, cos 1 and sin 0 behind the real columns
        cos_part = torch.cat([cos_full[:, :rd // 2], torch.ones_like(cos_full[:, rd // 2:])], dim=1).contiguous()
        sin_part = torch.cat([sin_full[:, :rd // 2], torch.zeros_like(sin_full[:, rd // 2:])], dim=1).contiguous()
        qw, kw = H * hd, G * hd
        for label, n_seqs, new, start in (("prefill", 1, T, 0), ("decode", 64, 1, ctx)):
            n = n_seqs * new
            pages_per = (start + new + 63) // 64
            k_pool = torch.randn(n_seqs * pages_per + 1, G, 64, hd, device=dev).to(bf)
            v_pool = torch.randn(n_seqs * pages_per + 1, G, hd, 64, device=dev).to(bf)
            table = torch.arange(n_seqs * pages_per, dtype=torch.int32, device=dev).reshape(n_seqs, pages_per)
            seq = torch.arange(n_seqs, dtype=torch.int32, device=dev).repeat_interleave(new)
            pos = (torch.arange(new, dtype=torch.int32, device=dev) + start).repeat(n_seqs)
            i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
            plan = AttentionPlan(n_seqs, new, start + new, new == 1, i32([start] * n_seqs), i32([new] * n_seqs),
                                 i32([new * b for b in range(n_seqs + 1)]), i32([start + new] * n_seqs), [start] * n_seqs, [new] * n_seqs)
            y = torch.randn(n, qw + 2 * kw + H + (-H % 16), device=dev).to(bf)
            q, k, v, g = y[:, :qw], y[:, qw:qw + kw], y[:, qw + kw:qw + 2 * kw], y[:, qw + 2 * kw:qw + 2 * kw + H]
            biases = tuple(torch.randn(m, device=dev) for m in (qw, kw, kw))
            moved = n * (2 * qw + 2 * kw) * 2                                     # q read and written, k and v read and written
            row(f"rotation of a part of the head + biases + cache write {label}",
                lambda: ops.rope_cache_write(q, k, v, cos_part, sin_part, hd, seq, pos, table, k_pool, v_pool, H, G, hd, biases=biases), bytes_=moved)
            row(f"llama rotation + cache write {label}",
                lambda: ops.rope_cache_write(q, k, v, cos_full, sin_full, hd, seq, pos, table, k_pool, v_pool, H, G, hd), bytes_=moved)
            kv_bytes = n_seqs * (start + new) * 2 * kw * 2
            att_flops = 4 * H * hd * (n_seqs * (new * start + new * (new + 1) // 2))
            att_io = kv_bytes + n * 2 * qw * 2
            row(f"attention + head gate {label}", lambda: ops.attention(q, k_pool, v_pool, seq, pos, table, H, G, hd, hd ** -0.5, plan=plan, gate=g),
                bytes_=att_io + n * 2 * qw * 2, flops=att_flops)
            row(f"llama attention {label}", lambda: ops.attention(q, k_pool, v_pool, seq, pos, table, H, G, hd, hd ** -0.5, plan=plan),
                bytes_=att_io, flops=att_flops)
            if new == 1:
                row("rotation + biases + cache write, attention and gate in one launch (decode)",
                    lambda: ops.rope_cache_attention(q, k, v, cos_part, sin_part, hd, seq, pos, table, k_pool, v_pool, H, G, hd, hd ** -0.5,
                                                     plan=plan, biases=biases, gate=g), bytes_=att_io + moved)
                row("llama rotation, cache write and attention in one launch (decode)",
                    lambda: ops.rope_cache_attention(q, k, v, cos_full, sin_full, hd, seq, pos, table, k_pool, v_pool, H, G, hd, hd ** -0.5,
                                                     plan=plan), bytes_=att_io + moved)
            del k_pool, v_pool
            # experts: one product with the square of relu, the score on the rows that go in
            x = torch.randn(n, W, device=dev).to(bf)
            wr = torch.randn(E + 8, W, device=dev).to(bf)                       # the experts' rows, the shared expert's gate, rows of padding
            wu, wd = (torch.randn(E, ff, W, device=dev) * 0.02).to(bf), (torch.randn(E, W, ff, device=dev) * 0.02).to(bf)
            wgu = (torch.randn(E, 2 * ff, W, device=dev) * 0.02).to(bf)
            ids, wts, zl = ops.route_topk(x, wr, None, top, scoring="sigmoid", experts=E, with_logits=True)
            shared = torch.randn(n, W, device=dev)
            used = min(E, n * top)
            row(f"route_topk, sigmoid scores {label}", lambda: ops.route_topk(x, wr, None, top, scoring="sigmoid", experts=E),
                bytes_=n * W * 2 + E * W * 2, flops=2 * n * E * W)
            if ops.experts_grouped_takes(x, ids, wu, wd):
                row(f"experts sorted on tensor cores {label}",
                    lambda: ops.experts_grouped(x, ids, None, wu, wd, "relu2", addend=shared, row_scale=wts, addend_gate=zl[:, E:E + 1]),
                    bytes_=used * 2 * ff * W * 2 + n * W * (2 + 4 + 4) + n * top * (W * 2 + ff * 4 + W * 8), flops=2 * n * top * 2 * ff * W)
                row(f"kubedra experts (gate and up) sorted on tensor cores {label}",
                    lambda: ops.experts_grouped(x, ids, wts, wgu, wd, "clamped_sigmoid", 7.0, 1.702, addend=shared),
                    bytes_=used * 3 * ff * W * 2 + n * W * (2 + 4 + 4) + n * top * (W * 2 + ff * 4 + W * 8), flops=2 * n * top * 3 * ff * W)
            else:
                row(f"expert up, row by row {label}", lambda: ops.expert_gate_up(x, ids, wu, "relu2", row_scale=wts),
                    bytes_=used * ff * W * 2 + n * W * 2 + n * top * ff * 2, flops=2 * n * top * ff * W)
                h = ops.expert_gate_up(x, ids, wu, "relu2", row_scale=wts)
                row(f"expert down, row by row {label}", lambda: ops.expert_down(h, ids, None, wd, addend=shared, addend_gate=zl[:, E:E + 1]),
                    bytes_=used * ff * W * 2 + n * top * ff * 2 + n * W * 8, flops=2 * n * top * ff * W)
                row(f"kubedra expert gate and up, row by row {label}", lambda: ops.expert_gate_up(x, ids, wgu, "clamped_sigmoid", 7.0, 1.702),
                    bytes_=used * 2 * ff * W * 2 + n * W * 2 + n * top * ff * 2, flops=2 * n * top * 2 * ff * W)
            # the shared expert's first product with its activation, beside the Llama path's gated product of the same width
            ws, wl = (torch.randn(z["shared_ff"], W, device=dev) * 0.02).to(bf), (torch.randn(2 * z["shared_ff"], W, device=dev) * 0.02).to(bf)
            row(f"shared expert: product + square of relu {label}", lambda: ops.activated_linear(x, ws, "relu2", resident=True),
                bytes_=z["shared_ff"] * W * 2 + n * W * 2 + n * z["shared_ff"] * 2, flops=2 * n * z["shared_ff"] * W)
            row(f"llama gated product of that width {label}", lambda: ops.gated_linear(x, wl, resident=True),
                bytes_=2 * z["shared_ff"] * W * 2 + n * W * 2 + n * z["shared_ff"] * 2, flops=2 * n * 2 * z["shared_ff"] * W)
            logits = torch.randn(n_seqs, 32000, device=dev)
            row(f"cap on the logits {label}", lambda: ops.softcap(logits, 30.0), bytes_=n_seqs * 32000 * 8)
            del wu, wd, wgu, ws, wl
        return rows

    out = {}
    for name in sizes:
        z = KOMULORN_SIZES[name]
        vocab = 32000
        mixer = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
                 "rot": {"dims": z["rot"], "base": 10000.0, "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}
        moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"]},
               "shared": {"ff": z["shared_ff"]}}
        own = lambda: {"type": "attention", "mixer": dict(mixer), "mlp": moe}
        reads = lambda j: {"type": "attention", "mixer": dict(mixer, kv_from=j), "mlp": moe}
        kcfg = {"architecture": "Komulorn", "vocab": vocab, "width": z["width"], "max_positions": 8192, "norm": {"eps": 1e-5},
                "logit_softcap": 30.0, "layers": [own(), reads(0), own(), reads(2)]}
        lcfg = dict(LLAMA_31_8B, num_hidden_layers=4, hidden_size=z["width"], num_attention_heads=z["heads"],
                    num_key_value_heads=z["kv_heads"], head_dim=max(z["dim"], z["vdim"]), intermediate_size=z["ff"], vocab_size=vocab,
                    max_position_embeddings=8192, tie_word_embeddings=True)
        point = {}
        for label, cfg_dict in (("komulorn", kcfg), ("llama", lcfg)):
            model = Model.random(config_from_dict(cfg_dict), seed=0, dtype="bfloat16", device="cuda:0", on_device=True)
            point[label] = model_points(model, vocab)
            print(f"[bench] {name} {label}: {point[label]}", file=sys.stderr, flush=True)
            del model
            torch.cuda.empty_cache()
        if z["dim"] == z["vdim"]:
            point["kernels"] = kernel_table(z)
            for k, v in point["kernels"].items():
                print(f"[bench] {name} {k}: {v}", file=sys.stderr, flush=True)
        out[name] = point
    first = out[sizes[0]]
    print(json.dumps({"metric": "komulorn_decode_tokens_per_second", "value": first["komulorn"]["decode_b8_tok_s"], "unit": "tokens/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "higher_is_better": True, "dtype": "bf16",
                      "data": "synthetic", "vs_baseline": None, "clocks": sampler.stop(),
                      "config": {"model": "Komulorn, four layers at the sizes named", "batch": 8, "context": ctx, "prefill_tokens": T,
                                 "l2": "flushed between a kernel's timed launches"},
                      "peaks": pk, "sizes": out}))
    return 0


ZEMEZEN_SIZES = {
    # width, heads and feed-forward of the Llama shape of the same name, state and latent sizes of the Kubedra sizes above; four
    # layers: delta rule + dense, delta rule + experts, latent attention + experts, windowed attention + dense
    "1b": dict(width=2048, heads=16, key=64, value=128, conv=4, kv_rank=128, att_dim=128, att_heads=16, att_kv=4, window=1024,
               keep=4, rot=64, ff=8192, experts=16, top=2, groups=(4, 2), expert_ff=2048),
    "8b": dict(width=4096, heads=32, key=64, value=128, conv=4, kv_rank=128, att_dim=128, att_heads=32, att_kv=8, window=1024,
               keep=4, rot=64, ff=14336, experts=32, top=4, groups=(8, 4), expert_ff=2048),
}


def zemezen_workload(args):
    """Prefill (one prompt of 2,048 tokens) and decode (batch 8 and 64 at context 2,048) tokens per second of a four-layer
    Zemezen model at a real model's layer sizes, beside a four-layer Kubedra (the closest design here: a recurrent state
    per head, latent attention, routed experts) of the same width, heads, state, latent, window and feed-forward sizes;
    then every kernel the design added, alone, against its roofline, beside the like kernel of the Kubedra or Llama path.
    Random weights, synthetic tokens, bfloat16, CUDA events, an L2 flush between the timed launches of a kernel."""
    import numpy as np
    import torch
    from dotllm_b200 import Model
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.engine.step import AttentionPlan
    from dotllm_b200.kernels import ops
    tools = design_bench_tools(args)
    pk, hbm, tflops, dev, T, ctx, sampler, timed, model_points = (tools.pk, tools.hbm, tools.tflops, tools.dev, tools.T, tools.ctx,
                                                                  tools.sampler, tools.timed, tools.model_points)
    sizes = ["1b", "8b"] if args.shape not in ("1b",) else ["1b"]

    def kernel_table(z):
        W, H, dk, dv, K, E, top = z["width"], z["heads"], z["key"], z["value"], z["conv"], z["experts"], z["top"]
        nh, nkv, hd, window, keep = z["att_heads"], z["att_kv"], z["att_dim"], z["window"], z["keep"]
        bf = torch.bfloat16
        rows = {}
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)

        def row(name, fn, bytes_=0, flops=0):
            us = timed(fn) * 1000.0
            need = max(bytes_ / hbm, flops / tflops) * 1e6
            rows[name] = {"us": round(us, 1), "roofline_us": round(need, 2), "frac": round(need / us, 4)}
        for label, n, n_seqs in (("prefill", T, 1), ("decode", 64, 64)):
            # the delta rule (convolutions, unit lengths, decays, the recurrence) beside the gated-linear-attention scan
            kw, vw = H * dk, H * dv
            C = 2 * kw + vw
            proj = torch.randn(n, C + H, device=dev).to(bf)
            taps = (torch.randn(C, K, device=dev) * 0.5).to(bf)
            zz, zb, a_log = torch.randn(n, kw, device=dev), torch.zeros(kw, device=dev), torch.zeros(H, device=dev)
            memory = torch.zeros(n_seqs + 1, H * dk * dv + (K - 1) * C, device=dev)
            cu = torch.arange(0, n + 1, n // n_seqs, dtype=torch.int32, device=dev)
            seq = torch.arange(n, dtype=torch.int32, device=dev) // (n // n_seqs)
            slots = torch.arange(n_seqs, dtype=torch.int32, device=dev)
            delta = lambda: ops.delta_rule(proj, taps, proj[:, C:], zz, zb, a_log, seq, cu, slots, memory, H, H, dk, dv, dk ** -0.5, 1e-6)
            io = n * (C * 2 + kw * 4 + vw * 4) + 2 * n_seqs * H * dk * dv * 4
            row(f"delta_rule (prepare + scan) {label}", delta, bytes_=io, flops=6 * n * H * dk * dv)
            state = torch.zeros(n_seqs + 1, H, dk, dv, device=dev)
            gla = lambda: ops.gla_scan(proj[:, :kw], proj[:, kw:2 * kw], proj[:, 2 * kw:2 * kw + vw], zz, zb, cu, slots, state,
                                       H, dk, dv, dk ** -0.5, 16.0)
            row(f"kubedra gla_scan {label}", gla, bytes_=n * (C * 2 + kw * 4 + vw * 4) + 2 * n_seqs * H * dk * dv * 4, flops=4 * n * H * dk * dv)
            o = gla()
            g = torch.randn(n, vw, device=dev).to(bf)
            for gate in ("sigmoid", "silu"):
                row(f"head_norm_gate {gate} {label}", lambda: ops.head_norm_gate(o, g, torch.ones(dv, device=dev), H, dv, 1e-5, bf, gate=gate),
                    bytes_=n * vw * (4 + 2 + 2))
            # queries and keys normalised per head; windowed attention with kept tokens and sinks beside the same window without
            qk = torch.randn(n, (nh + 2 * nkv) * hd, device=dev).to(bf)
            gq = torch.ones(hd, device=dev)
            row(f"head_rmsnorm (queries and keys) {label}", lambda: ops.head_rmsnorm(qk[:, :(nh + nkv) * hd], gq, nh, hd, 1e-5, gq, nkv),
                bytes_=n * (nh + nkv) * hd * 4)
            per = ctx if label == "decode" else n
            pages = (per + 63) // 64
            k_pool = torch.randn(n_seqs * pages + 1, nkv, 64, hd, device=dev).to(bf)
            v_pool = torch.randn(n_seqs * pages + 1, nkv, hd, 64, device=dev).to(bf)
            table = torch.arange(n_seqs * pages, dtype=torch.int32, device=dev).reshape(n_seqs, pages)
            starts, news = ([0], [n]) if label == "prefill" else ([ctx - 1] * n_seqs, [1] * n_seqs)
            totals = [a + b for a, b in zip(starts, news)]
            pos = i32([a + i for a, b in zip(starts, news) for i in range(b)])
            q = qk[:, :nh * hd]
            sinks = torch.zeros(nh, device=dev)
            seen = sum(min(p + 1, window + keep) for p in pos.tolist())             # keys the step's queries see, per KV head
            att_bytes = (min(per, window + 64) * n_seqs if label == "decode" else per) * nkv * hd * 2 * 2 + n * nh * hd * 4
            for name, kw_ in (("windowed attention, kept tokens and sinks", dict(keep_first=keep, sinks=sinks)), ("llama windowed attention", {})):
                plan = AttentionPlan(n_seqs, max(news), max(totals), label == "decode", i32(starts), i32(news),
                                     i32([0] + list(np.cumsum(news))), i32(totals), list(starts), list(news))
                row(f"{name} {label}", lambda: ops.attention(q, k_pool, v_pool, seq, pos, table, nh, nkv, hd, hd ** -0.5, window, plan=plan, **kw_),
                    bytes_=att_bytes, flops=4 * seen * nh * hd)
            del k_pool, v_pool
            # the router: softmax over all experts and groups, beside the softmax over the chosen
            x = torch.randn(n, W, device=dev).to(bf)
            wr = torch.randn(E, W, device=dev).to(bf)
            row(f"route_topk, softmax over all, groups {label}", lambda: ops.route_topk(x, wr, None, top, scoring="softmax_all", groups=z["groups"]),
                bytes_=n * W * 2 + E * W * 2, flops=2 * n * E * W)
            row(f"kubedra route_topk {label}", lambda: ops.route_topk(x, wr, None, top), bytes_=n * W * 2 + E * W * 2, flops=2 * n * E * W)
        return rows

    out = {}
    for name in sizes:
        z = ZEMEZEN_SIZES[name]
        vocab = 32000
        moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]},
               "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": z["groups"][0], "keep": z["groups"][1]}}}
        dense = {"kind": "dense", "ff": z["ff"]}
        mix_d = {"heads": z["heads"], "kv_heads": z["heads"], "dim": z["key"], "vdim": z["value"], "conv": z["conv"], "ranks": [64, 64]}
        mix_l = {"heads": z["heads"], "dim": z["att_dim"], "vdim": z["att_dim"], "kv_rank": z["kv_rank"], "scale": z["att_dim"] ** -0.5}
        mix_a = {"heads": z["att_heads"], "kv_heads": z["att_kv"], "dim": z["att_dim"], "vdim": z["att_dim"], "scale": z["att_dim"] ** -0.5,
                 "mask": {"size": z["window"], "keep_first": z["keep"]}, "rot": {"dims": z["rot"], "base": 10000.0}}
        zcfg = {"architecture": "Zemezen", "vocab": vocab, "width": z["width"], "max_positions": 8192, "norm": {"eps": 1e-5},
                "layers": [{"type": "channel_delta", "mixer": mix_d, "mlp": dense}, {"type": "channel_delta", "mixer": mix_d, "mlp": moe},
                           {"type": "latent_attention", "mixer": mix_l, "mlp": moe}, {"type": "attention", "mixer": mix_a, "mlp": dense}]}
        kz = KUBEDRA_SIZES[name]
        mix_g = {"heads": kz["heads"], "dim": kz["key"], "vdim": kz["value"], "tau": 16.0, "decay_rank": 64}
        mix_kl = {"heads": kz["heads"], "dim": kz["att_dim"], "vdim": kz["att_dim"], "q_rank": kz["q_rank"], "kv_rank": kz["kv_rank"],
                  "mask": {"size": kz["window"]}}
        kmoe = {"kind": "moe", "expert": {"ff": kz["expert_ff"], "limit": 7.0}, "router": {"experts": kz["experts"], "top": kz["top"]}}
        kcfg = {"architecture": "Kubedra", "vocab": vocab, "width": kz["width"], "max_positions": 8192, "norm": {"eps": 1e-5},
                "layers": [{"type": "gla", "mixer": mix_g, "mlp": dense}, {"type": "gla", "mixer": mix_g, "mlp": kmoe},
                           {"type": "latent_attention", "mixer": mix_kl, "mlp": kmoe},
                           {"type": "latent_attention", "mixer": mix_kl, "mlp": dense}]}
        point = {}
        for label, cfg_dict in (("zemezen", zcfg), ("kubedra", kcfg)):
            model = Model.random(config_from_dict(cfg_dict), seed=0, dtype="bfloat16", device="cuda:0", on_device=True)
            point[label] = model_points(model, vocab)
            print(f"[bench] {name} {label}: {point[label]}", file=sys.stderr, flush=True)
            del model
            torch.cuda.empty_cache()
        point["kernels"] = kernel_table(z)
        for k, v in point["kernels"].items():
            print(f"[bench] {name} {k}: {v}", file=sys.stderr, flush=True)
        out[name] = point
    first = out[sizes[0]]
    print(json.dumps({"metric": "zemezen_decode_tokens_per_second", "value": first["zemezen"]["decode_b8_tok_s"], "unit": "tokens/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "higher_is_better": True, "dtype": "bf16",
                      "data": "synthetic", "vs_baseline": None, "clocks": sampler.stop(),
                      "config": {"model": "Zemezen, four layers at the sizes named", "batch": 8, "context": ctx, "prefill_tokens": T,
                                 "l2": "flushed between a kernel's timed launches"},
                      "peaks": pk, "sizes": out}))
    return 0


def sopalorn_workload(args):
    """Prefill (one prompt of 2,048 tokens) and decode (batch 8 and 64 at context 2,048) tokens per second of a four-layer
    Sopalorn model at a real model's layer sizes (two copies of the stream), beside a four-layer Zemezen (the closest design
    here: a delta rule, windowed attention with sinks, experts scored by a softmax over all) of the same width, heads,
    state, window and feed-forward sizes; then every kernel the design added or changed, alone, against its roofline, beside
    the like kernel of the closest path.  Random weights, synthetic tokens, bfloat16, CUDA events, an L2 flush between the
    timed launches of a kernel."""
    import numpy as np
    import torch
    from dotllm_b200 import Model
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.engine.step import AttentionPlan
    from dotllm_b200.kernels import ops
    tools = design_bench_tools(args)
    pk, hbm, tflops, dev, T, ctx, sampler, timed, model_points = (tools.pk, tools.hbm, tools.tflops, tools.dev, tools.T, tools.ctx,
                                                                  tools.sampler, tools.timed, tools.model_points)
    sizes = ["1b", "8b"] if args.shape not in ("1b",) else ["1b"]
    COPIES = 2

    def kernel_table(z):
        W, H, dk, dv, K, E, top = z["width"], z["heads"], z["key"], z["value"], z["conv"], z["experts"], z["top"]
        nh, nkv, hd, window = z["att_heads"], z["att_kv"], z["att_dim"], z["window"]
        bf = torch.bfloat16
        rows = {}
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)

        def row(name, fn, bytes_=0, flops=0):
            us = timed(fn) * 1000.0
            need = max(bytes_ / hbm, flops / tflops) * 1e6
            rows[name] = {"us": round(us, 1), "roofline_us": round(need, 2), "frac": round(need / us, 4)}
        for label, n, n_seqs in (("prefill", T, 1), ("decode", 64, 64)):
            # the stream of copies: write, read and layer norm in one pass, beside the residual add fused into an RMS norm
            x = torch.randn(n, COPIES * W, device=dev)
            y = torch.randn(n, W, device=dev)
            ones = torch.ones(W, device=dev)
            write = ops.StreamWrite(y, ones, torch.eye(COPIES, device=dev), torch.ones(COPIES, device=dev))
            read = torch.full((COPIES,), 1.0 / COPIES, device=dev)
            row(f"stream_norm (write, read, layer norm; {COPIES} copies) {label}",
                lambda: ops.stream_norm(x, COPIES, write, read, ones, ones, 1e-5, bf), bytes_=n * W * (8 * COPIES + 4 + 2))
            xr = torch.randn(n, W, device=dev)
            row(f"llama add_rmsnorm {label}", lambda: ops.add_rmsnorm(xr, y, ones, 1e-5, bf), bytes_=n * W * (8 + 4 + 2))
            # the two recurrences: a constant decay per head beside a decay per key channel from logits; a decay per head in
            # the delta rule beside one per key channel
            kw, vw = H * dk, H * dv
            C = 2 * kw + vw
            proj = torch.randn(n, C + H, device=dev).to(bf)
            cu = torch.arange(0, n + 1, n // n_seqs, dtype=torch.int32, device=dev)
            seq = torch.arange(n, dtype=torch.int32, device=dev) // (n // n_seqs)
            slots = torch.arange(n_seqs, dtype=torch.int32, device=dev)
            state = torch.zeros(n_seqs + 1, H, dk, dv, device=dev)
            decay = torch.full((H,), 0.97, device=dev)
            zz, zb = torch.randn(n, kw, device=dev), torch.zeros(kw, device=dev)
            scan_io = 2 * n_seqs * H * dk * dv * 4 + n * vw * 4
            row(f"gla_scan, constant decays, silu {label}",
                lambda: ops.gla_scan(proj[:, :kw], proj[:, kw:2 * kw], proj[:, 2 * kw:2 * kw + vw], None, decay, cu, slots, state, H, dk, dv, 1.0),
                bytes_=n * C * 2 + scan_io, flops=4 * n * H * dk * dv)
            row(f"kubedra gla_scan {label}",
                lambda: ops.gla_scan(proj[:, :kw], proj[:, kw:2 * kw], proj[:, 2 * kw:2 * kw + vw], zz, zb, cu, slots, state, H, dk, dv,
                                     dk ** -0.5, 16.0), bytes_=n * (C * 2 + kw * 4) + scan_io, flops=4 * n * H * dk * dv)
            taps = (torch.randn(C, K, device=dev) * 0.5).to(bf)
            memory = torch.zeros(n_seqs + 1, H * dk * dv + (K - 1) * C, device=dev)
            zh, zhb, a_log = torch.randn(n, H, device=dev), torch.zeros(H, device=dev), torch.zeros(H, device=dev)
            row(f"delta_rule, a decay per head {label}",
                lambda: ops.delta_rule(proj, taps, proj[:, C:], zh, zhb, a_log, seq, cu, slots, memory, H, H, dk, dv, dk ** -0.5, 1e-6,
                                       head_decay=True), bytes_=n * (C * 2 + H * 4) + scan_io, flops=6 * n * H * dk * dv)
            row(f"zemezen delta_rule, a decay per key channel {label}",
                lambda: ops.delta_rule(proj, taps, proj[:, C:], zz, zb, a_log, seq, cu, slots, memory, H, H, dk, dv, dk ** -0.5, 1e-6),
                bytes_=n * (C * 2 + kw * 4) + scan_io, flops=6 * n * H * dk * dv)
            o = torch.randn(n, vw, device=dev)
            g = torch.randn(n, vw, device=dev).to(bf)
            row(f"head_norm_gate over all heads at once, sigmoid {label}",
                lambda: ops.head_norm_gate(o, g, torch.ones(vw, device=dev), 1, vw, 1e-5, bf, gate="sigmoid"), bytes_=n * vw * (4 + 2 + 2))
            row(f"zemezen head_norm_gate per head, sigmoid {label}",
                lambda: ops.head_norm_gate(o, g, torch.ones(dv, device=dev), H, dv, 1e-5, bf, gate="sigmoid"), bytes_=n * vw * (4 + 2 + 2))
            # queries and keys normalised over their whole projections beside the norm per head
            qk = torch.randn(n, (nh + 2 * nkv) * hd, device=dev).to(bf)
            row(f"group_rmsnorm (whole query and key projections) {label}",
                lambda: ops.group_rmsnorm(qk[:, :(nh + nkv) * hd], torch.ones((nh + nkv) * hd, device=dev), nh * hd, nkv * hd, 1e-5),
                bytes_=n * (nh + nkv) * hd * 4)
            gq = torch.ones(hd, device=dev)
            row(f"zemezen head_rmsnorm (queries and keys) {label}", lambda: ops.head_rmsnorm(qk[:, :(nh + nkv) * hd], gq, nh, hd, 1e-5, gq, nkv),
                bytes_=n * (nh + nkv) * hd * 4)
            # the two sides of a parallel layer normalised and averaged, beside a branch normalised and added
            a, b = torch.randn(n, W, device=dev), torch.randn(n, W, device=dev)
            row(f"pair_norm_sum {label}", lambda: ops.pair_norm_sum(a, b, ones, ones, 1e-5), bytes_=n * W * 12)
            row(f"kubedra branch_norm_add {label}", lambda: ops.add_normed_branch(xr, ops.NormedBranch(a, ones, 1e-5)), bytes_=n * W * 12)
            # attention over every earlier key with one added to the denominator beside plain attention; the window with
            # learned sinks is the Zemezen path's kernel as it is
            per = ctx if label == "decode" else n
            pages = (per + 63) // 64
            k_pool = torch.randn(n_seqs * pages + 1, nkv, 64, hd, device=dev).to(bf)
            v_pool = torch.randn(n_seqs * pages + 1, nkv, hd, 64, device=dev).to(bf)
            table = torch.arange(n_seqs * pages, dtype=torch.int32, device=dev).reshape(n_seqs, pages)
            starts, news = ([0], [n]) if label == "prefill" else ([ctx - 1] * n_seqs, [1] * n_seqs)
            totals = [s0 + s1 for s0, s1 in zip(starts, news)]
            pos = i32([s0 + i for s0, s1 in zip(starts, news) for i in range(s1)])
            q = qk[:, :nh * hd]
            sinks = torch.zeros(nh, device=dev)
            seen = sum(p + 1 for p in pos.tolist())
            att_bytes = per * n_seqs * nkv * hd * 2 * 2 + n * nh * hd * 4
            for name, kw_ in (("attention, one added to the denominator", dict(sinks=sinks)), ("llama attention", {})):
                plan = AttentionPlan(n_seqs, max(news), max(totals), label == "decode", i32(starts), i32(news),
                                     i32([0] + list(np.cumsum(news))), i32(totals), list(starts), list(news))
                row(f"{name} {label}", lambda: ops.attention(q, k_pool, v_pool, seq, pos, table, nh, nkv, hd, hd ** -0.5, 0, plan=plan, **kw_),
                    bytes_=att_bytes, flops=4 * seen * nh * hd)
            del k_pool, v_pool
            # the router: corrected shares, normalised and scaled weights, beside the softmax over all with groups
            xb = torch.randn(n, W, device=dev).to(bf)
            n_id = z["identity"]
            wr = torch.randn((E + n_id + 7) // 8 * 8, W, device=dev).to(bf)
            corr = torch.randn(E + n_id, device=dev) * 0.01
            row(f"route_topk, corrected shares, normalised {label}",
                lambda: ops.route_topk(xb, wr, None, top, scoring="softmax_all", experts=E + n_id, correction=corr, normalise=True, weight_scale=2.0),
                bytes_=n * W * 2 + (E + n_id) * W * 2, flops=2 * n * (E + n_id) * W)
            row(f"zemezen route_topk, groups {label}", lambda: ops.route_topk(xb, wr[:E], None, top, scoring="softmax_all", groups=z["groups"]),
                bytes_=n * W * 2 + E * W * 2, flops=2 * n * E * W)
        return rows

    out = {}
    for name in sizes:
        z = dict(ZEMEZEN_SIZES[name], identity=4)
        vocab = 32000
        smoe = {"kind": "moe", "expert": {"ff": z["expert_ff"]},
                "router": {"experts": z["experts"], "identity": z["identity"], "top": z["top"], "scale": 2.0}}
        sdense = {"kind": "dense", "ff": z["ff"], "limit": 7.0}
        rot = {"dims": z["rot"], "base": 10000.0, "scaling": {"factor": 4.0, "original": 2048, "fast": 16.0, "slow": 2.0}}
        att = {"heads": z["att_heads"], "kv_heads": z["att_kv"], "dim": z["att_dim"], "vdim": z["att_dim"], "scale": z["att_dim"] ** -0.5, "rot": rot}
        left = {"heads": z["att_heads"], "kv_heads": z["att_kv"], "dim": z["att_dim"], "vdim": z["att_dim"], "scale": z["att_dim"] ** -0.5,
                "mask": {"size": z["window"]}}
        right = {"heads": z["heads"], "kv_heads": z["heads"], "dim": z["key"], "vdim": z["value"], "conv": z["conv"]}
        light = {"heads": z["heads"], "dim": z["key"], "vdim": z["value"], "decay": [1.0 - 2.0 ** -(2 + i % 8) for i in range(z["heads"])]}
        scfg = {"architecture": "Sopalorn", "vocab": vocab, "width": z["width"], "max_positions": 8192, "norm": {"eps": 1e-5},
                "embedding": {"scale": 1.0}, "logit_scale": 1.0, "streams": COPIES,
                "layers": [{"type": "lightning", "mixer": light, "mlp": sdense},
                           {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": smoe},
                           {"type": "attention", "mixer": att, "mlp": sdense},
                           {"type": "attention", "mixer": dict(att, kv_from=2), "mlp": smoe}]}
        moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]},
               "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": z["groups"][0], "keep": z["groups"][1]}}}
        dense = {"kind": "dense", "ff": z["ff"]}
        mix_d = {"heads": z["heads"], "kv_heads": z["heads"], "dim": z["key"], "vdim": z["value"], "conv": z["conv"], "ranks": [64, 64]}
        mix_a = {"heads": z["att_heads"], "kv_heads": z["att_kv"], "dim": z["att_dim"], "vdim": z["att_dim"], "scale": z["att_dim"] ** -0.5,
                 "mask": {"size": z["window"], "keep_first": z["keep"]}, "rot": {"dims": z["rot"], "base": 10000.0}}
        mix_full = dict(mix_a)
        del mix_full["mask"]
        # the closest model here, layer by layer: a recurrence + dense, a delta rule + experts (the parallel layer's windowed
        # attention is the fourth layer's kernel), attention over every key + dense, windowed attention + experts
        zcfg = {"architecture": "Zemezen", "vocab": vocab, "width": z["width"], "max_positions": 8192, "norm": {"eps": 1e-5},
                "layers": [{"type": "channel_delta", "mixer": mix_d, "mlp": dense}, {"type": "channel_delta", "mixer": mix_d, "mlp": moe},
                           {"type": "attention", "mixer": mix_full, "mlp": dense}, {"type": "attention", "mixer": mix_a, "mlp": moe}]}
        point = {}
        for label, cfg_dict in (("sopalorn", scfg), ("zemezen", zcfg)):
            model = Model.random(config_from_dict(cfg_dict), seed=0, dtype="bfloat16", device="cuda:0", on_device=True)
            point[label] = model_points(model, vocab)
            print(f"[bench] {name} {label}: {point[label]}", file=sys.stderr, flush=True)
            del model
            torch.cuda.empty_cache()
        point["kernels"] = kernel_table(z)
        for k, v in point["kernels"].items():
            print(f"[bench] {name} {k}: {v}", file=sys.stderr, flush=True)
        out[name] = point
    first = out[sizes[0]]
    print(json.dumps({"metric": "sopalorn_decode_tokens_per_second", "value": first["sopalorn"]["decode_b8_tok_s"], "unit": "tokens/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "higher_is_better": True, "dtype": "bf16",
                      "data": "synthetic", "vs_baseline": None, "clocks": sampler.stop(),
                      "config": {"model": "Sopalorn, four layers at the sizes named", "batch": 8, "context": ctx, "prefill_tokens": T,
                                 "l2": "flushed between a kernel's timed launches"},
                      "peaks": pk, "sizes": out}))
    return 0


def short_prompt_workload(args, model, cfg, gen, shape_name, dtype_name):
    """The time from a prompt's tokens on the host to its first token on the host, for single prompts
    of random lengths in five ranges: stepped eagerly (the host launches every kernel) and through
    captured steps that prompts of other lengths share (`Model.step(graphs=True)`: a prompt's tokens
    are filled up to the next multiple of 64, a power of two below, and forgotten after the step).
    Median of ten prompts after four that warm up and capture.  Prints its own JSON line."""
    import random
    import torch
    from dotllm_b200 import StepEntry
    rng = random.Random(3)
    out = {}
    for lo, hi in ((20, 32), (65, 128), (193, 256), (449, 512), (961, 1024)):
        cell = {}
        for label, graphs in (("eager_ms", False), ("captured_ms", True)):
            cache = model.new_cache(max_tokens=4096)
            times = []
            for _ in range(14):
                prompt = torch.randint(0, cfg.vocab_size, (rng.randint(lo, hi),), generator=gen).tolist()
                seq = cache.open_sequence()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                first = int(model.step(cache, [StepEntry(seq, prompt)], graphs=graphs).argmax())
                times.append((time.perf_counter() - t0) * 1e3)
                cache.close_sequence(seq)
            assert 0 <= first < cfg.vocab_size
            cell[label] = round(sorted(times[4:])[5], 3)
            del cache
        out[f"{lo}-{hi}"] = cell
    print(json.dumps({"metric": "time to the first token of one short prompt", "model": shape_name, "dtype": dtype_name, "unit": "ms",
                      "prompt_tokens": out, "data": "synthetic: seeded random weights, prompt lengths and token ids"}))
    return 0


def staggered_workload(args, model, cfg, gen, shape_name, dtype_name):
    """`Model.generate` on 64 prompts of 128 tokens whose requests end one by one, five steps apart
    (request i generates 40 + 5 i tokens: 12,640 in all, 355 steps, every batch size from 64 to 1):
    what the loop's ways of stepping cost and give when the batch keeps shrinking.  Three generators,
    each on a cache of its own, each called four times: without graphs; with graphs of a few widths;
    with those and every step started before the host has the tokens of the step before it.  The
    first call of a generator captures its graphs.  Prints its own JSON line."""
    import torch
    from dotllm_b200 import InferenceOptions
    n = 64
    prompts = [torch.randint(0, cfg.vocab_size, (128,), generator=gen).tolist() for _ in range(n)]
    options = [InferenceOptions(temperature=0.0, max_tokens=40 + 5 * i, stop_token_ids=[]) for i in range(n)]
    total = sum(o.max_tokens for o in options)
    out = {}
    for label, use_graphs, ahead in (("eager", False, False), ("graphs", True, False), ("graphs_ahead", True, True)):
        cache = model.new_cache(max_tokens=n * 512, max_sequences=n)
        generator = model.generator(cache=cache, max_batch=n, use_graphs=use_graphs, ahead=ahead)
        seconds = []
        for _ in range(4):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            results = generator.generate(prompts, options)
            torch.cuda.synchronize()
            seconds.append(time.perf_counter() - t0)
            assert sum(r.generated_token_count for r in results) == total
        runner = getattr(cache, "_decode_graphs", None)
        out[label] = {"first_call": round(total / seconds[0], 1), "later_calls": round(total / min(seconds[1:]), 1),
                      "first_call_s": round(seconds[0], 3), "later_call_s": round(min(seconds[1:]), 3),
                      "graphs": len(runner.captured) if runner is not None else 0, "steps_ahead": generator.ahead_steps}
        del generator, cache
    print(json.dumps({"metric": "generate tokens/s while 64 requests end one by one", "model": shape_name, "dtype": dtype_name,
                      "requests": n, "prompt_tokens": 128, "new_tokens": total, "unit": "tokens/s", **out,
                      "data": "synthetic: seeded random weights and token ids; greedy, stop tokens off"}))
    return 0


def unequal_workload(args, model, cache, cfg, gen, pk, shape_name, dtype_name, compute_peak, weight_bytes, prefill_flops):
    """64 prompts with lengths uniform in [16, 2048] in ONE prefill step, then 256 decode steps at batch
    64 (the Llama-3.2-1B-shaped workload).  Prints its own JSON line."""
    import numpy as np
    import torch
    from dotllm_b200 import StepEntry
    from dotllm_b200.kernels import ops
    n_seqs, n_decode = 64, 256
    lens = torch.randint(16, 2049, (n_seqs,), generator=gen).tolist()
    prompts = [np.asarray(torch.randint(0, cfg.vocab_size, (n,), generator=gen)) for n in lens]
    need = sum((n + n_decode + 63) // 64 * 64 for n in lens)
    big = model.new_cache(max_tokens=need, max_sequences=n_seqs) if need > cache.max_tokens else cache
    results = {"prefill_ms": [], "decode_ms": [], "plan_ms": []}
    from dotllm_b200.engine.step import plan_step
    for rep in range(1 + min(args.repeats, 3)):
        seqs = [big.open_sequence() for _ in prompts]
        entries = [StepEntry(s, p) for s, p in zip(seqs, prompts)]
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_host = time.perf_counter()
        a.record()
        logits = model.step(big, entries)
        b.record()
        torch.cuda.synchronize()
        graphs = model.decode_graphs(big)
        tokens = ops.sample(logits).tolist()
        dec = [StepEntry(s, [t]) for s, t in zip(seqs, tokens)]
        lg = graphs.run(dec)
        tok_buf = graphs.token_buffer(n_seqs)
        ops.sample(lg, out=tok_buf)
        torch.cuda.synchronize()
        c, d = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c.record()
        for _ in range(n_decode - 1):
            ops.sample(graphs.run(dec, device_tokens=True), out=tok_buf)
        d.record()
        torch.cuda.synchronize()
        mean_len = sum(s.length for s in seqs) / n_seqs - n_decode / 2
        for s in seqs:
            big.close_sequence(s)
        # what planning alone costs on the host, without the model
        seqs = [big.open_sequence() for _ in prompts]
        t0 = time.perf_counter()
        plan_step([StepEntry(s, p) for s, p in zip(seqs, prompts)], big, cfg.vocab_size, 1 << 30, model.runtime.device)
        plan_ms = (time.perf_counter() - t0) * 1e3
        for s in seqs:
            big.close_sequence(s)
        if rep:                                              # the first round warms up (captures the graph)
            results["prefill_ms"].append(a.elapsed_time(b))
            results["decode_ms"].append(c.elapsed_time(d) / (n_decode - 1))
            results["plan_ms"].append(plan_ms)
    total = sum(lens)
    p_ms, d_ms = min(results["prefill_ms"]), min(results["decode_ms"])
    flops = prefill_flops(total, n_seqs) + cfg.num_hidden_layers * sum(2 * n * n * cfg.q_dim for n in lens)
    step_bytes = weight_bytes + n_seqs * mean_len * big.bytes_per_token()
    print(json.dumps({
        "metric": "unequal batch: prefill tokens/s and decode tokens/s", "model": shape_name, "dtype": dtype_name,
        "sequences": n_seqs, "prompt_tokens": total, "decode_steps": n_decode,
        "prefill": {"value": round(total * 1e3 / p_ms, 1), "ms": round(p_ms, 2), "planning_ms": round(min(results["plan_ms"]), 2),
                    "frac": round(flops / (p_ms * 1e-3) / (compute_peak * 1e12), 4)},
        "decode": {"value": round(n_seqs * 1e3 / d_ms, 1), "ms_per_step": round(d_ms, 4),
                   "roofline_frac": round(step_bytes / (d_ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)},
        "data": "synthetic: seeded random weights, seeded prompt lengths and token ids"}))
    return 0


def cpp_model_tokens_per_second(tmp, folder, cfg, tokens):
    """The one-file C++ float32 model under tests/cpu_reference, compiled here and timed on one prompt."""
    import shutil
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        return None
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from test_cpu_reference import SOURCE, arguments
    exe = tmp / "llama_f32"
    if subprocess.run([cxx, "-O2", "-std=c++17", "-o", str(exe), str(SOURCE)], capture_output=True).returncode != 0:
        return None
    (tmp / "tokens.txt").write_text(" ".join(str(t) for t in tokens))
    res = subprocess.run([str(exe), str(folder / "model.safetensors"), str(tmp / "tokens.txt"), str(tmp / "out.f32"), *arguments(cfg)],
                         capture_output=True, text=True)
    return json.loads(res.stdout)["tokens_per_second"] if res.returncode == 0 else None


def plain_cpu_baseline():
    """The plain implementation (tests/plain_llama.py, float32, PyTorch on the host's cores) timed on the
    tiny test models and on a short prompt through one Llama-3.2-1B-shaped layer stack: the CPU line
    that stands where the reference's own CPU numbers would."""
    import tempfile
    from pathlib import Path
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_llama
    import tiny_models
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.weights import write_random_model
    out = {"impl": "plain-cpu", "threads": torch.get_num_threads(), "cells": {}}
    with tempfile.TemporaryDirectory() as tmp:
        for which, lens, n_new in (("A", tiny_models.TINY_A_PROMPTS, tiny_models.TINY_A_DECODE),
                                   ("B", tiny_models.TINY_B_PROMPTS, tiny_models.TINY_B_DECODE)):
            folder = tiny_models.make_folder(Path(tmp), which, seed=0)
            cfg, weights = plain_llama.read_model_folder(folder)
            prompts = [tiny_models.random_tokens(n, cfg["vocab_size"], 3 + n) for n in lens]
            t0 = time.perf_counter()
            for p in prompts:
                plain_llama.forward(cfg, weights, p)
            prefill_s = time.perf_counter() - t0
            t0 = time.perf_counter()
            for p in prompts:
                plain_llama.greedy_generate(cfg, weights, p, n_new)
            out["cells"][f"tiny_{which}"] = {"prefill_tok_s": round(sum(lens) / prefill_s, 1),
                                             "generate_tok_s_no_cache": round(len(lens) * n_new / (time.perf_counter() - t0), 1)}
            cpp = cpp_model_tokens_per_second(Path(tmp), folder, cfg, prompts[-1])
            if cpp is not None:
                out["cells"][f"tiny_{which}"]["cpp_f32_prefill_tok_s"] = cpp
        one_b = dict(LLAMA_32_1B, num_hidden_layers=2, max_position_embeddings=4096)
        folder = write_random_model(Path(tmp) / "1b", config_from_dict(one_b), seed=0, dtype=torch.bfloat16)
        cfg, weights = plain_llama.read_model_folder(folder)
        prompt = tiny_models.random_tokens(128, cfg["vocab_size"], 9)
        plain_llama.forward(cfg, weights, prompt[:8])
        t0 = time.perf_counter()
        plain_llama.forward(cfg, weights, prompt)
        dt = time.perf_counter() - t0
        out["cells"]["llama_3.2_1b_shape_2_of_16_layers"] = {"prefill_tokens": 128, "seconds": round(dt, 3),
                                                             "prefill_tok_s_2_layers_and_head": round(128 / dt, 1)}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
