#!/usr/bin/env python3
"""Measures generation on one B200: decode tokens a second at batch 8 (the headline), at
batch 1 and 64, and prefill of 2,048 tokens, on the Mistral-7B-v0.3 layer sizes with
random weights and random token ids.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  A step is one decode step of the whole batch.  `value` times K
steps with CUDA events on the launching stream (engine step + token choice; the chosen
tokens stay on the device and feed the next step); `e2e` is the same number through the Python entry point
(`Model.generate`): host token ids in, host token ids out, every step copying its
inputs from pinned host memory and reading its chosen tokens back.  Weights (14.5 GB)
exceed the 126 MB L2, so no L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
            if d.get("bf16_tflops_sustained"):
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0) -> None:
        self.index = index
        self.proc = None
        self.path = None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            self.out.close()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            with open(self.path) as f:
                for line in f:
                    p = [x.strip() for x in line.split(",")]
                    if len(p) < 7:
                        continue
                    try:
                        sm.append(float(p[0])); mx.append(float(p[1]))
                    except ValueError:
                        continue
                    for n, v in zip(names, p[3:7]):
                        if v.lower().startswith("active"):
                            reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg, n_layers):
    """Bytes a decode step reads and FLOPs a prefill does, from the configuration."""
    hs, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nq, nk, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    per_layer_params = (nq + 2 * nk) * hd * hs + hs * nq * hd + 3 * I * hs + 2 * hs
    weight_bytes = 2 * (n_layers * per_layer_params + V * hs + hs)          # layers, head, final norm
    kv_bytes_per_token = n_layers * 2 * nk * hd * 2
    return per_layer_params, weight_bytes, kv_bytes_per_token


def prefill_flops(cfg, n_layers, T):
    hs, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nq, nk, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    lin = 2 * T * ((nq + 2 * nk) * hd * hs + hs * nq * hd + 3 * I * hs)
    attn = 2 * 2 * nq * hd * (T * (T + 1) // 2)                             # causal QK^T and PV
    return n_layers * (lin + attn) + 2 * V * hs


def device_timed_decode(engine, sampler_kernels, prompts, steps, warmup):
    """K decode steps of the whole batch, timed with CUDA events; returns (seconds, context at start)."""
    import torch
    slots = [engine.open() for _ in prompts]
    logits = engine.step(list(zip(slots, prompts)), want="last")
    out = torch.empty(len(prompts), dtype=torch.int32, device=engine.device)
    sampler_kernels.argmax(logits, out)
    toks = out.tolist()
    for _ in range(warmup):
        logits = engine.step([(s, [t]) for s, t in zip(slots, toks)], want="last")
        sampler_kernels.argmax(logits, out)
    ctx0 = engine.length(slots[0])
    entries = [(s, [0]) for s in slots]                  # placeholders: each step takes its tokens from `out`
    rows = list(range(len(slots)))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = engine.kernels.launches
    e0.record()
    for _ in range(steps):
        logits = engine.step(entries, want="last", device_tokens=(out, rows))
        sampler_kernels.argmax(logits, out)
    e1.record()
    torch.cuda.synchronize()
    engine.check()
    launches = engine.kernels.launches - launches0
    for s in slots:
        engine.close(s)
    return e0.elapsed_time(e1) / 1e3, ctx0, launches


def sm_clock_reader():
    """A function that reads the SM clock in MHz (a query only), or None without NVML."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(0)
        return lambda: int(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
    except Exception:
        return None


def steps_after_a_prefill(engine, prompts, n=40):
    """The first `n` decode steps right after a batch's prefill, one by one: the time of each
    (host clock around a synchronised step) and the SM clock read after it.  Shows how long the
    clocks take to come back after the prefill's power draw, which is the difference between the
    device-timed number (taken after warm-up steps) and the one through the entry point."""
    import torch
    read_mhz = sm_clock_reader()
    slots = [engine.open() for _ in prompts]
    logits = engine.step(list(zip(slots, prompts)), want="last")
    out = torch.empty(len(prompts), dtype=torch.int32, device=engine.device)
    engine.kernels.argmax(logits, out)
    torch.cuda.synchronize()
    ms, mhz = [], []
    entries, rows = [(s, [0]) for s in slots], list(range(len(slots)))
    for _ in range(n):
        t0 = time.perf_counter()
        logits = engine.step(entries, want="last", device_tokens=(out, rows))
        engine.kernels.argmax(logits, out)
        torch.cuda.synchronize()
        ms.append(round((time.perf_counter() - t0) * 1e3, 3))
        mhz.append(read_mhz() if read_mhz else None)
    for s in slots:
        engine.close(s)
    prod = [round(a * b / 1e3, 2) for a, b in zip(ms, mhz)] if read_mhz else None      # ms x GHz: clock-free work
    return {"step_ms": ms, "sm_mhz": mhz, "ms_times_ghz": prod}


def run_ours(args):
    import torch
    from braidinfer_b200.api import Model
    from braidinfer_b200.config import preset
    from braidinfer_b200.engine import Engine
    from braidinfer_b200.sampling import SamplingParams

    pk = peaks()
    cfg_dict = preset("mistral_7b_v03")
    full_layers = cfg_dict["num_hidden_layers"]
    if args.quick and not args.layers:
        args.layers = 4
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    n_layers = cfg_dict["num_hidden_layers"]
    B, prompt_len, gen_len, ctx_len = args.batch, 2048, 256, 4096
    steps, warmup = args.steps, max(3, args.warmup)
    t0 = time.time()
    cache_seqs = B if args.quick else 64
    engine = Engine.from_random(cfg_dict, seed=0, dtype="bfloat16", on_device=True, max_tokens=cache_seqs * ctx_len,
                                max_slots=64, use_graphs=not args.no_graphs, verbose=True)
    cfg = engine.config
    model = Model(engine, max_batch=64)
    g = torch.Generator().manual_seed(0)

    def prompts_for(b, n=prompt_len):
        return [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for _ in range(b)]

    _, weight_bytes, kv_per_tok = model_numbers(cfg, n_layers)

    # ---- prefill of 2,048 tokens (one sequence), timed on the device
    p1 = prompts_for(1)
    times = []
    for i in range(3 + 3):
        s = engine.open()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.step([(s, p1[0])], want="last")
        e1.record()
        torch.cuda.synchronize()
        engine.close(s)
        if i >= 3:
            times.append(e0.elapsed_time(e1))
    pre_ms = statistics.median(times)
    pre_flops = prefill_flops(cfg, n_layers, prompt_len)
    prefill = {"value": prompt_len / (pre_ms / 1e3), "tokens": prompt_len, "ms": pre_ms,
               "frac": pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), "unit": "tokens/s",
               "peak": f"{pk['bf16_tflops']} TFLOP/s bf16, {pk['source']}"}
    if pk.get("bf16_tflops_sustained"):
        # the step is timed as the median of back-to-back repeats, under the power cap: the library's
        # product measured the same way is the second yardstick
        prefill["frac_of_sustained"] = pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12)
    if not args.quick:
        # the same prompt by itself, as one arrives in use: half a second of rest before each of three
        # repeats, so that the step starts below the power cap (the burst peak was measured so)
        rested = []
        for i in range(3):
            time.sleep(0.5)
            s = engine.open()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step([(s, p1[0])], want="last")
            e1.record()
            torch.cuda.synchronize()
            engine.close(s)
            rested.append(e0.elapsed_time(e1))
        r_ms = statistics.median(rested)
        prefill["after_rest"] = {"ms": r_ms, "value": prompt_len / (r_ms / 1e3),
                                 "frac": pre_flops / (r_ms / 1e3) / (pk["bf16_tflops"] * 1e12)}

    # ---- decode at the headline batch, device-timed, with clocks sampled meanwhile
    with ClockSampler() as cs:
        secs, ctx0, launches = device_timed_decode(engine, engine.kernels, prompts_for(B), steps, warmup)
    clocks = cs.summary()
    value = B * steps / secs
    ms_per_step = secs / steps * 1e3
    avg_ctx = ctx0 + steps / 2
    step_bytes = weight_bytes + B * avg_ctx * kv_per_tok + B * cfg.hidden_size * 2
    achieved = step_bytes / (secs / steps) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "peak_source": pk["source"], "bytes_per_step": step_bytes}

    # ---- the same through the Python entry point: host tokens in, host tokens out
    e2e = None
    if not args.quick:
        outs = model.generate(prompts_for(B), SamplingParams.greedy(), stop_tokens=(),
                              max_new_tokens=min(steps, gen_len) + 1)
        st = model.last_stats
        e2e = {"value": st.decode_tokens / st.decode_seconds if st.decode_seconds > 0 else 0.0, "unit": "tokens/s",
               "h2d_bytes_per_step": engine.packer.h2d_bytes_last, "d2h_bytes_per_step": B * 4,
               "prefill_tokens_per_s": st.prompt_tokens / st.prefill_seconds if st.prefill_seconds > 0 else 0.0}

    # ---- other batch sizes, temperature sampling, and the steps right after a prefill
    points = {}
    after_prefill = None
    for b in (() if args.quick else (1, 64)):
        k = min(steps, 64)
        s2, _, _ = device_timed_decode(engine, engine.kernels, prompts_for(b), k, warmup)
        points[f"decode_b{b}"] = b * k / s2
    if not args.quick:
        warm = SamplingParams(temperature=0.8, seed=1)
        model.generate(prompts_for(B, 64), warm, stop_tokens=(), max_new_tokens=4)      # the sampling kernel's first call
        model.generate(prompts_for(B), warm, stop_tokens=(), max_new_tokens=min(steps, gen_len) + 1)
        st = model.last_stats
        points["decode_b8_temperature"] = st.decode_tokens / st.decode_seconds if st.decode_seconds > 0 else 0.0
        # a short prompt by itself (time to its first logits): such steps go through CUDA graphs from the
        # third step of a shape on
        short = prompts_for(1, 64)[0]
        ms = []
        for i in range(6):
            slot = engine.open()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step([(slot, short)], want="last")
            e1.record()
            torch.cuda.synchronize()
            engine.close(slot)
            ms.append(e0.elapsed_time(e1))
        points["prompt_64_tokens_ms"] = statistics.median(ms[3:])
        after_prefill = steps_after_a_prefill(engine, prompts_for(B))

    line = {
        "metric": "decode tokens/s at batch 8, Mistral-7B-v0.3 sizes, bf16 (also batch 1, 64; prefill of 2,048 tokens)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02) seed 0, uniform random token ids",
        "impl": "ours",
        "config": {"model": "Mistral-7B-v0.3 sizes", "layers": n_layers, "layers_of_full_model": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "rope_theta": cfg.rope_theta, "rms_eps": cfg.rms_norm_eps, "global_batch": B,
                   "seq_len": ctx_len, "prompt_len": prompt_len, "context_at_timing": int(avg_ctx),
                   "cache_tokens": cache_seqs * ctx_len, "parallelism": "single GPU",
                   "l2": "inputs (14.5 GB of weights) exceed L2; no flush"},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "prefill": prefill, "roofline": roofline,
        "points": points, "after_prefill": after_prefill, "setup_seconds": time.time() - t0,
    }
    print(json.dumps(line))
    return 0


def run_other_size(args):
    """The other sizes the measurements are quoted on:
    `mistral_7b_v01`: sliding window 4096, context 8192, batch 8, prompts of 6,000-8,000 tokens;
    `mistral_nemo_12b`: head_dim 128 with hidden 5120, vocabulary 131072, context 16384, batch 16, prompts of
    512-8,192 tokens.  One JSON line with the same keys as the default run: `value` is decode tokens a second
    timed on the device, `prefill` the batch's prompt step, `roofline` the bytes a decode step has to read
    (every weight once, and the keys and values that each sequence's window still sees) over its time,
    `e2e` the same batch through `Model.generate`."""
    import random
    import torch
    from braidinfer_b200.api import Model
    from braidinfer_b200.config import preset
    from braidinfer_b200.engine import Engine
    from braidinfer_b200.sampling import SamplingParams
    pk = peaks()
    rng = random.Random(0)
    g = torch.Generator().manual_seed(0)
    if args.preset == "mistral_7b_v01":
        B, ctx, lens = 8, 8192, [rng.randint(6000, 8000) for _ in range(8)]
    else:
        B, ctx, lens = 16, 16384, [rng.randint(512, 8192) for _ in range(16)]
    cfg_dict = preset(args.preset)
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    n_layers = cfg_dict["num_hidden_layers"]
    t0 = time.time()
    engine = Engine.from_random(cfg_dict, seed=0, dtype="bfloat16", on_device=True, max_tokens=B * ctx, max_slots=B)
    cfg = engine.config
    model = Model(engine, max_batch=B)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    steps, warmup = min(args.steps, 128), max(3, args.warmup)
    _, weight_bytes, kv_per_tok = model_numbers(cfg, n_layers)

    # the batch's prompts in one step (unequal lengths), timed on the device after one warm-up run
    pre_ms = None
    for i in range(2):
        slots = [engine.open() for _ in prompts]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.step(list(zip(slots, prompts)), want="last")
        e1.record()
        torch.cuda.synchronize()
        pre_ms = e0.elapsed_time(e1)
        for sl in slots:
            engine.close(sl)
    window = cfg.sliding_window
    lin = 2 * ((cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim * cfg.hidden_size
               + cfg.hidden_size * cfg.num_attention_heads * cfg.head_dim + 3 * cfg.intermediate_size * cfg.hidden_size)
    att = sum(sum(min(p + 1, window) if window else p + 1 for p in range(n)) for n in lens) * 4 * cfg.num_attention_heads * cfg.head_dim
    pre_flops = n_layers * (lin * sum(lens) + att) + 2 * cfg.vocab_size * cfg.hidden_size * B
    prefill = {"value": sum(lens) / (pre_ms / 1e3), "tokens": sum(lens), "ms": pre_ms, "unit": "tokens/s",
               "frac": pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12),
               "peak": f"{pk['bf16_tflops']} TFLOP/s bf16, {pk['source']}"}

    with ClockSampler() as cs:
        secs, _, launches = device_timed_decode(engine, engine.kernels, prompts, steps, warmup)
    clocks = cs.summary()
    seen = [min(n + warmup + steps / 2, window) if window else n + warmup + steps / 2 for n in lens]
    step_bytes = weight_bytes + sum(seen) * kv_per_tok + B * cfg.hidden_size * 2
    achieved = step_bytes / (secs / steps) / 1e9
    outs = model.generate(prompts, SamplingParams.greedy(), stop_tokens=(), max_new_tokens=steps + 1)
    st = model.last_stats
    engine.check()
    print(json.dumps({
        "metric": f"decode tokens/s at batch {B}, {args.preset} sizes, bf16 (unequal prompts; also their prefill)",
        "value": B * steps / secs, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": secs / steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02) seed 0, uniform random token ids", "impl": "ours",
        "config": {"model": args.preset, "layers": n_layers, "layers_of_full_model": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "sliding_window": window, "global_batch": B, "seq_len": ctx, "prompt_tokens": sum(lens),
                   "prompt_len_min": min(lens), "prompt_len_max": max(lens), "parallelism": "single GPU",
                   "weights_gb": round(engine.weight_bytes / 1e9, 2), "cache_gb": round(engine.cache.nbytes() / 1e9, 2),
                   "l2": "inputs (weights) exceed L2; no flush"},
        "e2e": {"value": st.decode_tokens / st.decode_seconds if st.decode_seconds > 0 else 0.0, "unit": "tokens/s",
                "h2d_bytes_per_step": engine.packer.h2d_bytes_last, "d2h_bytes_per_step": B * 4,
                "prefill_tokens_per_s": st.prompt_tokens / st.prefill_seconds if st.prefill_seconds > 0 else 0.0},
        "gpu_launches": launches, "clocks": clocks, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "peak_source": pk["source"], "bytes_per_step": step_bytes},
        "setup_seconds": time.time() - t0}))
    return 0


def run_sweep(args):
    """Decode at batch 1, 8, 64 over contexts of 512 to 32,768 tokens and prefill of 512 to 16,384
    tokens, on the default sizes: one JSON line with time, achieved bandwidth or FLOP rate, and the
    fraction of the peak, for every point.  Not the contract's line."""
    import torch
    from braidinfer_b200.config import preset
    from braidinfer_b200.engine import Engine
    pk = peaks()
    cfg_dict = preset("mistral_7b_v03")
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    n_layers = cfg_dict["num_hidden_layers"]
    engine = Engine.from_random(cfg_dict, seed=0, dtype="bfloat16", on_device=True, max_tokens=64 * (8192 + 128),
                                max_slots=64, verbose=True)
    cfg = engine.config
    g = torch.Generator().manual_seed(0)
    _, weight_bytes, kv_per_tok = model_numbers(cfg, n_layers)
    decode, prefill = [], []
    for T in (512, 2048, 8192, 16384):
        p = torch.randint(0, cfg.vocab_size, (T,), generator=g).tolist()
        times = []
        for i in range(5):
            s = engine.open()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step([(s, p)], want="last")
            e1.record()
            torch.cuda.synchronize()
            engine.close(s)
            if i >= 2:
                times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        fl = prefill_flops(cfg, n_layers, T)
        prefill.append({"tokens": T, "ms": round(ms, 3), "tokens_per_s": round(T / ms * 1e3),
                        "tflops": round(fl / ms / 1e9, 1), "frac": round(fl / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 3)})
    for ctx in (512, 2048, 8192, 32768):
        for b in (1, 8, 64):
            if b * (ctx + 128) > engine.max_tokens:
                continue
            prompts = [torch.randint(0, cfg.vocab_size, (ctx,), generator=g).tolist() for _ in range(b)]
            steps = 48
            secs, ctx0, _ = device_timed_decode(engine, engine.kernels, prompts, steps, 24)    # clocks settle after the prompts
            step_bytes = weight_bytes + b * (ctx0 + steps / 2) * kv_per_tok
            gbs = step_bytes / (secs / steps) / 1e9
            decode.append({"batch": b, "context": ctx, "ms_per_step": round(secs / steps * 1e3, 3),
                           "tokens_per_s": round(b * steps / secs, 1), "gb_per_s": round(gbs),
                           "frac": round(gbs / pk["hbm_gbs"], 3)})
    print(json.dumps({"metric": "sweep over batch, context and prompt length, Mistral-7B-v0.3 sizes, bf16", "impl": "ours",
                      "layers": n_layers, "peaks": pk, "prefill": prefill, "decode": decode}))
    return 0


def run_timeline(args):
    """Where a decode step's time goes: one CUDA-graph step of the default sizes under the torch
    profiler (device activity only), printed as one JSON line: for the kernels of one layer in the
    middle of the step, the time from the end of the kernel before to the end of this one (kernels
    overlap their predecessors' tails through programmatic dependent launch, so durations would
    count time twice).  Not the contract's line."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from braidinfer_b200.config import preset
    from braidinfer_b200.engine import Engine
    cfg_dict = preset("mistral_7b_v03")
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    B = args.batch
    engine = Engine.from_random(cfg_dict, seed=0, dtype="bfloat16", on_device=True, max_tokens=B * 4096, max_slots=B,
                                verbose=True)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, engine.config.vocab_size, (2048,), generator=g).tolist() for _ in range(B)]
    slots = [engine.open() for _ in prompts]
    engine.step(list(zip(slots, prompts)))
    for _ in range(8):
        engine.step([(s, [5]) for s in slots])
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(2):
            engine.step([(s, [5]) for s in slots])
        torch.cuda.synchronize()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "trace.json")
        prof.export_chrome_trace(path)
        with open(path) as f:
            ev = [e for e in json.load(f)["traceEvents"] if e.get("cat") == "kernel"]
    ev.sort(key=lambda e: e["ts"])
    first = [i for i, e in enumerate(ev) if "embed" in e["name"]][-1]
    step = ev[first:]
    span = step[-1]["ts"] + step[-1]["dur"] - step[0]["ts"]
    # a layer = from one attention kernel to the next
    att = [i for i, e in enumerate(step) if "attn_" in e["name"] and "combine" not in e["name"]]
    mid = len(att) // 2
    start, per_layer = att[mid], att[mid + 1] - att[mid]
    rows, prev_end = [], step[start - 1]["ts"] + step[start - 1]["dur"]
    for e in step[start:start + per_layer]:
        end = e["ts"] + e["dur"]
        rows.append({"kernel": e["name"].split("(")[0][:48], "until_its_end_us": round(end - prev_end, 2)})
        prev_end = end
    print(json.dumps({"metric": "one decode step under the profiler, Mistral-7B-v0.3 sizes, bf16", "impl": "ours",
                      "batch": B, "kernels_in_step": len(step), "step_us": round(span, 1), "kernels_a_layer": per_layer,
                      "layer_us": round(sum(r["until_its_end_us"] for r in rows), 1), "one_layer": rows}))
    return 0


def run_prompt_timeline(args):
    """Where a prompt's time goes, by prompt length: for each length given (--prompt-timeline 256,512,...), one prompt
    step of the default layer sizes (8 layers unless --layers says otherwise) under the torch profiler, and for the
    kernels of one layer in the middle the time from the end of the kernel before to the end of this one, as
    run_timeline does for a decode step.  Lengths up to 256 go through a CUDA graph from the third step on, as they
    do in generation.  One JSON line a length.  Not the contract's line."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from braidinfer_b200.config import preset
    from braidinfer_b200.engine import Engine
    cfg_dict = preset("mistral_7b_v03")
    cfg_dict["num_hidden_layers"] = args.layers or 8
    lengths = [int(t) for t in args.prompt_timeline.split(",")]
    engine = Engine.from_random(cfg_dict, seed=0, dtype="bfloat16", on_device=True,
                                max_tokens=2 * max(max(lengths), 4096), max_slots=2, verbose=True)
    c = engine.config
    per_token = 2 * (c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
                     + c.num_attention_heads * c.head_dim * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
    pk = peaks()
    g = torch.Generator().manual_seed(0)
    for T in lengths:
        prompt = torch.randint(0, c.vocab_size, (T,), generator=g).tolist()
        for _ in range(3):
            s = engine.open()
            engine.step([(s, prompt)])
            engine.close(s)
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            s = engine.open()
            engine.step([(s, prompt)])
            engine.close(s)
            torch.cuda.synchronize()
        with tempfile.TemporaryDirectory() as d:
            path = os.path.join(d, "trace.json")
            prof.export_chrome_trace(path)
            with open(path) as f:
                ev = [e for e in json.load(f)["traceEvents"] if e.get("cat") == "kernel"]
        ev.sort(key=lambda e: e["ts"])
        att = [i for i, e in enumerate(ev) if "attn_" in e["name"] and "combine" not in e["name"]]
        mid = len(att) // 2
        start, per_layer = att[mid], att[mid + 1] - att[mid]
        rows, prev_end = [], ev[start - 1]["ts"] + ev[start - 1]["dur"]
        for e in ev[start:start + per_layer]:
            end = e["ts"] + e["dur"]
            rows.append({"kernel": e["name"].split("(")[0][:48], "until_its_end_us": round(end - prev_end, 2)})
            prev_end = end
        layer_us = sum(r["until_its_end_us"] for r in rows)
        print(json.dumps({"metric": "one prompt step under the profiler, Mistral-7B-v0.3 layer sizes, bf16", "impl": "ours",
                          "tokens": T, "layers": cfg_dict["num_hidden_layers"], "layer_us": round(layer_us, 1),
                          "layer_flops_over_burst_peak_us": round(T * per_token / (pk["bf16_tflops"] * 1e12) * 1e6, 1),
                          "frac_of_burst": round(T * per_token / (pk["bf16_tflops"] * 1e12) * 1e6 / layer_us, 3),
                          "step_us": round(ev[-1]["ts"] + ev[-1]["dur"] - ev[0]["ts"], 1), "one_layer": rows}), flush=True)
    return 0


def run_chain(args):
    """What the chain of dependent kernels of a decode step costs, at the default sizes: products alone chained to
    themselves, and product + reducer pairs, each six times over distinct weights in one CUDA graph, timed with
    events (L2 flushed before each replay).  With BRAIDINFER_TRACE=1 in the environment the library is built with
    time stamps at the phase boundaries of the product and of the reduce + norm kernel (csrc/trace.cuh); the
    line then also carries, for the o product + reducer chain, the median over CTAs of every stamp, in
    microseconds from the chain's first entry.  Not the contract's line."""
    import ctypes
    import numpy as np
    import torch
    from braidinfer_b200.csrc import build
    from braidinfer_b200.csrc.api import get_kernels, interleave_gate_up
    K = get_kernels(verbose=True)
    dev, B = "cuda", args.batch
    hs, I, nq, nk, hd, NL = 4096, 14336, 32, 8, 128, 6
    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *sh: (torch.randn(*sh, device=dev, generator=g) * 0.02).bfloat16()
    W = {"qkv": [rn((nq + 2 * nk) * hd, hs) for _ in range(NL)], "o": [rn(hs, nq * hd) for _ in range(NL)],
         "gate_up": [interleave_gate_up(rn(I, hs), rn(I, hs)) for _ in range(NL)], "down": [rn(hs, I) for _ in range(NL)]}
    X = {"qkv": rn(B, hs), "o": rn(B, nq * hd), "gate_up": rn(B, hs), "down": rn(B, I)}
    wn = torch.ones(hs, device=dev, dtype=torch.bfloat16)
    h = torch.zeros(B, hs, device=dev)
    out = torch.empty(B, hs, device=dev, dtype=torch.bfloat16)
    act = torch.empty(B, I, device=dev, dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, device=dev, dtype=torch.uint8)

    def product_only(name):
        def f(l):
            K.gemm_tc_partial(X[name], W[name][l])
            K.pending_partial = None
        return f

    def with_reducer(name):
        def f(l):
            p = K.gemm_tc_partial(X[name], W[name][l])
            if name == "gate_up":
                K.streamk_reduce(p, act, swiglu=True)
            else:
                K.streamk_reduce_norm(p, h, wn, out, 1e-5)
        return f

    def graph_of(fn):
        body = lambda: [fn(l) for l in range(NL)]
        body()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            body()
        K.pending_partial = None
        return gr

    def timed(gr, reps=20):
        ts = []
        for _ in range(reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); gr.replay(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / NL)
        return round(statistics.median(ts), 2)

    pk = peaks()
    res = {}
    for name in ("o", "qkv", "down", "gate_up"):
        ideal = W[name][0].numel() * 2 / (pk["hbm_gbs"] * 1e3)
        res[name] = {"bytes_over_bandwidth_us": round(ideal, 2), "product_alone_us": timed(graph_of(product_only(name))),
                     "product_and_reducer_us": timed(graph_of(with_reducer(name)))}
    line = {"metric": "chains of decode-step kernels, Mistral-7B-v0.3 layer sizes, bf16", "impl": "ours", "batch": B,
            "peaks": pk, "per_kernel_or_pair": res}
    if build.trace_build():
        gr = graph_of(with_reducer("o"))
        for _ in range(2):
            flush.zero_(); gr.replay()
        traces = {}
        for kname, ctas, names in (("gemm_tc", 160, ["entry", "set_up", "ring_asked", "wait_over", "first_stage_full",
                                                     "last_accumulator", "epilogue_done", "all_done"]),
                                   ("reduce_norm", 64, ["entry", "before_wait", "wait_over", "loaded_and_added",
                                                        "block_sum_done", "stored"])):
            read = getattr(K.lib, f"braid_{kname}_trace_read")
            buf = (ctypes.c_ulonglong * (64 * ctas * 8))()
            read(buf, 1)                                   # forget the warm-up launches
            traces[kname] = (read, buf, ctas, names)
        flush.zero_()
        torch.cuda.synchronize()
        gr.replay()
        torch.cuda.synchronize()
        t0, table = None, {}
        for kname, (read, buf, ctas, names) in traces.items():
            read(buf, 0)
            t = np.frombuffer(buf, dtype=np.uint64).reshape(64, ctas, 8).astype(np.float64)
            if t0 is None:
                t0 = t[0, :, 0][t[0, :, 0] > 0].min()
            rows = []
            for l in range(NL):
                ok = t[l, :, 0] > 0
                if ok.any():
                    rows.append({n: round(float(np.median(t[l, ok, i]) - t0) / 1e3, 2) for i, n in enumerate(names)})
            table[kname] = rows
        line["trace_o_product_and_reducer_us"] = table
    print(json.dumps(line))
    return 0


def run_reference(args):
    print(json.dumps({"impl": "reference", "unavailable":
                      "mcelrath/braidinfer is Rust + HIP for AMD RDNA3: pip finds neither setup.py nor pyproject.toml, "
                      "and this image has no cargo, rustc, hipcc or ROCm"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    ap.add_argument("--quick", action="store_true",
                    help="a small case for profilers: 4 layers unless --layers says otherwise, a cache for this batch "
                         "only, no batch-1/64 points and no end-to-end run; the number it prints is not a bench value")
    ap.add_argument("--no-graphs", action="store_true", help="launch every step kernel by kernel")
    ap.add_argument("--preset", default="mistral_7b_v03",
                    choices=["mistral_7b_v03", "mistral_7b_v01", "mistral_nemo_12b"],
                    help="the default is the contract's run; the other two print their own line (see run_other_size)")
    ap.add_argument("--sweep", action="store_true",
                    help="decode over batch and context, prefill over prompt length; prints its own line (see run_sweep)")
    ap.add_argument("--chain", action="store_true",
                    help="what chains of decode-step kernels cost, with phase time stamps under BRAIDINFER_TRACE=1 "
                         "(see run_chain)")
    ap.add_argument("--prompt-timeline", default="", metavar="T1,T2,...",
                    help="a prompt step of each length under the torch profiler: a layer's kernels with their share "
                         "(see run_prompt_timeline)")
    ap.add_argument("--timeline", action="store_true",
                    help="one decode step under the torch profiler: a layer's kernels with their share (see run_timeline)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.sweep:
        return run_sweep(args)
    if args.prompt_timeline:
        return run_prompt_timeline(args)
    if args.timeline:
        return run_timeline(args)
    if args.chain:
        return run_chain(args)
    if args.preset != "mistral_7b_v03":
        return run_other_size(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
