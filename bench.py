#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second, prefill, roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--shape NAME]
                    [--workload decode|serve|tufirax|vipelix|tibepel|tugodra] [--impl ours|reference]

The default run has the layer sizes of Llama-3.1-8B (32 layers, hidden 4096, 32 query heads,
8 key/value heads of 128, MLP 14336, vocabulary 128256, llama3 rotary scaling) with random
bfloat16 weights: a batch of 8 requests decodes after 2,048-token prompts (context limit 4096).
A "step" is one decode step of the whole batch.  One JSON line is printed:

  value        decoded tokens per second of K steps, timed on the device with CUDA events
  e2e          the same through the Python entry point (LLM.add_request / LLM.step): every step
               copies its metadata from pinned host memory and reads the sampled ids back
  prefill      one 2,048-token prompt: tokens per second, milliseconds, fraction of the bf16 peak
  roofline     bytes a decode step has to read (every weight once + the live requests' cache)
               over its time, against the measured copy bandwidth
  points       decode tokens per second at batch 1 and 64 with their fractions of the HBM roofline,
               the end-to-end figure at batch 64, and the output tokens per second of the continuous
               batching workload at Qwen2.5-7B sizes (64 requests, prompts 128..4,096, 256 tokens each)

The reference arm (--impl reference) reports that the reference cannot be installed here: it is
a Rust workspace built with maturin and cargo, neither of which exists in this image.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA31_8B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
    "vocab_size": 128256, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "attention_bias": False, "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "bfloat16",
}
QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "hidden_size": 3584, "num_hidden_layers": 28,
    "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 18944,
    "vocab_size": 152064, "max_position_embeddings": 32768, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "bfloat16", "use_sliding_window": False,
}
QWEN25_32B = {
    "architectures": ["Qwen2ForCausalLM"], "hidden_size": 5120, "num_hidden_layers": 64,
    "num_attention_heads": 40, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 27648,
    "vocab_size": 152064, "max_position_embeddings": 32768, "rms_norm_eps": 1e-5, "rope_theta": 1000000.0,
    "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "bfloat16", "use_sliding_window": False,
}
# name -> (config.json keys, prompt length, context length) of the benchmark configurations
SHAPES = {"llama-3.1-8b": (LLAMA31_8B, 2048, 4096), "qwen2.5-7b": (QWEN25_7B, 2048, 8192),
          "qwen2.5-32b": (QWEN25_32B, 1024, 4096)}
PREFILL_TOKENS = 2048
PUBLISHED_BASELINE = None     # the reference published nothing for this model, precision or hardware


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def ensure_built():
    """Compile whatever kernel library is missing before anything is timed (a library is otherwise
    compiled when a step first needs it, which may be inside a timed region)."""
    from concurrent.futures import ThreadPoolExecutor

    from rvllm_b200.kernels import build as kb
    from rvllm_b200.kernels.variants import all_variants
    jobs = all_variants()
    with ThreadPoolExecutor(max_workers=8) as pool:
        list(pool.map(lambda j: kb.compile_library(j[0], j[1]), jobs))


def weight_bytes_per_step(cfg, layers, el=2):
    """Every weight a decode step uses once: the layers, the final norm and the LM head (the
    embedding table is only gathered from)."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (q + 2 * kv) * H + H * q + 2 * I * H + H * I + 2 * H
    return (layers * per_layer + H + V * H) * el


def kv_bytes_per_token(cfg, layers, el=2):
    return layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * el


def prefill_flops(cfg, layers, T):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    gemm = 2 * T * ((q + 2 * kv) * H + H * q + 2 * I * H + H * I)
    attn = 4 * q * T * T / 2
    return layers * (gemm + attn) + 2 * V * H


def run_ours(args):
    import torch

    from rvllm_b200 import LLM, SamplingParams, config_from_dict
    from rvllm_b200.engine import StepEntry
    from rvllm_b200.kernels.library import COUNTERS

    peaks = measured_peaks()
    shape, PROMPT_LEN, CONTEXT_LEN = SHAPES[args.shape]
    cfg_dict = dict(shape)
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers is None:
        args.layers = full_layers
    cfg_dict["num_hidden_layers"] = args.layers
    config = config_from_dict(cfg_dict)
    # the headline batch first (a fresh cache pool, as in a run without the points), then the others
    batches = [args.batch] + sorted({1, 64} - {args.batch}) if not args.no_points else [args.batch]
    max_b = max(batches)
    pages_per_req = CONTEXT_LEN // 16
    llm = LLM(config=config, random_weights=True, seed=0, dtype="bfloat16", block_size=16,
              num_blocks=max_b * pages_per_req + 8, max_model_len=CONTEXT_LEN, max_num_seqs=max_b,
              max_num_batched_tokens=max(2048, max_b), enforce_eager=args.eager)
    runner = llm.engine.runner
    kernels = llm.engine.kernels
    gen = torch.Generator().manual_seed(0)
    V = cfg_dict["vocab_size"]

    def prompts_for(b):
        return [torch.randint(0, V, (PROMPT_LEN,), generator=gen).tolist() for _ in range(b)]

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---- prefill of one 2,048-token prompt --------------------------------------------------------
    p = torch.randint(0, V, (PREFILL_TOKENS,), generator=gen).tolist()
    for _ in range(max(1, min(args.warmup, 3))):
        runner.step([StepEntry("warm", p, [PREFILL_TOKENS - 1])])
        runner.finish("warm")
    torch.cuda.synchronize()
    times = []
    for _ in range(3):
        a, b = ev(), ev()
        a.record()
        runner.step([StepEntry("pf", p, [PREFILL_TOKENS - 1])])
        b.record()
        torch.cuda.synchronize()
        runner.finish("pf")
        times.append(a.elapsed_time(b))
    pf_ms = min(times)
    pf_flops = prefill_flops(cfg_dict, args.layers, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / (pf_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 3),
               "frac": round(pf_flops / (pf_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}

    # ---- decode: device-timed steps through the step function ----------------------------------------
    def decode_device(b, steps, warmup, sample_clocks=False):
        ids = [f"d{b}_{i}" for i in range(b)]
        for rid, pr in zip(ids, prompts_for(b)):
            runner.step([StepEntry(rid, pr, [])])
        toks = [1] * b
        for _ in range(warmup):
            runner.step([StepEntry(r, [t], [0]) for r, t in zip(ids, toks)])
        torch.cuda.synchronize()
        clocks = ClockSampler()
        if sample_clocks:
            clocks.start()
            time.sleep(0.2)
        COUNTERS['launches'] = 0
        a, e = ev(), ev()
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):
            logits = runner.step([StepEntry(r, [t], [0]) for r, t in zip(ids, toks)])
        e.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(e) / steps
        launches = COUNTERS['launches']
        ck = clocks.stop() if sample_clocks else None
        ctx = PROMPT_LEN + warmup + steps // 2
        for rid in ids:
            runner.finish(rid)
        return ms, ctx, launches, ck

    # ---- decode end to end through the entry point ------------------------------------------------
    def decode_e2e(b, steps, warmup):
        sp = SamplingParams(temperature=0.0, max_tokens=warmup + steps + b + 16, ignore_eos=True)   # prompts enter one per step
        for pr in prompts_for(b):
            llm.add_request(pr, sp)
        while llm.scheduler.waiting or any(r.remaining > 1 for r in llm.scheduler.running):
            llm.step()
        for _ in range(warmup):
            llm.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            llm.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        h2d = runner.last_h2d_bytes
        for r in list(llm.scheduler.running):
            llm.scheduler.abort(r.req_id)
        return b * steps / dt, h2d, b * 4

    def hbm_gbs(b, ms, ctx):
        """Bytes a decode step of b requests has to read (weights once, the requests' cache) over its time."""
        step_bytes = weight_bytes_per_step(cfg_dict, args.layers) + b * ctx * kv_bytes_per_token(cfg_dict, args.layers)
        return step_bytes / (ms / 1e3) / 1e9

    points = {}
    main = None
    for b in batches:
        ms, ctx, launches, ck = decode_device(b, args.steps, args.warmup, sample_clocks=(b == args.batch))
        tps = b / (ms / 1e3)
        if b != args.batch or b in (1, 64):
            points[f"decode_b{b}"] = round(tps, 1)
            points[f"decode_b{b}_hbm_frac"] = round(hbm_gbs(b, ms, ctx) / peaks["hbm_gbs"], 4)
        if b == args.batch:
            main = (ms, ctx, launches, ck, tps)
    ms, ctx, launches, ck, tps = main
    e2e_tps, h2d, d2h = decode_e2e(args.batch, args.steps, args.warmup)
    if 64 in batches and args.batch != 64:
        points["e2e_b64"] = round(decode_e2e(64, args.steps, args.warmup)[0], 1)
    achieved = hbm_gbs(args.batch, ms, ctx)
    if not args.no_points and args.shape == "llama-3.1-8b" and args.layers == full_layers:
        # continuous batching at Qwen2.5-7B sizes (64 requests, prompts 128..4,096, 256 tokens each, 2,048 tokens
        # a step): output tokens per second, measured with a model of its own after this one is gone
        del runner, kernels
        llm = None
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        try:
            sv = serve_workload("qwen2.5-7b", None, 64, 256, 2048, args.eager)
            points["serve_qwen2.5-7b_output_tok_s"] = sv["value"]
            points["serve_qwen2.5-7b_seconds"] = sv["seconds"]
        except Exception as exc:     # the decode line stands on its own
            points["serve_qwen2.5-7b_output_tok_s"] = None
            points["serve_error"] = f"{type(exc).__name__}: {exc}"[:200]
    line = {
        "metric": f"decode tokens/s ({args.shape} layer sizes, bf16, random weights, {PROMPT_LEN}-token prompts)",
        "value": round(tps, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None if PUBLISHED_BASELINE is None else round(tps / PUBLISHED_BASELINE, 3),
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "impl": "ours",
        "config": {"model": f"{args.shape}-shape", "layers": args.layers, "layers_full": full_layers,
                   "hidden": cfg_dict["hidden_size"], "heads": cfg_dict["num_attention_heads"],
                   "kv_heads": cfg_dict["num_key_value_heads"], "head_dim": cfg_dict["head_dim"],
                   "intermediate": cfg_dict["intermediate_size"], "vocab": cfg_dict["vocab_size"], "global_batch": args.batch, "prompt_len": PROMPT_LEN, "seq_len": CONTEXT_LEN,
                   "decode_context": ctx, "block_size": 16, "parallelism": "single-gpu",
                   "l2": "inputs larger than L2: a step streams all weights", "cuda_graph": not args.eager},
        "e2e": {"value": round(e2e_tps, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "peaks": peaks["source"]},
        "points": points,
        "clocks": ck,
    }
    print(json.dumps(line))


def serve_workload(shape_name, layers, requests, output_len, budget, eager):
    """Continuous batching through the entry point: `requests` prompts of uneven length arrive at once,
    prompts are cut into portions under a token budget and run beside the decoding requests."""
    import torch

    from rvllm_b200 import LLM, SamplingParams, config_from_dict
    from rvllm_b200.kernels.library import COUNTERS

    shape, _, context = SHAPES[shape_name]
    cfg_dict = dict(shape)
    full_layers = cfg_dict["num_hidden_layers"]
    cfg_dict["num_hidden_layers"] = layers or full_layers
    gen = torch.Generator().manual_seed(0)
    lo, hi = 128, min(4096, context - output_len)
    lengths = torch.randint(lo, hi + 1, (requests,), generator=gen).tolist()
    prompts = [torch.randint(0, cfg_dict["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
    pages = sum((n + output_len + 15) // 16 + 1 for n in lengths)
    llm = LLM(config=config_from_dict(cfg_dict), random_weights=True, seed=0, dtype="bfloat16", block_size=16,
              num_blocks=pages + 8, max_model_len=context, max_num_seqs=requests,
              max_num_batched_tokens=budget, enforce_eager=eager)
    sp = SamplingParams(temperature=0.0, max_tokens=output_len, ignore_eos=True)
    llm.generate(prompts[:2], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))     # warm-up
    graphs = llm.capture_graphs(hi + output_len)      # as a service does when it starts, not while it serves
    clocks = ClockSampler()
    clocks.start()
    COUNTERS["launches"] = 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = llm.generate(prompts, sp)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    ck = clocks.stop()
    n_out = sum(len(o.outputs[0].token_ids) for o in outs)
    return {
        "metric": f"continuous batching, output tokens/s ({shape_name} layer sizes, bf16, random weights)",
        "value": round(n_out / dt, 1), "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
        "impl": "ours", "data": "synthetic: random weights, uniform random token ids, all requests arrive at once",
        "seconds": round(dt, 3), "prompt_tokens": sum(lengths), "output_tokens": n_out,
        "total_tokens_per_s": round((sum(lengths) + n_out) / dt, 1),
        "preemptions": sum(o.num_preemptions for o in outs), "gpu_launches": COUNTERS["launches"],
        "config": {"model": f"{shape_name}-shape", "layers": cfg_dict["num_hidden_layers"], "layers_full": full_layers,
                   "requests": requests, "prompt_len": f"uniform {lo}..{hi}", "output_len": output_len,
                   "token_budget": budget, "seq_len": context, "block_size": 16, "cuda_graph": not eager,
                   "graphs_captured_before": graphs},
        "clocks": ck}


# ---------------------------------------------------------------------------------------------------------
# --workload tufirax: the Tufirax design (attention with whole-row q/k norms, capped scores, a sink and a head gate;
# mamba2 mixers; GELU-gated feed-forwards; norms on the sublayers' outputs around a float32 stream) at layer sizes
# that resemble real models, beside the Llama decoder of this engine at the same width, heads, feed-forward and
# depth; then each of the design's own kernels alone beside the like kernel of the Llama path, with the bytes it has
# to move over its time against the measured copy bandwidth.  Random weights; its own JSON line.
TUFIRAX_SIZES = {
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, rot=64, ff=8192, m_heads=64, m_vdim=64, state=128, groups=8, layers=8),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, rot=128, ff=14336, m_heads=128, m_vdim=64, state=128, groups=8, layers=8),
}


def tufirax_pair(size: dict, vocab: int = 32768):
    """(Tufirax configuration, Llama configuration) of equal width, heads, feed-forward and depth.  The Tufirax layers
    alternate attention and mamba2, each with a feed-forward."""
    att = {"type": "attention", "mixer": {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": size["dim"], "vdim": size["dim"],
                                          "scale": size["dim"] ** -0.5, "softcap": 30.0, "rot": {"dims": size["rot"], "base": 500000.0}},
           "mlp": {"kind": "dense", "ff": size["ff"]}}
    mam = {"type": "mamba2", "mixer": {"heads": size["m_heads"], "vdim": size["m_vdim"], "state": size["state"], "groups": size["groups"],
                                       "conv": 4, "norm_groups": size["groups"]}, "mlp": {"kind": "dense", "ff": size["ff"]}}
    tfx = {"architecture": "Tufirax", "width": size["width"], "vocab": vocab, "norm": {"eps": 1e-6},
           "layers": [att if i % 2 == 0 else mam for i in range(size["layers"])]}
    llama = {"architectures": ["LlamaForCausalLM"], "hidden_size": size["width"], "num_hidden_layers": size["layers"],
             "num_attention_heads": size["heads"], "num_key_value_heads": size["kv_heads"], "head_dim": size["dim"],
             "intermediate_size": size["ff"], "vocab_size": vocab, "max_position_embeddings": 8192, "rms_norm_eps": 1e-6,
             "rope_theta": 500000.0, "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "bfloat16"}
    return tfx, llama


def _time_kernel(fn, iters=5, flush=None):
    """Milliseconds of one call of fn, the best of `iters`, each after a write of a buffer larger than L2."""
    import torch
    best = float("inf")
    fn()
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b))
    return best


def run_tufirax(args):
    import torch

    from rvllm_b200 import LLM, config_from_dict
    from rvllm_b200.engine import StepEntry
    from rvllm_b200.kernels import AttentionMeta

    peaks = measured_peaks()
    PROMPT, CTX, batch = 2048, 4096, args.batch
    gen = torch.Generator().manual_seed(0)
    out = {"workload": "tufirax", "dtype": "bf16", "data": "synthetic", "peaks": peaks["source"], "prompt_len": PROMPT, "batch": batch,
           "steps": args.steps, "warmup": args.warmup, "models": {}, "kernels": {}}

    def measure(cfg_dict):
        config = config_from_dict(cfg_dict)
        llm = LLM(config=config, random_weights=True, seed=0, dtype="bfloat16", block_size=16, num_blocks=batch * (CTX // 16) + 8,
                  max_model_len=CTX, max_num_seqs=batch, max_num_batched_tokens=PROMPT, enforce_eager=args.eager)
        runner, V = llm.engine.runner, llm.engine.spec.vocab_size
        p = torch.randint(0, V, (PROMPT,), generator=gen).tolist()
        for _ in range(3):
            runner.step([StepEntry("w", p, [PROMPT - 1])])
            runner.finish("w")
        torch.cuda.synchronize()
        pf = []
        for _ in range(3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            runner.step([StepEntry("p", p, [PROMPT - 1])])
            b.record()
            torch.cuda.synchronize()
            runner.finish("p")
            pf.append(a.elapsed_time(b))
        ids = [f"d{i}" for i in range(batch)]
        for rid in ids:
            runner.step([StepEntry(rid, torch.randint(0, V, (PROMPT,), generator=gen).tolist(), [])])
        for _ in range(args.warmup):
            runner.step([StepEntry(r, [1], [0]) for r in ids])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            runner.step([StepEntry(r, [1], [0]) for r in ids])
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        for rid in ids:
            runner.finish(rid)
        kernels = llm.engine.kernels
        del llm
        torch.cuda.empty_cache()
        return {"prefill_ms": round(min(pf), 3), "prefill_tok_s": round(PROMPT / (min(pf) / 1e3), 1),
                "decode_ms_per_step": round(ms, 4), "decode_tok_s": round(batch / (ms / 1e3), 1)}, kernels

    K = None
    for name in (args.sizes.split(",") if args.sizes else list(TUFIRAX_SIZES)):
        tfx, llama = tufirax_pair(TUFIRAX_SIZES[name])
        a, K = measure(tfx)
        b, K = measure(llama)
        out["models"][name] = {"tufirax": a, "llama_same_size": b, "layers": TUFIRAX_SIZES[name]["layers"],
                               "prefill_ratio": round(a["prefill_tok_s"] / b["prefill_tok_s"], 3),
                               "decode_ratio": round(a["decode_tok_s"] / b["decode_tok_s"], 3)}

    # ---- the design's kernels alone, at the "4k" sizes, beside the like kernel of the Llama path ------------------
    z = TUFIRAX_SIZES["4k"]
    dev, bf = "cuda", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    bw = peaks["hbm_gbs"] * 1e9

    def row(name, ms, nbytes, like=None):
        out["kernels"][name] = {"ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / (ms / 1e3) / bw, 3)}
        if like is not None:
            out["kernels"][name]["like"] = like

    T, W, FF = PROMPT, z["width"], z["ff"]
    y = torch.randn(T, W, device=dev)
    g = torch.ones(W, dtype=bf, device=dev)
    res = torch.randn(T, W, device=dev)
    xb = torch.randn(T, W, device=dev).to(bf)
    ms_like = _time_kernel(lambda: K.rmsnorm(xb, g, 1e-6), flush=flush)
    like = {"kernel": "rmsnorm", "ms": round(ms_like, 4), "frac_hbm": round(T * W * 4 / (ms_like / 1e3) / bw, 3)}
    row("residual_rmsnorm", _time_kernel(lambda: K.residual_rmsnorm(y, g, 1e-6, res, bf), flush=flush), T * W * (4 + 4 + 4 + 2), like)
    gu = torch.randn(T, 2 * FF, device=dev)
    gub = gu.to(bf)
    ms_like = _time_kernel(lambda: K.silu_mul(gub), flush=flush)
    like = {"kernel": "silu_mul", "ms": round(ms_like, 4), "frac_hbm": round(T * FF * 6 / (ms_like / 1e3) / bw, 3)}
    row("act_mul_gelu", _time_kernel(lambda: K.act_mul(gu, "gelu_tanh", bf), flush=flush), T * FF * (8 + 2), like)

    # attention: one prompt of 2,048 tokens, and a decode step of `batch` sequences behind 2,048 tokens
    nh, nkv, hd = z["heads"], z["kv_heads"], z["dim"]
    sinks = torch.zeros(nh, device=dev)
    # what follows the q/k(/v) product: norms over the whole rows, rotation, cache write, gate - beside bias-free rotation and cache write
    pages = PROMPT // 16
    cache1 = torch.zeros(pages, 2, nkv, 16, hd, dtype=bf, device=dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * torch.tensor([500000.0 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64)[None, :]
    cos, sin = torch.cos(ang).float().to(dev), torch.sin(ang).float().to(dev)
    proj_qkg = torch.randn(T, (nh + nkv) * hd + nh, device=dev)
    proj_qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=dev)
    wq, wk = torch.ones(nh * hd, dtype=bf, device=dev), torch.ones(nkv * hd, dtype=bf, device=dev)
    ms_like = _time_kernel(lambda: K.rope_cache_write(proj_qkv, None, pos, cos, sin, pos, cache1, nh, nkv, hd, out_dtype=bf), flush=flush)
    like = {"kernel": "rope_cache_write", "ms": round(ms_like, 4), "frac_hbm": round(T * (nh + 2 * nkv) * hd * 6 / (ms_like / 1e3) / bw, 3)}
    row("qk_norm_rope_cache_write", _time_kernel(lambda: K.qk_norm_rope_cache_write(proj_qkg, wq, wk, 1e-6, pos, cos, sin, pos, cache1, nh, nkv, hd,
                                                                                    bf, with_gate=True), flush=flush),
        T * ((nh + nkv) * hd * 6 + nkv * hd * 2 + nh * 8), like)

    def attention_case(q_len, ctx, seqs):
        pages = seqs * (ctx // 16)
        cache = torch.randn(pages, 2, nkv, 16, hd, device=dev).to(bf)
        tables = torch.arange(pages, dtype=torch.int32, device=dev).view(seqs, ctx // 16)
        cu = torch.arange(seqs + 1, dtype=torch.int32, device=dev) * q_len
        meta = AttentionMeta(tables, cu, torch.full((seqs,), ctx, dtype=torch.int32, device=dev),
                             torch.arange(seqs, dtype=torch.int32, device=dev).repeat_interleave(q_len), None, seqs, q_len, ctx, 16,
                             seqs if q_len == 1 else 0)
        q = torch.randn(seqs * q_len, nh * hd, device=dev).to(bf)
        gate = torch.rand(seqs * q_len, nh, device=dev)
        return q, cache, meta, gate

    q, cache, meta, gate = attention_case(PROMPT, PROMPT, 1)
    flops = 4.0 * nh * hd * PROMPT * PROMPT / 2
    ms_like = _time_kernel(lambda: K.paged_attention(q, cache, meta, nh, nkv, hd, hd ** -0.5, None), flush=flush)
    ms = _time_kernel(lambda: K.paged_attention(q, cache, meta, nh, nkv, hd, hd ** -0.5, None, softcap=30.0, sinks=sinks, gate=gate), flush=flush)
    out["kernels"]["attention_prefill_cap_sink_gate"] = {
        "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "frac_bf16": round(flops / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 3),
        "like": {"kernel": "attention_prefill", "ms": round(ms_like, 4), "frac_bf16": round(flops / (ms_like / 1e3) / (peaks["bf16_tflops"] * 1e12), 3)}}
    q, cache, meta, gate = attention_case(1, PROMPT, batch)
    nbytes = batch * PROMPT * 2 * nkv * hd * 2
    ms_like = _time_kernel(lambda: K.paged_attention(q, cache, meta, nh, nkv, hd, hd ** -0.5, None), flush=flush)
    like = {"kernel": "attention_decode", "ms": round(ms_like, 4), "frac_hbm": round(nbytes / (ms_like / 1e3) / bw, 3)}
    row("attention_decode_cap_sink_gate",
        _time_kernel(lambda: K.paged_attention(q, cache, meta, nh, nkv, hd, hd ** -0.5, None, softcap=30.0, sinks=sinks, gate=gate), flush=flush),
        nbytes, like)

    # the state-space mixer's kernels: a 2,048-token prompt, and a decode step of `batch` sequences
    H, P, N, G = z["m_heads"], z["m_vdim"], z["state"], z["groups"]
    inner, ch = H * P, H * P + 2 * G * N
    wide = 2 * inner + 2 * G * N + H
    conv_w, conv_b = torch.randn(ch, 4, device=dev).to(bf), torch.zeros(ch, dtype=bf, device=dev)
    dt_bias, a_log, d_skip = torch.zeros(H, device=dev), torch.zeros(H, device=dev), torch.ones(H, device=dev)
    norm_w = torch.ones(inner, dtype=bf, device=dev)
    for label, q_len, seqs in (("prefill", PROMPT, 1), ("decode", 1, batch)):
        rows = q_len * seqs
        proj = torch.randn(rows, wide, device=dev)
        state = torch.zeros(seqs, H * N * P + 3 * ch, device=dev)
        seq_of = torch.arange(seqs, dtype=torch.int32, device=dev).repeat_interleave(q_len)
        cu = torch.arange(seqs + 1, dtype=torch.int32, device=dev) * q_len
        slots = torch.arange(seqs, dtype=torch.int32, device=dev)
        xbc = K.causal_conv_silu(proj, inner, ch, conv_w, conv_b, seq_of, cu, slots, state, H * N * P, bf)
        row(f"causal_conv_silu_{label}", _time_kernel(lambda: K.causal_conv_silu(proj, inner, ch, conv_w, conv_b, seq_of, cu, slots, state,
                                                                                 H * N * P, bf), flush=flush), rows * ch * (4 + 2))
        yv = K.ssm_scan(xbc, proj, inner + ch, dt_bias, a_log, d_skip, cu, slots, state, H, P, N, G)
        ms = _time_kernel(lambda: K.ssm_scan(xbc, proj, inner + ch, dt_bias, a_log, d_skip, cu, slots, state, H, P, N, G), flush=flush)
        row(f"ssm_scan_{label}", ms, rows * (ch * 2 + inner * 4) + seqs * H * N * P * 8)
        out["kernels"][f"ssm_scan_{label}"]["gflops"] = round(rows * H * P * N * 5 / ms / 1e6, 1)
        row(f"gated_group_rmsnorm_{label}", _time_kernel(lambda: K.gated_group_rmsnorm(yv, proj, norm_w, 1e-6, G, bf), flush=flush),
            rows * inner * (4 + 4 + 2))
    print(json.dumps(out))


# ---------------------------------------------------------------------------------------------------------
# --workload vipelix: the Vipelix design (latent attention over one cached row per token, a norm in front of and behind
# every sublayer around a float32 stream, a dense feed-forward with a PolyNorm activation, experts chosen by a table
# lookup plus a shared expert, a span of layers that runs twice) at layer sizes that resemble real models, beside the
# Llama decoder of this engine at the same width, heads and depth whose feed-forward is as wide as what a token of
# the mixture activates; then each of the design's own kernels alone beside the like kernel of the Llama path, with
# its bytes or FLOPs over its time against the measured copy bandwidth or bf16 peak.  Random weights; its own JSON line.
VIPELIX_SIZES = {
    "2k": dict(width=2048, heads=16, dim=128, rot=64, vdim=128, rank=192, ff=8192, e_ff=1408, experts=16, top=2, shared=2816, layers=4, times=2),
    "4k": dict(width=4096, heads=32, dim=128, rot=64, vdim=128, rank=192, ff=14336, e_ff=2048, experts=32, top=4, shared=4096, layers=4, times=2),
}


def vipelix_pair(size: dict, vocab: int = 32768):
    """(Vipelix configuration, Llama configuration).  The Vipelix stack: a dense layer, then layers of experts; all of
    them run `times` times.  The Llama stack has as many layers as the Vipelix one has layer runs."""
    mixer = {"heads": size["heads"], "dim": size["dim"], "rot_dim": size["rot"], "vdim": size["vdim"], "kv_rank": size["rank"],
             "scale": (size["dim"] + size["rot"]) ** -0.5, "rot": {"dims": size["rot"], "base": 500000.0}}
    dense = {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": size["ff"]}}
    moe = {"type": "latent_attention", "mixer": mixer,
           "mlp": {"kind": "moe", "expert": {"ff": size["e_ff"]}, "router": {"experts": size["experts"], "top": size["top"]},
                   "shared": {"ff": size["shared"]}}}
    vip = {"architecture": "Vipelix", "width": size["width"], "vocab": vocab, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
           "loop": {"start": 0, "stop": size["layers"], "times": size["times"]},
           "layers": [dense] + [moe] * (size["layers"] - 1)}
    llama = {"architectures": ["LlamaForCausalLM"], "hidden_size": size["width"], "num_hidden_layers": size["layers"] * size["times"],
             "num_attention_heads": size["heads"], "num_key_value_heads": size["heads"] // 4, "head_dim": size["dim"],
             "intermediate_size": size["top"] * size["e_ff"] + size["shared"], "vocab_size": vocab, "max_position_embeddings": 8192,
             "rms_norm_eps": 1e-6, "rope_theta": 500000.0, "tie_word_embeddings": True, "hidden_act": "silu", "torch_dtype": "bfloat16"}
    return vip, llama


def run_vipelix(args):
    import torch

    from rvllm_b200 import LLM, config_from_dict
    from rvllm_b200.engine import StepEntry
    from rvllm_b200.kernels import AttentionMeta

    peaks = measured_peaks()
    PROMPT, CTX, batch = 2048, 4096, args.batch
    gen = torch.Generator().manual_seed(0)
    out = {"workload": "vipelix", "dtype": "bf16", "data": "synthetic", "peaks": peaks["source"], "prompt_len": PROMPT, "batch": batch,
           "steps": args.steps, "warmup": args.warmup, "models": {}, "kernels": {}}

    def measure(cfg_dict):
        config = config_from_dict(cfg_dict)
        llm = LLM(config=config, random_weights=True, seed=0, dtype="bfloat16", block_size=16, num_blocks=batch * (CTX // 16) + 8,
                  max_model_len=CTX, max_num_seqs=batch, max_num_batched_tokens=PROMPT, enforce_eager=args.eager)
        runner, V = llm.engine.runner, llm.engine.spec.vocab_size
        p = torch.randint(0, V, (PROMPT,), generator=gen).tolist()
        for _ in range(3):
            runner.step([StepEntry("w", p, [PROMPT - 1])])
            runner.finish("w")
        torch.cuda.synchronize()
        pf = []
        for _ in range(3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            runner.step([StepEntry("p", p, [PROMPT - 1])])
            b.record()
            torch.cuda.synchronize()
            runner.finish("p")
            pf.append(a.elapsed_time(b))
        ids = [f"d{i}" for i in range(batch)]
        for rid in ids:
            runner.step([StepEntry(rid, torch.randint(0, V, (PROMPT,), generator=gen).tolist(), [])])
        for _ in range(args.warmup):
            runner.step([StepEntry(r, [1], [0]) for r in ids])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            runner.step([StepEntry(r, [1], [0]) for r in ids])
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        for rid in ids:
            runner.finish(rid)
        kernels = llm.engine.kernels
        kernels.raise_on_abort()
        del llm
        torch.cuda.empty_cache()
        return {"prefill_ms": round(min(pf), 3), "prefill_tok_s": round(PROMPT / (min(pf) / 1e3), 1),
                "decode_ms_per_step": round(ms, 4), "decode_tok_s": round(batch / (ms / 1e3), 1)}, kernels

    K = None
    for name in (args.sizes.split(",") if args.sizes else list(VIPELIX_SIZES)):
        vip, llama = vipelix_pair(VIPELIX_SIZES[name])
        a, K = measure(vip)
        b, K = measure(llama)
        out["models"][name] = {"vipelix": a, "llama_same_size": b, "layer_runs": VIPELIX_SIZES[name]["layers"] * VIPELIX_SIZES[name]["times"],
                               "prefill_ratio": round(a["prefill_tok_s"] / b["prefill_tok_s"], 3),
                               "decode_ratio": round(a["decode_tok_s"] / b["decode_tok_s"], 3)}

    # ---- the design's kernels alone, at the "4k" sizes, beside the like kernel of the Llama path ------------------
    torch.manual_seed(0)           # (which experts the tokens of the expert cases choose)
    z = VIPELIX_SIZES["4k"]
    dev, bf = "cuda", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    bw, peak = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12

    def by_bytes(name, ms, nbytes, like=None):
        out["kernels"][name] = {"ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / (ms / 1e3) / bw, 3)}
        if like is not None:
            out["kernels"][name]["like"] = like

    def by_flops(name, ms, flops, like=None):
        out["kernels"][name] = {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "frac_bf16": round(flops / (ms / 1e3) / peak, 3)}
        if like is not None:
            out["kernels"][name]["like"] = like

    T, W, FF = PROMPT, z["width"], z["ff"]
    H, D, RD, V, R = z["heads"], z["dim"], z["rot"], z["vdim"], z["rank"]
    ROW = R + RD
    y, res = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev)
    g = torch.ones(W, dtype=bf, device=dev)
    xb = torch.randn(T, W, device=dev).to(bf)
    ms_like = _time_kernel(lambda: K.rmsnorm(xb, g, 1e-6), flush=flush)
    like = {"kernel": "rmsnorm", "ms": round(ms_like, 4), "frac_hbm": round(T * W * 4 / (ms_like / 1e3) / bw, 3)}
    by_bytes("residual_rmsnorm_then_norm", _time_kernel(lambda: K.residual_rmsnorm(y, g, 1e-6, res, bf, next_norm=(g, 1e-6)), flush=flush),
             T * W * (4 + 4 + 4 + 2), like)
    zf = torch.randn(T, FF, device=dev)
    gub = torch.randn(T, 2 * FF, device=dev).to(bf)
    ms_like = _time_kernel(lambda: K.silu_mul(gub), flush=flush)
    like = {"kernel": "silu_mul", "ms": round(ms_like, 4), "frac_hbm": round(T * FF * 6 / (ms_like / 1e3) / bw, 3)}
    coef = torch.tensor([0.5, 0.3, 0.2, 0.1], device=dev)
    by_bytes("polynorm", _time_kernel(lambda: K.polynorm(zf, coef, 1e-6, bf), flush=flush), T * FF * (4 + 2), like)

    # what follows the stacked projection: the latent's norm, the rotations, the cache row, the split of q, the gate
    pages = PROMPT // 16
    cache1 = torch.zeros(pages, 1, 1, 16, ROW, dtype=bf, device=dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * torch.tensor([500000.0 ** (-2.0 * i / RD) for i in range(RD // 2)], dtype=torch.float64)[None, :]
    cos, sin = torch.cos(ang).float().to(dev), torch.sin(ang).float().to(dev)
    proj = torch.randn(T, H * (D + RD) + ROW + H, device=dev)
    gamma = torch.ones(R, dtype=bf, device=dev)
    nkv = H // 4
    cache2 = torch.zeros(pages, 2, nkv, 16, D, dtype=bf, device=dev)
    ang2 = torch.arange(T, dtype=torch.float64)[:, None] * torch.tensor([500000.0 ** (-2.0 * i / D) for i in range(D // 2)], dtype=torch.float64)[None, :]
    cos2, sin2 = torch.cos(ang2).float().to(dev), torch.sin(ang2).float().to(dev)
    proj_qkv = torch.randn(T, (H + 2 * nkv) * D, device=dev)
    ms_like = _time_kernel(lambda: K.rope_cache_write(proj_qkv, None, pos, cos2, sin2, pos, cache2, H, nkv, D, out_dtype=bf), flush=flush)
    like = {"kernel": "rope_cache_write", "ms": round(ms_like, 4), "frac_hbm": round(T * (H + 2 * nkv) * D * 6 / (ms_like / 1e3) / bw, 3)}
    by_bytes("latent_prepare", _time_kernel(lambda: K.latent_prepare(proj, gamma, 1e-6, pos, cos, sin, pos, cache1, H, D, RD, R, bf), flush=flush),
             T * (proj.shape[1] * 4 + (H * (D + RD) + ROW) * 2 + H * 4), like)

    # the per-head products (the key up-projection moved onto the query; the value up-projection of the attended latent)
    q_plain, q_row = torch.randn(T, H, D, device=dev).to(bf), torch.zeros(T, H, ROW, dtype=bf, device=dev)
    uk_t, uv = torch.randn(H, R, D, device=dev).to(bf), torch.randn(H, V, R, device=dev).to(bf)
    wl = torch.randn(H * R, W, device=dev).to(bf)
    ms_like = _time_kernel(lambda: K.linear(xb, wl), flush=flush)
    like = {"kernel": "linear (tcgen05), 2,048 x %d x %d" % (H * R, W), "ms": round(ms_like, 4),
            "frac_bf16": round(2.0 * T * H * R * W / (ms_like / 1e3) / peak, 3)}
    by_flops("head_linear_absorb", _time_kernel(lambda: K.head_linear(q_plain, uk_t, q_row[:, :, :R]), flush=flush), 2.0 * T * H * R * D, like)
    o_lat = torch.randn(T, H, R, device=dev).to(bf)
    by_flops("head_linear_values", _time_kernel(lambda: K.head_linear(o_lat, uv, None), flush=flush), 2.0 * T * H * R * V)
    # (K is one head's 128 to 192 elements: the operands' bytes, not the products, set these kernels' floor)
    for name, nbytes in (("head_linear_absorb", T * H * (D + R) * 2 + H * R * D * 2), ("head_linear_values", T * H * (R + V) * 2 + H * R * V * 2)):
        out["kernels"][name]["frac_hbm"] = round(nbytes / (out["kernels"][name]["ms"] / 1e3) / bw, 3)

    def latent_case(q_len, ctx, seqs):
        n = seqs * (ctx // 16)
        cache = torch.randn(n, 1, 1, 16, ROW, device=dev).to(bf)
        tables = torch.arange(n, dtype=torch.int32, device=dev).view(seqs, ctx // 16)
        cu = torch.arange(seqs + 1, dtype=torch.int32, device=dev) * q_len
        meta = AttentionMeta(tables, cu, torch.full((seqs,), ctx, dtype=torch.int32, device=dev),
                             torch.arange(seqs, dtype=torch.int32, device=dev).repeat_interleave(q_len), None, seqs, q_len, ctx, 16,
                             seqs if q_len == 1 else 0)
        return torch.randn(seqs * q_len, H, ROW, device=dev).to(bf), cache, meta, torch.rand(seqs * q_len, H, device=dev)

    def llama_case(q_len, ctx, seqs):
        n = seqs * (ctx // 16)
        cache = torch.randn(n, 2, nkv, 16, D, device=dev).to(bf)
        tables = torch.arange(n, dtype=torch.int32, device=dev).view(seqs, ctx // 16)
        cu = torch.arange(seqs + 1, dtype=torch.int32, device=dev) * q_len
        meta = AttentionMeta(tables, cu, torch.full((seqs,), ctx, dtype=torch.int32, device=dev),
                             torch.arange(seqs, dtype=torch.int32, device=dev).repeat_interleave(q_len), None, seqs, q_len, ctx, 16,
                             seqs if q_len == 1 else 0)
        return torch.randn(seqs * q_len, H * D, device=dev).to(bf), cache, meta

    q, cache, meta, gate = latent_case(PROMPT, PROMPT, 1)
    ql, cl, ml = llama_case(PROMPT, PROMPT, 1)
    ms_like = _time_kernel(lambda: K.paged_attention(ql, cl, ml, H, nkv, D, D ** -0.5, None), flush=flush)
    like = {"kernel": "attention_prefill (tcgen05, heads of %d)" % D, "ms": round(ms_like, 4),
            "frac_bf16": round(4.0 * H * D * PROMPT * PROMPT / 2 / (ms_like / 1e3) / peak, 3)}
    by_flops("latent_attention_prefill", _time_kernel(lambda: K.latent_attention(q, cache, meta, H, ROW, R, 0.07, gate=gate), flush=flush),
             2.0 * H * (ROW + R) * PROMPT * PROMPT / 2, like)
    q, cache, meta, gate = latent_case(1, PROMPT, batch)
    ql, cl, ml = llama_case(1, PROMPT, batch)
    ms_like = _time_kernel(lambda: K.paged_attention(ql, cl, ml, H, nkv, D, D ** -0.5, None), flush=flush)
    like = {"kernel": "attention_decode", "ms": round(ms_like, 4), "frac_hbm": round(batch * PROMPT * 2 * nkv * D * 2 / (ms_like / 1e3) / bw, 3)}
    by_bytes("latent_attention_decode", _time_kernel(lambda: K.latent_attention(q, cache, meta, H, ROW, R, 0.07, gate=gate), flush=flush),
             batch * PROMPT * ROW * 2, like)

    # the experts: a prompt's tokens sorted by expert through the grouped products, and a decode step's through the streaming kernels
    E, top, EF = z["experts"], z["top"], z["e_ff"]
    gate_up, down = torch.randn(E, 2 * EF, W, device=dev).to(bf) * 0.02, torch.randn(E, W, EF, device=dev).to(bf) * 0.02
    table = torch.rand(32768, E, device=dev).argsort(1)[:, :top].to(torch.int32).contiguous()
    tokens = torch.randint(0, 32768, (T,), device=dev, dtype=torch.int32)
    chosen = K.gather_rows(table, tokens)
    wgu = torch.randn(2 * top * EF, W, device=dev).to(bf) * 0.02
    wd = torch.randn(W, top * EF, device=dev).to(bf) * 0.02
    ms_like = _time_kernel(lambda: K.linear(K.gate_up_silu(xb, wgu), wd, out_dtype=torch.float32), flush=flush)
    flops = 6.0 * T * top * EF * W
    like = {"kernel": "gated MLP as wide as the chosen experts (two tcgen05 products)", "ms": round(ms_like, 4),
            "frac_bf16": round(flops / (ms_like / 1e3) / peak, 3)}
    by_flops("moe_experts_prefill", _time_kernel(lambda: K.moe_experts(xb, chosen, gate_up, down, 1.0 / top, out_dtype=torch.float32), flush=flush),
             flops, like)
    xd = xb[:batch].contiguous()
    cd = chosen[:batch].contiguous()
    touched = len(set(cd.flatten().tolist()))
    ms_like = _time_kernel(lambda: K.linear(K.gate_up_silu(xd, wgu), wd, out_dtype=torch.float32), flush=flush)
    like = {"kernel": "gated MLP as wide as the chosen experts (decode GEMMs)", "ms": round(ms_like, 4),
            "frac_hbm": round(3 * top * EF * W * 2 / (ms_like / 1e3) / bw, 3)}
    by_bytes("moe_experts_decode", _time_kernel(lambda: K.moe_experts(xd, cd, gate_up, down, 1.0 / top, out_dtype=torch.float32), flush=flush),
             touched * 3 * EF * W * 2, like)
    out["kernels"]["moe_experts_decode"]["experts_touched"] = touched
    K.raise_on_abort()
    print(json.dumps(out))


# ---------------------------------------------------------------------------------------------------------
# --workload tugodra: the Tugodra design (window attention with unit-norm queries and keys and borrowed keys, latent
# attention with a sink, mLSTM matrix memories, Dynamic-Tanh norms around every sublayer, routed squared-relu experts with a
# gated shared expert) at layer sizes that resemble real models, beside the Vipelix decoder of this engine - the closest
# design: a float32 stream with a norm in front of and behind every sublayer, latent attention, experts plus a shared one -
# at the same width, depth and experts; then each of the design's own kernels alone beside the like kernel of that path,
# with its bytes or FLOPs over its time against the measured copy bandwidth or bf16 peak.  Random weights; its own JSON line.
TUGODRA_SIZES = {
    "2k": dict(width=2048, heads=16, kv=4, dim=128, window=1024, l_dim=128, rot=64, rank=192, m_heads=8, m_dim=128, m_vdim=256,
               e_ff=1408, experts=16, top=2, groups=4, keep=2, shared=2816, layers=8),
    "4k": dict(width=4096, heads=32, kv=8, dim=128, window=1024, l_dim=128, rot=64, rank=192, m_heads=16, m_dim=128, m_vdim=256,
               e_ff=2048, experts=32, top=4, groups=8, keep=4, shared=4096, layers=8),
}


def tugodra_pair(size: dict, vocab: int = 32768):
    """(Tugodra configuration, Vipelix configuration): layers of matrix memory, window attention, latent attention and a
    window attention that borrows its keys, in turn, each with experts; beside as many Vipelix layers of experts."""
    mlp = {"kind": "moe", "expert": {"ff": size["e_ff"]},
           "router": {"experts": size["experts"], "top": size["top"], "groups": {"count": size["groups"], "keep": size["keep"]}},
           "shared": {"ff": size["shared"]}}
    att = {"heads": size["heads"], "kv_heads": size["kv"], "dim": size["dim"], "vdim": size["dim"], "scale": size["dim"] ** 0.5 * 0.1,
           "mask": {"size": size["window"]}, "rot": {"dims": size["dim"], "base": 1e6}}
    lat = {"heads": size["heads"], "dim": size["l_dim"], "rot_dim": size["rot"], "vdim": size["l_dim"], "kv_rank": size["rank"],
           "scale": (size["l_dim"] + size["rot"]) ** -0.5, "rot": {"dims": size["rot"], "base": 500000.0}}
    mem = {"heads": size["m_heads"], "dim": size["m_dim"], "vdim": size["m_vdim"], "gate_cap": 15.0}
    layers = []
    for i in range(size["layers"]):
        k = i % 4
        if k == 0:
            layers.append({"type": "mlstm", "mixer": mem, "mlp": mlp})
        elif k == 1:
            layers.append({"type": "attention", "mixer": att, "mlp": mlp})
        elif k == 2:
            layers.append({"type": "latent_attention", "mixer": lat, "mlp": mlp})
        else:
            layers.append({"type": "attention", "mixer": dict(att, kv_from=i - 2), "mlp": mlp})
    tug = {"architecture": "Tugodra", "width": size["width"], "vocab": vocab, "norm": {"eps": 1e-6}, "embedding": {"scale": size["width"] ** 0.5},
           "layers": layers}
    vmoe = {"type": "latent_attention", "mixer": dict(lat),
            "mlp": {"kind": "moe", "expert": {"ff": size["e_ff"]}, "router": {"experts": size["experts"], "top": size["top"]},
                    "shared": {"ff": size["shared"]}}}
    vip = {"architecture": "Vipelix", "width": size["width"], "vocab": vocab, "norm": {"eps": 1e-6}, "layers": [vmoe] * size["layers"]}
    return tug, vip


def run_tugodra(args):
    import torch

    from rvllm_b200 import LLM, config_from_dict
    from rvllm_b200.engine import StepEntry
    from rvllm_b200.kernels import AttentionMeta

    peaks = measured_peaks()
    PROMPT, CTX, batch = 2048, 4096, args.batch
    gen = torch.Generator().manual_seed(0)
    out = {"workload": "tugodra", "dtype": "bf16", "data": "synthetic", "peaks": peaks["source"], "prompt_len": PROMPT, "batch": batch,
           "steps": args.steps, "warmup": args.warmup, "models": {}, "kernels": {}}

    def measure(cfg_dict):
        config = config_from_dict(cfg_dict)
        llm = LLM(config=config, random_weights=True, seed=0, dtype="bfloat16", block_size=16, num_blocks=batch * (CTX // 16) + 8,
                  max_model_len=CTX, max_num_seqs=batch, max_num_batched_tokens=PROMPT, enforce_eager=args.eager)
        runner, V = llm.engine.runner, llm.engine.spec.vocab_size
        p = torch.randint(0, V, (PROMPT,), generator=gen).tolist()
        for _ in range(3):
            runner.step([StepEntry("w", p, [PROMPT - 1])])
            runner.finish("w")
        torch.cuda.synchronize()
        pf = []
        for _ in range(3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            runner.step([StepEntry("p", p, [PROMPT - 1])])
            b.record()
            torch.cuda.synchronize()
            runner.finish("p")
            pf.append(a.elapsed_time(b))
        ids = [f"d{i}" for i in range(batch)]
        for rid in ids:
            runner.step([StepEntry(rid, torch.randint(0, V, (PROMPT,), generator=gen).tolist(), [])])
        for _ in range(args.warmup):
            runner.step([StepEntry(r, [1], [0]) for r in ids])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            runner.step([StepEntry(r, [1], [0]) for r in ids])
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        for rid in ids:
            runner.finish(rid)
        kernels = llm.engine.kernels
        kernels.raise_on_abort()
        del llm
        torch.cuda.empty_cache()
        return {"prefill_ms": round(min(pf), 3), "prefill_tok_s": round(PROMPT / (min(pf) / 1e3), 1),
                "decode_ms_per_step": round(ms, 4), "decode_tok_s": round(batch / (ms / 1e3), 1)}, kernels

    K = None
    for name in (args.sizes.split(",") if args.sizes else list(TUGODRA_SIZES)):
        tug, vip = tugodra_pair(TUGODRA_SIZES[name])
        a, K = measure(tug)
        b, K = measure(vip)
        out["models"][name] = {"tugodra": a, "vipelix_same_size": b, "layers": TUGODRA_SIZES[name]["layers"],
                               "prefill_ratio": round(a["prefill_tok_s"] / b["prefill_tok_s"], 3),
                               "decode_ratio": round(a["decode_tok_s"] / b["decode_tok_s"], 3)}
    if K is None:
        from rvllm_b200.kernels import get_library
        K = get_library("cuda:0")

    # ---- the design's kernels alone, at the "4k" sizes, beside the like kernel of the Vipelix path ----------------
    torch.manual_seed(0)
    z = TUGODRA_SIZES["4k"]
    dev, bf = "cuda", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    bw, peak = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12

    def by_bytes(name, ms, nbytes, like=None):
        out["kernels"][name] = {"ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / (ms / 1e3) / bw, 3)}
        if like is not None:
            out["kernels"][name]["like"] = like

    def by_flops(name, ms, flops, like=None):
        out["kernels"][name] = {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "frac_bf16": round(flops / (ms / 1e3) / peak, 3)}
        if like is not None:
            out["kernels"][name]["like"] = like

    def like_bytes(kernel, ms, nbytes):
        return {"kernel": kernel, "ms": round(ms, 4), "frac_hbm": round(nbytes / (ms / 1e3) / bw, 3)}

    def like_flops(kernel, ms, flops):
        return {"kernel": kernel, "ms": round(ms, 4), "frac_bf16": round(flops / (ms / 1e3) / peak, 3)}

    T, W = PROMPT, z["width"]
    H, G, D, WIN = z["heads"], z["kv"], z["dim"], z["window"]
    # -- the sum with both norms
    y, res = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev)
    g = torch.ones(W, dtype=bf, device=dev)
    dyt = (torch.full((1,), 0.7, device=dev), torch.ones(W, device=dev), torch.zeros(W, device=dev))
    ms_like = _time_kernel(lambda: K.residual_rmsnorm(y, g, 1e-6, res, bf, next_norm=(g, 1e-6)), flush=flush)
    by_bytes("residual_dynamic_tanh_then_norm", _time_kernel(lambda: K.residual_dynamic_tanh(y, dyt, res, dyt, bf), flush=flush),
             T * W * (4 + 4 + 4 + 2), like_bytes("residual_rmsnorm with the next norm", ms_like, T * W * (4 + 4 + 4 + 2)))
    xf = torch.randn(T, W, device=dev)
    xb = xf.to(bf)
    ms_like = _time_kernel(lambda: K.rmsnorm(xf, g, 1e-6, out_dtype=bf), flush=flush)
    by_bytes("dynamic_tanh", _time_kernel(lambda: K.dynamic_tanh(xf, *dyt, out_dtype=bf), flush=flush), T * W * 6,
             like_bytes("rmsnorm", ms_like, T * W * 6))

    # -- rotation, unit norm and cache write of the window attention beside the latent's prepare kernel
    pages = PROMPT // 16
    pos = torch.arange(T, dtype=torch.int32, device=dev)

    def tables(dims, base):
        ang = torch.arange(T, dtype=torch.float64)[:, None] * torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)[None, :]
        return torch.cos(ang).float().to(dev), torch.sin(ang).float().to(dev)

    cos, sin = tables(D, 1e6)
    proj = torch.randn(T, H * D + 2 * G * D + H, device=dev)
    cache2 = torch.zeros(pages, 2, G, 16, D, dtype=bf, device=dev)
    LD, RD, R = z["l_dim"], z["rot"], z["rank"]
    ROW = R + RD
    cos_l, sin_l = tables(RD, 500000.0)
    proj_l = torch.randn(T, H * (LD + RD) + ROW, device=dev)
    cache1 = torch.zeros(pages, 1, 1, 16, ROW, dtype=bf, device=dev)
    gamma = torch.ones(R, dtype=bf, device=dev)
    ms_like = _time_kernel(lambda: K.latent_prepare(proj_l, gamma, 1e-6, pos, cos_l, sin_l, pos, cache1, H, LD, RD, R, bf, with_gate=False, halves=True), flush=flush)
    by_bytes("qk_unit_prepare", _time_kernel(lambda: K.qk_unit_prepare(proj, 1e-6, pos, cos, sin, pos, cache2, H, G, D, D, D, bf), flush=flush),
             T * (proj.shape[1] * 4 + (H + 2 * G) * D * 2 + H * 4),
             like_bytes("latent_prepare", ms_like, T * (proj_l.shape[1] * 4 + (H * (LD + RD) + ROW) * 2)))

    # -- attention inside a window (the engine's attention kernels with a window and a gate) beside the same kernels without
    def paged_case(q_len, ctx, seqs):
        n = seqs * (ctx // 16)
        cache = torch.randn(n, 2, G, 16, D, device=dev).to(bf)
        tbl = torch.arange(n, dtype=torch.int32, device=dev).view(seqs, ctx // 16)
        cu = torch.arange(seqs + 1, dtype=torch.int32, device=dev) * q_len
        meta = AttentionMeta(tbl, cu, torch.full((seqs,), ctx, dtype=torch.int32, device=dev),
                             torch.arange(seqs, dtype=torch.int32, device=dev).repeat_interleave(q_len), None, seqs, q_len, ctx, 16,
                             seqs if q_len == 1 else 0)
        return torch.randn(seqs * q_len, H * D, device=dev).to(bf), cache, meta, torch.rand(seqs * q_len, H, device=dev)

    q, cache, meta, gate = paged_case(PROMPT, PROMPT, 1)
    ms_like = _time_kernel(lambda: K.paged_attention(q, cache, meta, H, G, D, 0.09, None), flush=flush)
    seen = sum(min(i + 1, WIN) for i in range(PROMPT))
    by_flops("window_attention_prefill", _time_kernel(lambda: K.paged_attention(q, cache, meta, H, G, D, 1.1, WIN, gate=gate), flush=flush),
             4.0 * H * D * seen, like_flops("attention_prefill without a window", ms_like, 4.0 * H * D * PROMPT * PROMPT / 2))
    q, cache, meta, gate = paged_case(1, PROMPT, batch)
    ms_like = _time_kernel(lambda: K.paged_attention(q, cache, meta, H, G, D, 0.09, None), flush=flush)
    by_bytes("window_attention_decode", _time_kernel(lambda: K.paged_attention(q, cache, meta, H, G, D, 1.1, WIN, gate=gate), flush=flush),
             batch * WIN * 2 * G * D * 2, like_bytes("attention_decode without a window", ms_like, batch * PROMPT * 2 * G * D * 2))

    # -- latent attention with a sink beside the same kernel with a gate
    def latent_case(q_len, ctx, seqs):
        n = seqs * (ctx // 16)
        cache = torch.randn(n, 1, 1, 16, ROW, device=dev).to(bf)
        tbl = torch.arange(n, dtype=torch.int32, device=dev).view(seqs, ctx // 16)
        cu = torch.arange(seqs + 1, dtype=torch.int32, device=dev) * q_len
        meta = AttentionMeta(tbl, cu, torch.full((seqs,), ctx, dtype=torch.int32, device=dev),
                             torch.arange(seqs, dtype=torch.int32, device=dev).repeat_interleave(q_len), None, seqs, q_len, ctx, 16,
                             seqs if q_len == 1 else 0)
        return torch.randn(seqs * q_len, H, ROW, device=dev).to(bf), cache, meta, torch.rand(seqs * q_len, H, device=dev)

    sink = torch.zeros(H, device=dev)
    q, cache, meta, gate = latent_case(PROMPT, PROMPT, 1)
    ms_like = _time_kernel(lambda: K.latent_attention(q, cache, meta, H, ROW, R, 0.07, gate=gate), flush=flush)
    fl = 2.0 * H * (ROW + R) * PROMPT * PROMPT / 2
    by_flops("latent_attention_sink_prefill", _time_kernel(lambda: K.latent_attention(q, cache, meta, H, ROW, R, 0.07, sinks=sink), flush=flush), fl,
             like_flops("latent_attention with a gate", ms_like, fl))
    q, cache, meta, gate = latent_case(1, PROMPT, batch)
    ms_like = _time_kernel(lambda: K.latent_attention(q, cache, meta, H, ROW, R, 0.07, gate=gate), flush=flush)
    by_bytes("latent_attention_sink_decode", _time_kernel(lambda: K.latent_attention(q, cache, meta, H, ROW, R, 0.07, sinks=sink), flush=flush),
             batch * PROMPT * ROW * 2, like_bytes("latent_attention with a gate", ms_like, batch * PROMPT * ROW * 2))

    # -- the matrix memory beside the gated delta rule (the engine's other matrix-valued recurrence) at equal sizes
    MH, MD, MV = z["m_heads"], z["m_dim"], z["m_vdim"]
    cols = 2 * MH * MD + 2 * MH * MV + 2 * MH
    ib, fb, mnorm = torch.zeros(MH, device=dev), torch.full((MH,), 3.0, device=dev), torch.ones(MH * MV, device=dev)

    def memory_case(q_len, seqs):
        pr = torch.randn(seqs * q_len, cols, device=dev)
        cu = torch.arange(seqs + 1, dtype=torch.int32, device=dev) * q_len
        slots = torch.arange(seqs, dtype=torch.int32, device=dev)
        seq = slots.repeat_interleave(q_len)
        st = torch.zeros(seqs, MH * MD * (MV + 1) + MH, device=dev)
        return pr, cu, slots, seq, st

    def delta_case(q_len, seqs):
        qkv = torch.randn(seqs * q_len, 2 * MH * MD + MH * MV, device=dev).to(bf)
        pr = torch.randn(seqs * q_len, 2 * MH, device=dev)
        cu = torch.arange(seqs + 1, dtype=torch.int32, device=dev) * q_len
        slots = torch.arange(seqs, dtype=torch.int32, device=dev)
        st = torch.zeros(seqs, MH * MD * MV, device=dev)
        return qkv, pr, cu, slots, st

    alog, dtb = torch.zeros(MH, device=dev), torch.zeros(MH, device=dev)
    gcol = 2 * MH * MD + MH * MV
    for label, q_len, seqs in (("prefill", PROMPT, 1), ("decode", 1, batch)):
        pr, cu, slots, seq, st = memory_case(q_len, seqs)
        qkv, pr2, cu2, slots2, st2 = delta_case(q_len, seqs)
        state_bytes = seqs * MH * MD * (MV + 1) * 4 * 2
        io_bytes = seqs * q_len * (2 * MH * MD + MH * MV + MH * (MV + 1)) * 4
        ms_like = _time_kernel(lambda: K.delta_rule(qkv, pr2, 0, MH, alog, dtb, cu2, slots2, st2, MH, MH, MD, MV, 1e-6), flush=flush)
        lk = like_bytes("delta_rule", ms_like, seqs * MH * MD * MV * 8 + seqs * q_len * ((2 * MH * MD + MH * MV) * 2 + MH * MV * 4))
        by_bytes(f"mlstm_scan_{label}", _time_kernel(lambda: K.mlstm_scan(pr, gcol + MH * MV, gcol + MH * MV + MH, ib, fb, cu, slots, st, MH, MD, MV, 15.0), flush=flush),
                 state_bytes + io_bytes, lk)
        raw, top = K.mlstm_scan(pr, gcol + MH * MV, gcol + MH * MV + MH, ib, fb, cu, slots, st, MH, MD, MV, 15.0)
        o = torch.randn(seqs * q_len, MH * MV, device=dev)
        gam = torch.ones(MV, dtype=bf, device=dev)
        prg = torch.randn(seqs * q_len, MH * MV, device=dev)
        ms_like = _time_kernel(lambda: K.head_norm_gate(o, gam, 1e-6, prg, 0, MH, MV, bf), flush=flush)
        n_el = seqs * q_len * MH * MV
        by_bytes(f"mlstm_output_{label}", _time_kernel(lambda: K.mlstm_output(raw, top, mnorm, 1e-6, 1e-6, pr, gcol, MH, MD, MV, bf, seq, cu, slots, st), flush=flush),
                 n_el * (4 + 4 + 2), like_bytes("head_norm_gate", ms_like, n_el * (4 + 4 + 2)))

    # -- the router, and the experts beside the gated experts of the like design
    E, top_k, EF = z["experts"], z["top"], z["e_ff"]
    logits = torch.randn(T, E + 1, device=dev)
    corr = torch.zeros(E, device=dev)
    table = torch.rand(32768, E, device=dev).argsort(1)[:, :top_k].to(torch.int32).contiguous()
    tokens = torch.randint(0, 32768, (T,), device=dev, dtype=torch.int32)
    ms_like = _time_kernel(lambda: K.gather_rows(table, tokens), flush=flush)
    by_bytes("moe_route_top", _time_kernel(lambda: K.moe_route_top(logits, corr, E, top_k, z["groups"], z["keep"], 1e-20, shared_gate=True), flush=flush),
             T * ((E + 1) * 4 + top_k * 8 + 4), like_bytes("gather_rows of a choice table", ms_like, T * top_k * 8))
    chosen, wts, _ = K.moe_route_top(logits, corr, E, top_k, z["groups"], z["keep"], 1e-20, shared_gate=True)
    up, down = torch.randn(E, EF, W, device=dev).to(bf) * 0.02, torch.randn(E, W, EF, device=dev).to(bf) * 0.02
    gate_up = torch.randn(E, 2 * EF, W, device=dev).to(bf) * 0.02
    ms_like = _time_kernel(lambda: K.moe_experts(xb, chosen, gate_up, down, 1.0 / top_k, out_dtype=torch.float32), flush=flush)
    by_flops("routed_experts_prefill", _time_kernel(lambda: K.moe_experts(xb, chosen, up, down, 1.0, out_dtype=torch.float32, weights=wts, activation="relu2"), flush=flush),
             4.0 * T * top_k * EF * W, like_flops("gated experts chosen by table", ms_like, 6.0 * T * top_k * EF * W))
    xd, cd, wd = xb[:batch].contiguous(), chosen[:batch].contiguous(), wts[:batch].contiguous()
    touched = len(set(cd.flatten().tolist()))
    ms_like = _time_kernel(lambda: K.moe_experts(xd, cd, gate_up, down, 1.0 / top_k, out_dtype=torch.float32), flush=flush)
    by_bytes("routed_experts_decode", _time_kernel(lambda: K.moe_experts(xd, cd, up, down, 1.0, out_dtype=torch.float32, weights=wd, activation="relu2"), flush=flush),
             touched * 2 * EF * W * 2, like_bytes("gated experts chosen by table", ms_like, touched * 3 * EF * W * 2))
    out["kernels"]["routed_experts_decode"]["experts_touched"] = touched
    SF = z["shared"]
    u = torch.randn(T, SF, device=dev)
    gub = torch.randn(T, 2 * SF, device=dev).to(bf)
    sg = torch.rand(T, device=dev)
    ms_like = _time_kernel(lambda: K.silu_mul(gub), flush=flush)
    by_bytes("act_rows", _time_kernel(lambda: K.act_rows(u, "relu2", bf, row_scale=sg), flush=flush), T * SF * 6,
             like_bytes("silu_mul", ms_like, T * SF * 6))
    K.raise_on_abort()
    print(json.dumps(out))


# ---------------------------------------------------------------------------------------------------------
# --workload tibepel: the Tibepel design (chunked attention whose softmax weights are mixed across the heads beside a
# gated delta rule, mamba1 scans, clamped gated feed-forwards, a per-token side input, a float32 stream) at layer sizes that
# resemble real models, beside the Tufirax design of this engine - the closest one: attention and state-space layers
# around a float32 stream - at the same width, heads, feed-forward and depth; then each of the design's own kernels alone
# beside the like kernel of that path, with the bytes it has to move (or its FLOPs) over its time against the measured peaks.
# Random weights; its own JSON line.
TIBEPEL_SIZES = {
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, r_heads=16, r_kv=8, r_dim=128, r_vdim=128, inner=4096, state=16, dt_rank=128,
               m_heads=64, m_vdim=64, m_state=128, groups=8, rot=64, layers=8),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=14336, r_heads=32, r_kv=16, r_dim=128, r_vdim=128, inner=8192, state=16, dt_rank=256,
               m_heads=128, m_vdim=64, m_state=128, groups=8, rot=128, layers=8),
}
TIBEPEL_CHUNK = 4096       # positions per attention chunk (the prompts of this workload lie inside one chunk, as in the Tufirax run)


def tibepel_pair(size: dict, vocab: int = 32768):
    """(Tibepel configuration, Tufirax configuration) of equal width, attention heads, feed-forward and depth.  The Tibepel
    layers alternate side-by-side mixers and mamba1, the Tufirax layers attention and mamba2, each with a feed-forward."""
    par = {"type": "parallel",
           "mixer": {"left": {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": size["dim"], "vdim": size["dim"],
                              "scale": size["dim"] ** -0.5, "mask": {"size": TIBEPEL_CHUNK}}, "left_scale": 0.7,
                     "right": {"heads": size["r_heads"], "kv_heads": size["r_kv"], "dim": size["r_dim"], "vdim": size["r_vdim"], "conv": 4},
                     "right_scale": 0.7},
           "mlp": {"kind": "dense", "ff": size["ff"], "limit": 7.0}}
    mam = {"type": "mamba1", "mixer": {"inner": size["inner"], "state": size["state"], "dt_rank": size["dt_rank"], "conv": 4},
           "mlp": {"kind": "dense", "ff": size["ff"], "limit": 7.0}}
    tib = {"architecture": "Tibepel", "width": size["width"], "vocab": vocab, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
           "logit_softcap": 30.0, "token_side": {"dim": 64}, "layers": [par if i % 2 == 0 else mam for i in range(size["layers"])]}
    tfx = dict(width=size["width"], heads=size["heads"], kv_heads=size["kv_heads"], dim=size["dim"], rot=size["rot"], ff=size["ff"],
               m_heads=size["m_heads"], m_vdim=size["m_vdim"], state=size["m_state"], groups=size["groups"], layers=size["layers"])
    return tib, tufirax_pair(tfx, vocab)[0]


def run_tibepel(args):
    import torch

    from rvllm_b200 import LLM, config_from_dict
    from rvllm_b200.engine import StepEntry
    from rvllm_b200.kernels import AttentionMeta

    peaks = measured_peaks()
    PROMPT, CTX, batch = 2048, 4096, args.batch
    gen = torch.Generator().manual_seed(0)
    out = {"workload": "tibepel", "dtype": "bf16", "data": "synthetic", "peaks": peaks["source"], "prompt_len": PROMPT, "batch": batch,
           "steps": args.steps, "warmup": args.warmup, "models": {}, "kernels": {}}

    def measure(cfg_dict):
        config = config_from_dict(cfg_dict)
        llm = LLM(config=config, random_weights=True, seed=0, dtype="bfloat16", block_size=16, num_blocks=batch * (CTX // 16) + 8,
                  max_model_len=CTX, max_num_seqs=batch, max_num_batched_tokens=PROMPT, enforce_eager=args.eager)
        runner, V = llm.engine.runner, llm.engine.spec.vocab_size
        p = torch.randint(0, V, (PROMPT,), generator=gen).tolist()
        for _ in range(3):
            runner.step([StepEntry("w", p, [PROMPT - 1])])
            runner.finish("w")
        torch.cuda.synchronize()
        pf = []
        for _ in range(3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            runner.step([StepEntry("p", p, [PROMPT - 1])])
            b.record()
            torch.cuda.synchronize()
            runner.finish("p")
            pf.append(a.elapsed_time(b))
        ids = [f"d{i}" for i in range(batch)]
        for rid in ids:
            runner.step([StepEntry(rid, torch.randint(0, V, (PROMPT,), generator=gen).tolist(), [])])
        for _ in range(args.warmup):
            runner.step([StepEntry(r, [1], [0]) for r in ids])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            runner.step([StepEntry(r, [1], [0]) for r in ids])
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        for rid in ids:
            runner.finish(rid)
        kernels = llm.engine.kernels
        kernels.raise_on_abort()
        del llm
        torch.cuda.empty_cache()
        return {"prefill_ms": round(min(pf), 3), "prefill_tok_s": round(PROMPT / (min(pf) / 1e3), 1),
                "decode_ms_per_step": round(ms, 4), "decode_tok_s": round(batch / (ms / 1e3), 1)}, kernels

    K = None
    for name in (args.sizes.split(",") if args.sizes else list(TIBEPEL_SIZES)):
        tib, tfx = tibepel_pair(TIBEPEL_SIZES[name])
        a, K = measure(tib)
        b, K = measure(tfx)
        out["models"][name] = {"tibepel": a, "tufirax_same_size": b, "layers": TIBEPEL_SIZES[name]["layers"],
                               "prefill_ratio": round(a["prefill_tok_s"] / b["prefill_tok_s"], 3),
                               "decode_ratio": round(a["decode_tok_s"] / b["decode_tok_s"], 3)}
    if K is None:
        from rvllm_b200.kernels import get_library
        K = get_library("cuda:0")

    # ---- the design's kernels alone, at the "4k" sizes, beside the like kernel of the Tufirax path ----------------
    z = TIBEPEL_SIZES["4k"]
    dev, bf = "cuda", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    bw, peak = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12

    def by_bytes(name, ms, nbytes, like=None):
        out["kernels"][name] = {"ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / (ms / 1e3) / bw, 3)}
        if like is not None:
            out["kernels"][name]["like"] = like

    def like_bytes(kernel, ms, nbytes):
        return {"kernel": kernel, "ms": round(ms, 4), "frac_hbm": round(nbytes / (ms / 1e3) / bw, 3)}

    T, W, FF = PROMPT, z["width"], z["ff"]
    y, res = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev)
    g = torch.ones(W, dtype=bf, device=dev)
    gf = torch.ones(W, device=dev)
    ms_like = _time_kernel(lambda: K.residual_rmsnorm(y, g, 1e-6, res, bf), flush=flush)
    by_bytes("stream_add_norm", _time_kernel(lambda: K.stream_add_norm(res, y, (gf, 1e-6), bf), flush=flush), T * W * (4 + 4 + 4 + 2),
             like_bytes("residual_rmsnorm", ms_like, T * W * (4 + 4 + 4 + 2)))
    gu = torch.randn(T, 2 * FF, device=dev)
    ms_like = _time_kernel(lambda: K.act_mul(gu, "gelu_tanh", bf), flush=flush)
    by_bytes("act_mul_clamp", _time_kernel(lambda: K.act_mul(gu, "swiglu_clamp", bf, limit=7.0, alpha=1.702), flush=flush), T * FF * (8 + 2),
             like_bytes("act_mul_gelu", ms_like, T * FF * (8 + 2)))

    # attention: what follows the q/k/v product, one prompt of 2,048 tokens, and a decode step of `batch` sequences behind 2,048 tokens
    nh, nkv, hd = z["heads"], z["kv_heads"], z["dim"]
    pages = PROMPT // 16
    cache1 = torch.zeros(pages, 2, nkv, 16, hd, dtype=bf, device=dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * torch.tensor([500000.0 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64)[None, :]
    cos, sin = torch.cos(ang).float().to(dev), torch.sin(ang).float().to(dev)
    proj_qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=dev)
    ms_like = _time_kernel(lambda: K.rope_cache_write(proj_qkv, None, pos, cos, sin, pos, cache1, nh, nkv, hd, out_dtype=bf), flush=flush)
    by_bytes("kv_prepare", _time_kernel(lambda: K.kv_prepare(proj_qkv, pos, cache1, nh, nkv, hd, hd, 1e-6, bf), flush=flush),
             T * (nh + 2 * nkv) * hd * 6, like_bytes("rope_cache_write", ms_like, T * (nh + 2 * nkv) * hd * 6))
    r1, r2 = torch.full((nh,), 0.5, device=dev), torch.full((nh,), 0.3, device=dev)
    talk = (torch.eye(nh, device=dev) + 0.1 * torch.randn(nh, nh, device=dev)).contiguous()

    def attention_case(q_len, ctx, seqs):
        pages = seqs * (ctx // 16)
        cache = torch.randn(pages, 2, nkv, 16, hd, device=dev).to(bf)
        tables = torch.arange(pages, dtype=torch.int32, device=dev).view(seqs, ctx // 16)
        cu = torch.arange(seqs + 1, dtype=torch.int32, device=dev) * q_len
        meta = AttentionMeta(tables, cu, torch.full((seqs,), ctx, dtype=torch.int32, device=dev),
                             torch.arange(seqs, dtype=torch.int32, device=dev).repeat_interleave(q_len), None, seqs, q_len, ctx, 16,
                             seqs if q_len == 1 else 0)
        q = torch.randn(seqs * q_len, nh * hd, device=dev).to(bf)
        positions = (torch.arange(q_len, dtype=torch.int32, device=dev) + (ctx - q_len)).repeat(seqs)
        return q, cache, meta, positions

    q, cache, meta, positions = attention_case(PROMPT, PROMPT, 1)
    flops = 4.0 * nh * hd * PROMPT * PROMPT / 2
    ms_like = _time_kernel(lambda: K.paged_attention(q, cache, meta, nh, nkv, hd, hd ** -0.5, None), flush=flush)
    ms = _time_kernel(lambda: K.talking_attention(q, cache, meta, positions, nh, nkv, hd, hd, hd ** -0.5, r1, r2, talk, TIBEPEL_CHUNK), iters=3, flush=flush)
    out["kernels"]["talking_attention_prefill"] = {
        "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "frac_bf16": round(flops / (ms / 1e3) / peak, 3),
        "like": {"kernel": "attention_prefill", "ms": round(ms_like, 4), "frac_bf16": round(flops / (ms_like / 1e3) / peak, 3)}}
    q, cache, meta, positions = attention_case(1, PROMPT, batch)
    nbytes = batch * PROMPT * 2 * nkv * hd * 2
    ms_like = _time_kernel(lambda: K.paged_attention(q, cache, meta, nh, nkv, hd, hd ** -0.5, None), flush=flush)
    by_bytes("talking_attention_decode",
             _time_kernel(lambda: K.talking_attention(q, cache, meta, positions, nh, nkv, hd, hd, hd ** -0.5, r1, r2, talk, TIBEPEL_CHUNK), flush=flush),
             nbytes, like_bytes("attention_decode", ms_like, nbytes))

    # the recurrences: a 2,048-token prompt, and a decode step of `batch` sequences; beside the state-space scan of the Tufirax path
    H, P, N, G = z["m_heads"], z["m_vdim"], z["m_state"], z["groups"]
    m_inner, ch = H * P, H * P + 2 * G * N
    inner, N1, R = z["inner"], z["state"], z["dt_rank"]
    rh, rk, rd, rv = z["r_heads"], z["r_kv"], z["r_dim"], z["r_vdim"]
    for label, q_len, seqs in (("prefill", PROMPT, 1), ("decode", 1, batch)):
        rows = q_len * seqs
        cu = torch.arange(seqs + 1, dtype=torch.int32, device=dev) * q_len
        slots = torch.arange(seqs, dtype=torch.int32, device=dev)
        # the like kernel: the scan with one decay per head
        proj = torch.randn(rows, 2 * m_inner + 2 * G * N + H, device=dev)
        xbc = torch.randn(rows, ch, device=dev).to(bf)
        state = torch.zeros(seqs, H * N * P, device=dev)
        zeros_h, ones_h = torch.zeros(H, device=dev), torch.ones(H, device=dev)
        ms_like = _time_kernel(lambda: K.ssm_scan(xbc, proj, m_inner + ch, zeros_h, zeros_h, ones_h, cu, slots, state, H, P, N, G), flush=flush)
        like_b = rows * (ch * 2 + m_inner * 4) + seqs * H * N * P * 8
        like = dict(like_bytes("ssm_scan", ms_like, like_b), gflops=round(rows * H * P * N * 5 / ms_like / 1e6, 1))
        # mamba1: one state row per channel
        u = torch.randn(rows, inner, device=dev).to(bf)
        dt_raw, bc, zz = torch.randn(rows, inner, device=dev), torch.randn(rows, R + 2 * N1, device=dev), torch.randn(rows, 2 * inner, device=dev)
        A, dtb, dsk = -torch.rand(inner, N1, device=dev), torch.zeros(inner, device=dev), torch.ones(inner, device=dev)
        st1 = torch.zeros(seqs, inner * N1, device=dev)
        ms = _time_kernel(lambda: K.selective_scan(u, dt_raw, dtb, A, bc, R, R + N1, dsk, zz, inner, cu, slots, st1, bf), flush=flush)
        by_bytes(f"selective_scan_{label}", ms, rows * (inner * (2 + 4 + 4 + 2) + 2 * N1 * 4) + seqs * inner * N1 * 8 + inner * N1 * 4, like)
        out["kernels"][f"selective_scan_{label}"]["gflops"] = round(rows * inner * N1 * 6 / ms / 1e6, 1)
        # the gated delta rule
        qkv = torch.randn(rows, 2 * rk * rd + rh * rv, device=dev).to(bf)
        pr = torch.randn(rows, 2 * rh, device=dev)
        st2 = torch.zeros(seqs, rh * rd * rv, device=dev)
        al, db = torch.zeros(rh, device=dev), torch.zeros(rh, device=dev)
        ms = _time_kernel(lambda: K.delta_rule(qkv, pr, 0, rh, al, db, cu, slots, st2, rh, rk, rd, rv, 1e-6), flush=flush)
        by_bytes(f"delta_rule_{label}", ms, rows * ((2 * rk * rd + rh * rv) * 2 + rh * rv * 4 + 2 * rh * 4) + seqs * rh * rd * rv * 8, like)
        out["kernels"][f"delta_rule_{label}"]["gflops"] = round(rows * rh * rd * rv * 6 / ms / 1e6, 1)
        o = torch.randn(rows, rh * rv, device=dev)
        gate = torch.randn(rows, rh * rv, device=dev)
        gw = torch.ones(rv, dtype=bf, device=dev)
        yv, gproj, nw = torch.randn(rows, m_inner, device=dev), torch.randn(rows, m_inner, device=dev), torch.ones(m_inner, dtype=bf, device=dev)
        ms_like = _time_kernel(lambda: K.gated_group_rmsnorm(yv, gproj, nw, 1e-6, G, bf), flush=flush)
        by_bytes(f"head_norm_gate_{label}", _time_kernel(lambda: K.head_norm_gate(o, gw, 1e-6, gate, 0, rh, rv, bf), flush=flush),
                 rows * rh * rv * (4 + 4 + 2), like_bytes("gated_group_rmsnorm", ms_like, rows * m_inner * (4 + 4 + 2)))
    K.raise_on_abort()
    print(json.dumps(out))


def run_serve(args):
    print(json.dumps(serve_workload(args.shape, args.layers, args.requests, args.output_len, args.budget, args.eager)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (both numbers are reported)")
    ap.add_argument("--shape", default="llama-3.1-8b", choices=sorted(SHAPES), help="layer sizes of the model")
    ap.add_argument("--workload", default="decode", choices=["decode", "serve", "tufirax", "vipelix", "tibepel", "tugodra"],
                    help="decode: the benchmark's one JSON line; serve: continuous batching of uneven prompts; tufirax, vipelix, tibepel: "
                         "that design at real layer sizes beside the closest decoder of equal size, and its kernels alone")
    ap.add_argument("--sizes", default="", help="tufirax, vipelix, tibepel, tugodra: which sizes to run, with commas (default: all)")
    ap.add_argument("--requests", type=int, default=64, help="serve: number of requests")
    ap.add_argument("--output-len", type=int, default=256, help="serve: tokens generated per request")
    ap.add_argument("--budget", type=int, default=2048, help="serve: tokens per step")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--eager", action="store_true", help="no CUDA graphs")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Rust workspace packaged with "
                          "maturin; neither maturin nor cargo/rustc exists in this image, so pip cannot build it offline"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    ensure_built()
    if args.workload == "tufirax":
        run_tufirax(args)
    elif args.workload == "vipelix":
        run_vipelix(args)
    elif args.workload == "tibepel":
        run_tibepel(args)
    elif args.workload == "tugodra":
        run_tugodra(args)
    elif args.workload == "serve":
        run_serve(args)
    else:
        run_ours(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
