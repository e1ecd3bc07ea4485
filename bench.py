#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second, prefill, roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--shape NAME]
                    [--workload decode|serve] [--impl ours|reference]

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
    ap.add_argument("--workload", default="decode", choices=["decode", "serve"],
                    help="decode: the contract's line; serve: continuous batching of uneven prompts")
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
    if args.workload == "serve":
        run_serve(args)
    else:
        run_ours(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
