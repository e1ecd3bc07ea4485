"""The `rvllm` command line.

Sub-commands and option names follow the reference where it has them:

* `rvllm generate`  - its evaluation binary rvllm-eval (v3/crates/rvllm-bench/src/bin/rvllm_eval.rs:7-11,
  57-86,624-629): a prompt from --prompt or standard input, RVLLM_MAX_TOKENS (default 256), RVLLM_EOS;
  here also as options, and prompts may be given as token ids.
* `rvllm benchmark` - its `rvllm benchmark --model --n 1,32,64 --output-len 128 --max-model-len
  --gpu-memory-utilization --json` (bench_harness.py:21-30, deploy/bench_v2.sh:164-169) and the
  environment of rvllm-bench: RVLLM_MODEL_DIR, RVLLM_BATCH, RVLLM_ITERS, RVLLM_WARMUP
  (v3/crates/rvllm-bench/src/main.rs:5-20); one JSON line per batch size with the reference's keys
  {"batch", "iters", "tok_per_sec", "ms_per_step"} (main.rs:178-181).
* `rvllm info`, `rvllm random-weights`, `rvllm replay` have no counterpart there.

There is no `serve`: the HTTP server is outside this engine.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List, Optional


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def _engine_options(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--model", default=os.environ.get("RVLLM_MODEL_DIR"),
                    help="folder with config.json and model.safetensors (default: $RVLLM_MODEL_DIR)")
    ap.add_argument("--config", default=None, help="a config.json instead of a model folder, with --random-weights")
    ap.add_argument("--random-weights", action="store_true",
                    help="fill the model of --config with random weights on the device (N(0, 0.02), norms 1 + N(0, 0.1)) from --seed")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--device", default="cuda", help="cuda (the only device: the engine has no CPU path)")
    ap.add_argument("--max-model-len", type=int, default=None)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--max-num-batched-tokens", type=int, default=2048)
    ap.add_argument("--max-prefill-chunk", type=int, default=None)
    ap.add_argument("--block-size", type=int, default=int(os.environ.get("RVLLM_BLOCK_SIZE", 16)))
    ap.add_argument("--num-blocks", type=int, default=int(os.environ["RVLLM_NUM_BLOCKS"]) if "RVLLM_NUM_BLOCKS" in os.environ else None)
    ap.add_argument("--enforce-eager", action="store_true", default=os.environ.get("RVLLM_NO_GRAPH") == "1",
                    help="no CUDA graphs for decode steps (also RVLLM_NO_GRAPH=1)")
    ap.add_argument("--no-async-scheduling", action="store_true", default=os.environ.get("RVLLM_NO_ASYNC") == "1",
                    help="wait for every step's tokens before the next step is launched (also RVLLM_NO_ASYNC=1)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--capture-graphs", action="store_true",
                    help="capture the decode CUDA graphs of every batch and context bucket before the first request")


def _llm(args, **over):
    from . import LLM, config_from_dict
    if not str(args.device).startswith("cuda"):
        raise SystemExit(f"--device {args.device}: the engine runs its own CUDA kernels only and has no CPU path")
    if args.config and not args.random_weights:
        raise SystemExit("--config names no weights: add --random-weights, or give --model DIR")
    if args.random_weights and not args.config:
        raise SystemExit("--random-weights needs --config FILE (a config.json)")
    if not args.model and not args.config:
        raise SystemExit("no model: give --model DIR, set RVLLM_MODEL_DIR, or give --config FILE --random-weights")
    kw = dict(dtype=args.dtype, block_size=args.block_size, num_blocks=args.num_blocks,
              gpu_memory_utilization=args.gpu_memory_utilization, max_model_len=args.max_model_len,
              max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens,
              max_prefill_chunk=args.max_prefill_chunk, enforce_eager=args.enforce_eager, seed=args.seed,
              async_scheduling=not args.no_async_scheduling)
    kw.update(over)
    if args.config:
        with open(args.config) as f:
            llm = LLM(config=config_from_dict(json.load(f), args.config), random_weights=True, **kw)
    else:
        llm = LLM(args.model, **kw)
    if getattr(args, "capture_graphs", False):
        llm.capture_graphs()
    return llm


def cmd_generate(args) -> int:
    from . import SamplingParams
    prompts = []
    if args.prompt_ids:
        prompts = [_ids(p) for p in args.prompt_ids]
    elif args.prompt_ids_file:
        with open(args.prompt_ids_file) as f:
            prompts = [_ids(line) for line in f if line.strip()]
    elif args.prompt is not None or "RVLLM_PROMPT" in os.environ:
        prompts = [args.prompt if args.prompt is not None else os.environ["RVLLM_PROMPT"]]
    else:
        prompts = [sys.stdin.read()]
    llm = _llm(args)
    stops = tuple(_ids(args.eos)) if args.eos else ()
    sp = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                        seed=args.sampling_seed, max_tokens=args.max_tokens, stop_token_ids=stops,
                        ignore_eos=args.ignore_eos)
    t0 = time.perf_counter()
    outs = llm.generate(prompts, sp)
    dt = time.perf_counter() - t0
    for o in outs:
        c = o.outputs[0]
        rec = {"request_id": o.request_id, "prompt_tokens": len(o.prompt_token_ids), "token_ids": c.token_ids,
               "finish_reason": c.finish_reason}
        if c.text is not None:
            rec["text"] = c.text
        print(json.dumps(rec))
    n = sum(len(o.outputs[0].token_ids) for o in outs)
    print(f"generated {n} tokens in {dt:.3f} s ({n / dt:.1f} tok/s)", file=sys.stderr)
    return 0


def cmd_benchmark(args) -> int:
    import torch

    from . import SamplingParams
    batches = _ids(args.n) if args.n else [int(os.environ.get("RVLLM_BATCH", 128))]
    max_b = max(batches)
    need = args.input_len + args.output_len
    llm = _llm(args, max_num_seqs=max(args.max_num_seqs, max_b),
               max_num_batched_tokens=max(args.max_num_batched_tokens, max_b),
               max_model_len=args.max_model_len or need)
    vocab = llm.engine.spec.vocab_size
    gen = torch.Generator().manual_seed(args.seed)
    for b in batches:
        sp = SamplingParams(temperature=0.0, max_tokens=args.output_len, ignore_eos=True)
        for _ in range(b):
            llm.add_request(torch.randint(0, vocab, (args.input_len,), generator=gen).tolist(), sp)
        while llm.scheduler.waiting or any(r.remaining > 1 for r in llm.scheduler.running):
            llm.step()                                     # prefill is set-up, as in the reference's bench
        for _ in range(min(args.warmup, max(0, args.output_len - 2))):
            llm.step()
        iters = 0
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while llm.scheduler.has_unfinished() and (args.iters <= 0 or iters < args.iters):
            llm.step()
            iters += 1
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        for r in list(llm.scheduler.running):
            llm.scheduler.abort(r.req_id)
        rec = {"batch": b, "iters": iters, "tok_per_sec": round(b * iters / dt, 1), "ms_per_step": round(dt / max(iters, 1) * 1e3, 4)}
        print(json.dumps(rec) if args.json else
              f"bench: batch={b} iters={iters} -> {rec['tok_per_sec']:.0f} tok/s ({rec['ms_per_step']:.3f} ms/step)")
    return 0


def cmd_info(args) -> int:
    from . import load_config
    from .cache import CacheManager
    from .models import DecoderModel
    if not args.model:
        raise SystemExit("no model: give --model DIR or set RVLLM_MODEL_DIR")
    cfg = load_config(args.model)
    model = DecoderModel(cfg.to_spec())
    params = 0
    for name, ts in model.expected_tensors().items():
        n = 1
        for d in ts.shape:
            n *= d
        params += n
    import torch
    per_token = CacheManager.bytes_per_page(model.cache_needs(), 1, torch.bfloat16)
    print(json.dumps({"architecture": cfg.to_spec().architecture, "parameters": params,
                      "kv_bytes_per_token_bf16": per_token, "config": cfg.to_dict()}, indent=2))
    return 0


def cmd_random_weights(args) -> int:
    from . import config_from_dict, write_random_model
    with open(args.config) as f:
        cfg = config_from_dict(json.load(f), args.config)
    out = write_random_model(cfg, args.out, seed=args.seed, dtype={"bf16": "bfloat16", "fp32": "float32"}.get(args.dtype, args.dtype))
    print(out)
    return 0


def cmd_replay(args) -> int:
    from .engine.trace import build_engine, replay
    engine = build_engine(args.model, {"bf16": "bfloat16", "fp32": "float32"}.get(args.dtype, args.dtype),
                          args.max_tokens, args.block_size, max_live=args.max_live, graphs=args.graphs)
    with (open(args.trace) if args.trace else sys.stdin) as f:
        replay(engine, f, args.out, sys.stdout)
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="rvllm", description="LLM inference on one B200")
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate from prompts (token ids, or text with a tokenizer.json)")
    _engine_options(g)
    g.add_argument("--prompt", default=None, help="text prompt (default: $RVLLM_PROMPT, else standard input)")
    g.add_argument("--prompt-ids", action="append", help="a prompt as token ids, e.g. 1,2,3 (repeatable)")
    g.add_argument("--prompt-ids-file", help="one prompt of token ids per line")
    g.add_argument("--max-tokens", type=int, default=int(os.environ.get("RVLLM_MAX_TOKENS", 256)))
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--sampling-seed", type=int, default=None)
    g.add_argument("--eos", default=os.environ.get("RVLLM_EOS"), help="extra stop token ids, e.g. 2,151645 (also $RVLLM_EOS)")
    g.add_argument("--ignore-eos", action="store_true")
    g.set_defaults(fn=cmd_generate)

    b = sub.add_parser("benchmark", aliases=["bench"], help="decode throughput per batch size")
    _engine_options(b)
    b.add_argument("--n", default=None, help="batch sizes, e.g. 1,32,64 (default: $RVLLM_BATCH or 128)")
    b.add_argument("--input-len", type=int, default=int(os.environ.get("RVLLM_PREFILL_LEN", 16)))
    b.add_argument("--output-len", type=int, default=128)
    b.add_argument("--iters", type=int, default=int(os.environ.get("RVLLM_ITERS", 0)), help="timed steps (0: until done)")
    b.add_argument("--warmup", type=int, default=int(os.environ.get("RVLLM_WARMUP", 10)))
    b.add_argument("--json", action="store_true")
    b.set_defaults(fn=cmd_benchmark)

    i = sub.add_parser("info", help="parsed configuration, parameter count, cache bytes per token")
    i.add_argument("--model", default=os.environ.get("RVLLM_MODEL_DIR"))
    i.set_defaults(fn=cmd_info)

    r = sub.add_parser("random-weights", help="write a model folder with random weights from a config.json")
    r.add_argument("--config", required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    r.set_defaults(fn=cmd_random_weights)

    t = sub.add_parser("replay", help="feed a trace of token ids step by step and write logits (see bin/trace_run)")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", required=True, choices=["bfloat16", "float32", "bf16", "fp32"])
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, required=True)
    t.add_argument("--block-size", type=int, default=16)
    t.add_argument("--trace", default=None, help="file of JSON lines (default: standard input)")
    t.add_argument("--max-live", type=int, default=4, help="most requests live at a time")
    t.add_argument("--graphs", action="store_true", help="replay decode-only steps from CUDA graphs")
    t.set_defaults(fn=cmd_replay)

    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
