"""Trace replay: feed given token ids through the engine step by step and write logits.

It samples nothing and owns no forward pass, cache or loader: every step goes through
`ModelRunner.step`, the same function generation uses.  Steps arrive as JSON lines

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step that wants logits, `<out>/<step>.f32` receives them as little-endian float32
[wanted, vocab] in the order of the entries and of `want`.  After every step `done <step>` is
printed and flushed.  The reference has nothing comparable; its nearest tools are the
token-by-token perplexity loop (v3/crates/rvllm-runtime/src/bring_up.rs:1265-1329) and a debug
dump of logits (bring_up.rs:854-875).
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO, Optional

import numpy as np

from ..config import EngineConfig, load_config
from .core import Engine
from .step import StepEntry

ROUND_TO = 64   # a request's tokens are counted in multiples of this when sizing the pool


def build_engine(model_dir: str, dtype: str, max_tokens: int, block_size: int = 16, device: str = "cuda:0",
                 max_live: int = 4, graphs: bool = False) -> Engine:
    """The engine a replay runs on: a pool of exactly `max_tokens` (rounded up) tokens, `max_live`
    request slots.  `graphs`: decode-only steps are replayed from CUDA graphs, as generation does by
    default; otherwise every step is launched kernel by kernel."""
    if ROUND_TO % block_size and block_size % ROUND_TO:
        raise ValueError(f"block_size {block_size} neither divides nor is a multiple of {ROUND_TO}")
    cfg = load_config(model_dir)
    unit = max(block_size, ROUND_TO)
    pool_tokens = ((max_tokens + unit - 1) // unit) * unit
    ec = EngineConfig(dtype=dtype, block_size=block_size, num_blocks=max(1, pool_tokens // block_size),
                      max_model_len=min(cfg.to_spec().max_position_embeddings, pool_tokens),
                      max_num_seqs=max_live, max_num_batched_tokens=max(pool_tokens, max_live),
                      enforce_eager=not graphs, device=device)
    return Engine(model_dir, engine_config=ec)


def replay(engine: Engine, lines: IO[str], out_dir: str, echo: Optional[IO[str]] = None) -> int:
    os.makedirs(out_dir, exist_ok=True)
    n = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in rec.get("entries", ())]
        logits = engine.runner.step(entries) if entries else None
        if logits is not None:
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            check = getattr(engine.kernels, "raise_on_abort", None)
            if check is not None:
                check()      # a kernel that gave up a bounded wait has written no result: fail, write nothing
            arr.tofile(os.path.join(out_dir, f"{step}.f32"))
        for rid in rec.get("end", ()):
            engine.runner.finish(rid)
        if echo is not None:
            echo.write(f"done {step}\n")
            echo.flush()
        n += 1
    return n


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token ids through the engine and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each request rounded up to 64)")
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--max-live", type=int, default=4, help="most requests live at a time (request slots)")
    ap.add_argument("--graphs", action="store_true",
                    help="replay decode-only steps from CUDA graphs, as generation does (default: every step eager)")
    args = ap.parse_args(argv)
    engine = build_engine(args.model, args.dtype, args.max_tokens, args.block_size, args.device,
                          max_live=args.max_live, graphs=args.graphs)
    replay(engine, sys.stdin, args.out, sys.stdout)
    return 0
