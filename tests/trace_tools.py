"""Building replay traces for the four ways of cutting the same requests, and comparing what
a replay wrote with the plain implementation.

A request is a list of token ids.  Every schedule asks for the logits at EVERY position of every
request, so any schedule can be compared with the plain implementation position by position.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

ROUND = 64


def _round(n: int) -> int:
    return (n + ROUND - 1) // ROUND * ROUND


class Trace:
    def __init__(self):
        self.steps: List[dict] = []
        self.rows: Dict[int, List[Tuple[str, int]]] = {}     # step -> [(request, position)] in file order
        self._held: Dict[str, int] = {}
        self.max_tokens = 0

    def add(self, entries: Sequence[Tuple[str, Sequence[int], int]], end: Sequence[str] = ()):
        """entries: (request id, its next tokens, position of the first of them)."""
        step = len(self.steps)
        rec = {"step": step, "entries": [], "end": list(end)}
        rows = []
        for rid, toks, start in entries:
            rec["entries"].append({"id": rid, "tokens": list(map(int, toks)), "want": list(range(len(toks)))})
            rows.extend((rid, start + i) for i in range(len(toks)))
            self._held[rid] = self._held.get(rid, 0) + len(toks)
        self.max_tokens = max(self.max_tokens, sum(_round(n) for n in self._held.values()))
        for rid in end:
            self._held.pop(rid, None)
        self.steps.append(rec)
        self.rows[step] = rows

    def lines(self) -> str:
        return "".join(json.dumps(s) + "\n" for s in self.steps)


def schedule_whole(requests: Dict[str, List[int]]) -> Trace:
    """Each request alone and whole, in one step."""
    t = Trace()
    for rid, toks in requests.items():
        t.add([(rid, toks, 0)], end=[rid])
    return t


def schedule_bulk_tail(requests: Dict[str, List[int]], tail: int = 32) -> Trace:
    """Most of a request in one step, its last `tail` tokens one by one."""
    t = Trace()
    for rid, toks in requests.items():
        cut = max(0, len(toks) - tail)
        if cut:
            t.add([(rid, toks[:cut], 0)])
        for i in range(cut, len(toks)):
            t.add([(rid, toks[i:i + 1], i)], end=[rid] if i == len(toks) - 1 else [])
    return t


def schedule_portions(requests: Dict[str, List[int]], sizes=(7, 2, 16, 3, 5, 2, 33, 4)) -> Trace:
    """Each request alone, cut into portions of changing size, down to two tokens."""
    t = Trace()
    for rid, toks in requests.items():
        pos, k = 0, 0
        while pos < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - pos)
            k += 1
            t.add([(rid, toks[pos:pos + n], pos)], end=[rid] if pos + n == len(toks) else [])
            pos += n
    return t


def schedule_mixed(requests: Dict[str, List[int]], live: int = 4, seed: int = 0, prompt_frac: float = 0.6) -> Trace:
    """Up to `live` requests at a time: the first part of each request is fed in portions
    ("prompt"), the rest one token a step ("decode"); portions of some requests share steps with
    single tokens of others; a request may sit out a step; finished requests make room for the
    next ones, whose pages are the ones just given back."""
    rng = np.random.RandomState(seed)
    t = Trace()
    waiting = list(requests.items())
    active: Dict[str, dict] = {}
    while waiting or active:
        while waiting and len(active) < live:
            rid, toks = waiting.pop(0)
            active[rid] = {"toks": toks, "pos": 0, "prompt": max(1, int(len(toks) * prompt_frac))}
        entries, ended = [], []
        for rid, st in list(active.items()):
            if len(active) > 1 and rng.rand() < 0.2:
                continue                                   # left out of this step
            left_prompt = st["prompt"] - st["pos"]
            if left_prompt > 0:
                n = min(left_prompt, int(rng.choice([2, 3, 5, 8, 13, 21, 40])))
                if left_prompt - n == 1:                   # never leave a portion of one token behind
                    n += 1
            else:
                n = 1
            entries.append((rid, st["toks"][st["pos"]:st["pos"] + n], st["pos"]))
            st["pos"] += n
            if st["pos"] == len(st["toks"]):
                ended.append(rid)
                del active[rid]
        if entries:
            t.add(entries, end=ended)
    return t


def read_logits(out_dir: str, trace: Trace, vocab: int) -> Dict[Tuple[str, int], np.ndarray]:
    got = {}
    for step, rows in trace.rows.items():
        if not rows:
            continue
        arr = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4")
        assert arr.size == len(rows) * vocab, f"step {step}: {arr.size} floats for {len(rows)} rows of {vocab}"
        arr = arr.reshape(len(rows), vocab)
        for i, key in enumerate(rows):
            assert key not in got, f"position {key} written twice"
            got[key] = arr[i]
    return got


def compare(got: Dict[Tuple[str, int], np.ndarray], ref: Dict[str, torch.Tensor], tol: float, what: str):
    """Relative max-abs error per request against the plain logits; on failure names the first
    wrong position (the place to start looking: a page's edge, the start of a portion ...)."""
    worst = 0.0
    for rid, logits in ref.items():
        scale = float(logits.abs().max())
        for pos in range(logits.shape[0]):
            g = got[(rid, pos)]
            err = float(np.abs(g.astype(np.float64) - logits[pos].numpy()).max()) / scale
            assert np.isfinite(g).all(), f"{what}: request {rid} position {pos} has non-finite logits"
            assert err <= tol, (f"{what}: request {rid}, first wrong position {pos} of {logits.shape[0]}: "
                                f"relative error {err:.3e} > {tol:.1e}")
            worst = max(worst, err)
    return worst
