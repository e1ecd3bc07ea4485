"""Building replay traces for the four ways of cutting the same requests, and comparing what
a replay wrote with the plain implementation.

A request is a list of token ids.  Every schedule asks for the logits at EVERY position of every
request, so any schedule can be compared with the plain implementation position by position.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

ROUND = 64
TRACE_RUN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")


def run_trace_tool(folder: str, dtype: str, trace: "Trace", out_dir: str, block_size: int = 16, extra=(), timeout=900):
    """Replay `trace` with bin/trace_run in a process of its own, as a user runs it."""
    proc = subprocess.run([sys.executable, TRACE_RUN, "--model", folder, "--dtype", dtype, "--out", out_dir,
                           "--max-tokens", str(trace.max_tokens), "--block-size", str(block_size), *extra],
                          input=trace.lines(), capture_output=True, text=True, timeout=timeout)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert proc.stdout.splitlines() == [f"done {i}" for i in range(len(trace.steps))]
    return proc


def _round(n: int) -> int:
    return (n + ROUND - 1) // ROUND * ROUND


class Trace:
    def __init__(self):
        self.steps: List[dict] = []
        self.rows: Dict[int, List[Tuple[str, int]]] = {}     # step -> [(label, position)] in file order
        self._held: Dict[str, int] = {}
        self.max_tokens = 0
        self.preemptions = 0

    def add(self, entries: Sequence[Tuple[str, Sequence[int], int]], end: Sequence[str] = (), labels=None):
        """entries: (request id, its next tokens, position of the first of them).  `labels` maps a
        request id to the name its rows are filed under (default: the id itself); a request that
        is ended and fed again from position 0 files its first pass under "<id>#<pass>"."""
        step = len(self.steps)
        rec = {"step": step, "entries": [], "end": list(end)}
        rows = []
        for rid, toks, start in entries:
            rec["entries"].append({"id": rid, "tokens": list(map(int, toks)), "want": list(range(len(toks)))})
            label = (labels or {}).get(rid, rid)
            rows.extend((label, start + i) for i in range(len(toks)))
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


def schedule_mixed(requests: Dict[str, List[int]], live: int = 4, seed: int = 0, prompt_frac: float = 0.6,
                   preempt: int = 1, portions=(2, 3, 5, 8, 13, 21, 40)) -> Trace:
    """Up to `live` requests at a time: the first part of each request is fed in portions
    ("prompt"), the rest one token a step ("decode"); portions of some requests share steps with
    single tokens of others; a request may sit out a step; finished requests make room for the
    next ones, whose pages are the ones just given back.

    `preempt` live requests are, a few tokens into their decoding, ended while the others go on
    (what they hold is given back), wait until another request has taken pages, and are then fed
    again from position 0 under the same id - their earlier tokens as a prompt in portions, into
    pages that others have used since - as a scheduler does that pre-empts by recomputing.  The
    rows of the abandoned pass are filed under "<id>#0" and are compared too."""
    rng = np.random.RandomState(seed)
    t = Trace()
    waiting = list(requests.items())
    active: Dict[str, dict] = {}
    parked: List[Tuple[str, List[int], int]] = []         # pre-empted: (id, tokens, tokens it had been fed)
    preempted = set()
    left = preempt
    while waiting or active or parked:
        while (waiting or parked) and len(active) < live:
            if parked and (not waiting or parked[0][3] <= len(t.steps)):
                rid, toks, reached, _ = parked.pop(0)
                active[rid] = {"toks": toks, "pos": 0, "prompt": reached}
            elif waiting:
                rid, toks = waiting.pop(0)
                active[rid] = {"toks": toks, "pos": 0, "prompt": max(1, int(len(toks) * prompt_frac))}
            else:
                break
        entries, ended, labels = [], [], {}
        for rid, st in list(active.items()):
            if len(active) > 1 and rng.rand() < 0.2:
                continue                                   # left out of this step
            left_prompt = st["prompt"] - st["pos"]
            if left_prompt > 0:
                n = min(left_prompt, int(rng.choice(list(portions))))
                if left_prompt - n == 1:                   # never leave a portion of one token behind
                    n += 1
            else:
                n = 1
            entries.append((rid, st["toks"][st["pos"]:st["pos"] + n], st["pos"]))
            st["pos"] += n
            if st["pos"] == len(st["toks"]):
                ended.append(rid)
                del active[rid]
            elif (left > 0 and rid not in preempted and len(active) > 1 and st["pos"] >= st["prompt"] + 3
                  and len(st["toks"]) - st["pos"] > 8):
                # pre-empted: this pass ends here; its rows so far are re-filed as the abandoned pass
                left -= 1
                preempted.add(rid)
                for step_rows in t.rows.values():
                    for i, (label, pos) in enumerate(step_rows):
                        if label == rid:
                            step_rows[i] = (f"{rid}#0", pos)
                labels[rid] = f"{rid}#0"
                ended.append(rid)
                parked.append((rid, st["toks"], st["pos"], len(t.steps) + 3))
                del active[rid]
                t.preemptions += 1
        if entries:
            t.add(entries, end=ended, labels=labels)
        elif not active and parked and not waiting:
            parked[0] = parked[0][:3] + (0,)               # nothing else to run: bring it back now
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
    """Max-abs error of every written row against the plain logits of its position, relative to
    the largest |logit| OF THAT POSITION; on failure names the first wrong position (the place to
    start looking: a page's edge, the start of a portion ...).  Every position of every request
    must have been written; rows of an abandoned pass ("<id>#<n>") are compared as well."""
    worst = 0.0
    for rid, logits in ref.items():
        missing = [pos for pos in range(logits.shape[0]) if (rid, pos) not in got]
        assert not missing, f"{what}: request {rid} has no logits for positions {missing[:8]}"
    for (label, pos), g in sorted(got.items(), key=lambda kv: (kv[0][0], kv[0][1])):
        rid = label.split("#")[0]
        want = ref[rid][pos].numpy().astype(np.float64)
        scale = float(np.abs(want).max())
        assert np.isfinite(g).all(), f"{what}: request {label} position {pos} has non-finite logits"
        err = float(np.abs(g.astype(np.float64) - want).max()) / scale
        assert err <= tol, (f"{what}: request {label}, first wrong position {pos} of {ref[rid].shape[0]}: "
                            f"relative error {err:.3e} > {tol:.1e}")
        worst = max(worst, err)
    return worst


def position_errors(rows: Dict[Tuple[str, int], np.ndarray], ref: Dict[str, torch.Tensor]) -> Dict[Tuple[str, int], float]:
    """Max-abs error of each row against the plain logits, relative to the largest |logit| of its position."""
    out = {}
    for (label, pos), g in rows.items():
        want = ref[label.split("#")[0]][pos].numpy().astype(np.float64)
        out[(label, pos)] = float(np.abs(np.asarray(g, dtype=np.float64) - want).max() / np.abs(want).max())
    return out


def compare_bfloat16(got, ref: Dict[str, torch.Tensor], ref_rounded: Dict[str, torch.Tensor], what: str,
                     worst_factor: float = 1.5, median_factor: float = 1.25):
    """A bfloat16 engine against the plain logits, with the yardstick measured rather than guessed:
    `ref_rounded` are the plain implementation's logits with every stored activation rounded to
    bfloat16 (float64 arithmetic), so its error is what the precision costs by itself on these very
    requests.  The engine's error at any position may reach `worst_factor` times the yardstick's
    worst position, and its median over all positions `median_factor` times the yardstick's median
    (a kernel that loses precision of its own - sums kept in bfloat16, probabilities rounded twice -
    moves the median; a wrong key, page or row shows at its position)."""
    for rid, logits in ref.items():
        missing = [pos for pos in range(logits.shape[0]) if (rid, pos) not in got]
        assert not missing, f"{what}: request {rid} has no logits for positions {missing[:8]}"
    for key, g in got.items():
        assert np.isfinite(g).all(), f"{what}: request {key[0]} position {key[1]} has non-finite logits"
    yard = position_errors({(rid, pos): ref_rounded[rid][pos].numpy() for rid in ref for pos in range(ref[rid].shape[0])}, ref)
    errs = position_errors(got, ref)
    bound = worst_factor * max(yard.values())
    for (label, pos), e in sorted(errs.items()):
        assert e <= bound, (f"{what}: request {label}, first wrong position {pos}: relative error {e:.3e} > {bound:.3e} "
                            f"({worst_factor} x the worst error of bfloat16 storage alone)")
    med, yard_med = float(np.median(list(errs.values()))), float(np.median(list(yard.values())))
    assert med <= median_factor * yard_med, (f"{what}: median error {med:.3e} over {len(errs)} positions, but bfloat16 "
                                             f"storage alone gives {yard_med:.3e}: a kernel loses precision of its own")
    return max(errs.values()), bound
