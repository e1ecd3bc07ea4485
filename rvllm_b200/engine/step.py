"""The step function: one batch of (request, its next tokens) through the model.

A batch holds, in any order, whole prompts, portions of prompts cut anywhere and single
decoded tokens.  The step reserves cache room for exactly the tokens it is given, packs the
batch's metadata into one pinned buffer that goes to the device in one copy, runs the model
over these tokens against the cache that earlier steps left, and returns float32 logits at
the wanted places.

The reference runs a step either as all-decode or as all-prefill of equal-length prompts
(v3/crates/rvllm-runtime/src/layer_exec.rs:32-39,367-372; scheduler.rs:1-6) and fills its
metadata with separate synchronous copies (bring_up.rs:698-708); its packed layout
(v3/crates/rvllm-metadata/src/layout.rs:19-55: token ids, positions, context lengths, block
tables, slot mapping, sequence starts; padding rows have slot -1, pack.rs:79-86) is what the
buffer here follows, extended per cache group.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager
from ..errors import KvExhausted, SchedulerError
from ..kernels.library import COUNTERS, AttentionMeta


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places (indices into `tokens`)
    whose logits are wanted."""
    req_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepContext:
    """What the parts see of a step."""
    __slots__ = ("kernels", "num_tokens", "num_seqs", "token_ids", "positions", "token_seq", "cu_seqlens",
                 "state_slots", "logit_rows", "attention", "q_lens", "ctx_lens", "req_ids", "extras")

    def __init__(self):
        self.extras = {}


class ModelRunner:
    def __init__(self, model, cache: CacheManager, kernels, max_model_len: int, device,
                 graph_batch_sizes: Sequence[int] = ()):
        self.model, self.cache, self.kernels = model, cache, kernels
        self.graph_batch_sizes = tuple(sorted(graph_batch_sizes))
        self._graphs = {}
        self._graph_pool = None
        self._graph_event = None
        self.max_model_len = max_model_len
        self.device = torch.device(device)
        self.max_blocks = cache.blocks_for(max_model_len)
        # a small ring of pinned staging buffers: a buffer is rewritten only after the copy that
        # last read it has finished, so the host never waits for the step it has just launched
        self._ring: List[Optional[torch.Tensor]] = [None, None, None]
        self._ring_events: List[Optional[object]] = [None, None, None]
        self._ring_next = 0
        self._dev: Optional[torch.Tensor] = None
        self.steps_run = 0
        self.last_h2d_bytes = 0

    # ---- metadata buffers --------------------------------------------------------------------
    def _buffers(self, n_ints: int):
        i = self._ring_next
        self._ring_next = (i + 1) % len(self._ring)
        if self._ring_events[i] is not None:
            self._ring_events[i].synchronize()
        size = max(n_ints, 1 << 16)
        if self._ring[i] is None or self._ring[i].numel() < n_ints:
            self._ring[i] = torch.empty((size,), dtype=torch.int32, pin_memory=self.device.type == "cuda")
        if self._dev is None or self._dev.numel() < n_ints:
            self._dev = torch.empty((size,), dtype=torch.int32, device=self.device)
        return i, self._ring[i], self._dev

    # ---- one step ----------------------------------------------------------------------------
    def validate(self, entries: Sequence[StepEntry]) -> None:
        vocab = self.model.spec.vocab_size
        seen = set()
        for e in entries:
            if e.req_id in seen:
                raise SchedulerError(f"request {e.req_id!r} appears twice in one step")
            seen.add(e.req_id)
            n_tok = len(e.tokens)
            if n_tok == 0:
                raise SchedulerError(f"request {e.req_id!r} brings no tokens to the step")
            if n_tok == 1:
                bad = [] if 0 <= e.tokens[0] < vocab else [e.tokens[0]]
            else:
                lo, hi = min(e.tokens), max(e.tokens)
                bad = [] if (0 <= lo and hi < vocab) else [t for t in e.tokens if not 0 <= int(t) < vocab]
            if bad:
                raise SchedulerError(f"request {e.req_id!r}: token id {bad[0]} is outside the vocabulary of {vocab}")
            have = self.cache.num_tokens(e.req_id) if self.cache.has(e.req_id) else 0
            if have + len(e.tokens) > self.max_model_len:
                raise SchedulerError(f"request {e.req_id!r}: {have} + {len(e.tokens)} tokens exceed max_model_len {self.max_model_len}")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise SchedulerError(f"request {e.req_id!r}: wanted place {w} is outside its {len(e.tokens)} tokens")

    def reserve(self, entries: Sequence[StepEntry]) -> List[int]:
        """Admit unknown requests and take the pages of the whole batch, or nothing."""
        cache = self.cache
        n_groups = len(cache.groups)
        total = [0] * n_groups
        new = 0
        for e in entries:
            known = cache.has(e.req_id)
            new += 0 if known else 1
            need = cache.pages_needed(e.req_id if known else None, len(e.tokens))
            for g in range(n_groups):
                total[g] += need[g]
        if any(total):
            for need, have in zip(total, cache.num_free_pages()):
                if need > have:
                    raise KvExhausted(need, have, "the step's tokens do not fit the free pages")
        if new > cache.slots.num_free:
            raise SchedulerError(f"{new} new requests but only {cache.slots.num_free} request slots are free")
        starts = []
        for e in entries:
            if not cache.has(e.req_id):
                cache.admit(e.req_id)
            starts.append(cache.append(e.req_id, len(e.tokens)))
        return starts

    def pack(self, entries: Sequence[StepEntry], starts: List[int], pad_to: Optional[int] = None,
             buffers=None, late=None, ctx_limit: Optional[int] = None) -> StepContext:
        """Write the step's metadata into a pinned buffer and send it to the device in one copy.

        With `pad_to` the batch is padded to that many one-token sequences (padding rows: token
        0, context length 0, slot -1, state slot -1 - they write nothing and attend to nothing;
        v3/crates/rvllm-metadata/src/pack.rs:35-40,79-86 of the reference pads the same way), block
        tables get the full width, and the layout depends on `pad_to` alone, so that a captured
        CUDA graph can be replayed on the buffer; `ctx_limit` is then the context length that the
        graph's kernels are laid out for (no sequence of the batch is longer).

        `late` = (sampled ids on the device, one index per entry): an entry with index j >= 0 is a
        one-token sequence whose token is sampled[j], which the host has not read; its token is
        put in place on the device after the copy."""
        cache = self.cache
        n_real = len(entries)
        B = pad_to if pad_to is not None else n_real
        q_lens = [len(e.tokens) for e in entries] + [1] * (B - n_real)
        T = sum(q_lens)
        ctx_lens = [s + n for s, n in zip(starts, q_lens)] + [0] * (B - n_real)
        wants = [list(e.want) for e in entries]
        if pad_to is not None:
            wants = [[0]] * B
        R = sum(len(w) for w in wants)
        G = len(cache.groups)
        MB = self.max_blocks if pad_to is not None else max(1, cache.blocks_for(max(ctx_lens)))
        n_ints = 3 * T + (B + 1) + 2 * B + R + G * (T + B * MB) + B + 16
        if buffers is None:
            ring_i, host, dev = self._buffers(n_ints)
        else:
            ring_i, (host, dev) = None, buffers
        h = host.numpy()
        off = 0

        def take(n):
            nonlocal off
            a = off
            off += n
            return a

        o_tok, o_pos, o_seq = take(T), take(T), take(T)
        o_cu, o_ctx, o_state, o_rows = take(B + 1), take(B), take(B), take(R)
        if pad_to is not None:
            return self._pack_decode(entries, starts, B, MB, h, host, dev,
                                     (o_tok, o_pos, o_seq, o_cu, o_ctx, o_state, o_rows), take, late,
                                     ctx_limit or self.max_model_len)
        cu = 0
        rows: List[int] = []
        h[o_cu] = 0
        for i in range(B):
            n = q_lens[i]
            if i < n_real:
                e = entries[i]
                h[o_tok + cu:o_tok + cu + n] = np.asarray(e.tokens, dtype=np.int32)
                h[o_pos + cu:o_pos + cu + n] = np.arange(starts[i], starts[i] + n, dtype=np.int32)
                h[o_state + i] = cache.state_slot(e.req_id)
            else:
                h[o_tok + cu] = 0
                h[o_pos + cu] = 0
                h[o_state + i] = -1
            h[o_seq + cu:o_seq + cu + n] = i
            rows.extend(cu + w for w in wants[i])
            cu += n
            h[o_cu + i + 1] = cu
            h[o_ctx + i] = ctx_lens[i]
        if R:
            h[o_rows:o_rows + R] = np.asarray(rows, dtype=np.int32)
        group_offsets = []
        ps = cache.page_size
        for gi in range(G):
            o_slot, o_bt = take(T), take(B * MB)
            h[o_bt:o_bt + B * MB] = -1
            h[o_slot:o_slot + T] = -1
            cu = 0
            for i, e in enumerate(entries):
                table = cache.block_table(e.req_id, gi)
                nb = len(table)
                tb = np.asarray(table, dtype=np.int32)
                h[o_bt + i * MB:o_bt + i * MB + nb] = tb
                pos = np.arange(starts[i], starts[i] + q_lens[i])
                h[o_slot + cu:o_slot + cu + q_lens[i]] = tb[pos // ps] * ps + pos % ps
                cu += q_lens[i]
            group_offsets.append((o_slot, o_bt))
        o_late = take(B)
        if late is not None:
            h[o_late:o_late + n_real] = late[1]
            h[o_late + n_real:o_late + B] = -1
        dev[:off].copy_(host[:off], non_blocking=True)
        self.last_h2d_bytes = off * 4
        if self.device.type == "cuda" and ring_i is not None:
            ev = self._ring_events[ring_i] or torch.cuda.Event()
            ev.record()
            self._ring_events[ring_i] = ev

        ctx = StepContext()
        ctx.kernels = self.kernels
        ctx.num_tokens, ctx.num_seqs = T, B
        ctx.token_ids = dev[o_tok:o_tok + T]
        ctx.positions = dev[o_pos:o_pos + T]
        ctx.token_seq = dev[o_seq:o_seq + T]
        ctx.cu_seqlens = dev[o_cu:o_cu + B + 1]
        if late is not None:
            self.kernels.late_tokens(ctx.token_ids, ctx.cu_seqlens, dev[o_late:o_late + B], late[0])
        dev_ctx = dev[o_ctx:o_ctx + B]
        ctx.state_slots = dev[o_state:o_state + B]
        ctx.logit_rows = dev[o_rows:o_rows + R]
        ctx.q_lens, ctx.ctx_lens = q_lens, ctx_lens
        ctx.req_ids = [e.req_id for e in entries]
        ctx.attention = []
        max_ctx = self.max_model_len if pad_to is not None else max(ctx_lens)
        for (o_slot, o_bt) in group_offsets:
            ctx.attention.append(AttentionMeta(
                block_tables=dev[o_bt:o_bt + B * MB].view(B, MB), cu_seqlens=ctx.cu_seqlens, ctx_lens=dev_ctx,
                token_seq=ctx.token_seq, slot_mapping=dev[o_slot:o_slot + T], num_seqs=B,
                max_q_len=max(q_lens), max_ctx_len=max_ctx, page_size=ps,
                num_decode=sum(1 for n in q_lens if n == 1)))
        return ctx

    def _pack_decode(self, entries, starts, B, MB, h, host, dev, offs, take, late=None, ctx_limit=None) -> StepContext:
        """`pack` for a padded batch of one-token sequences (T = R = B): whole-array writes."""
        cache = self.cache
        o_tok, o_pos, o_seq, o_cu, o_ctx, o_state, o_rows = offs
        n = len(entries)
        ar = np.arange(B + 1, dtype=np.int32)
        h[o_tok:o_tok + B] = 0
        h[o_pos:o_pos + B] = 0
        h[o_ctx:o_ctx + B] = 0
        h[o_state:o_state + B] = -1
        if n:
            h[o_tok:o_tok + n] = [e.tokens[0] for e in entries]
            h[o_pos:o_pos + n] = starts
            h[o_ctx:o_ctx + n] = np.asarray(starts, dtype=np.int32) + 1
            h[o_state:o_state + n] = [cache.state_slot(e.req_id) for e in entries]
        h[o_seq:o_seq + B] = ar[:B]
        h[o_cu:o_cu + B + 1] = ar
        h[o_rows:o_rows + B] = ar[:B]
        ps = cache.page_size
        group_offsets = []
        for gi in range(len(cache.groups)):
            o_slot, o_bt = take(B), take(B * MB)
            bt = h[o_bt:o_bt + B * MB].reshape(B, MB)
            bt[:] = -1
            h[o_slot:o_slot + B] = -1
            for i, e in enumerate(entries):
                table = cache.block_table(e.req_id, gi)
                bt[i, :len(table)] = table
                pos = starts[i]
                h[o_slot + i] = table[pos // ps] * ps + pos % ps
            group_offsets.append((o_slot, o_bt))
        o_late = take(B)
        off = o_late
        if late is not None:
            h[o_late:o_late + n] = late[1]
            h[o_late + n:o_late + B] = -1
            off = o_late + B
        dev[:off].copy_(host[:off], non_blocking=True)
        self.last_h2d_bytes = off * 4
        ctx = StepContext()
        ctx.kernels = self.kernels
        ctx.num_tokens, ctx.num_seqs = B, B
        ctx.token_ids = dev[o_tok:o_tok + B]
        ctx.positions = dev[o_pos:o_pos + B]
        ctx.token_seq = dev[o_seq:o_seq + B]
        ctx.cu_seqlens = dev[o_cu:o_cu + B + 1]
        if late is not None:
            self.kernels.late_tokens(ctx.token_ids, ctx.cu_seqlens, dev[o_late:o_late + B], late[0])
        dev_ctx = dev[o_ctx:o_ctx + B]
        ctx.state_slots = dev[o_state:o_state + B]
        ctx.logit_rows = dev[o_rows:o_rows + B]
        ctx.q_lens = [1] * B
        ctx.ctx_lens = [s + 1 for s in starts] + [0] * (B - n)
        ctx.req_ids = [e.req_id for e in entries]
        ctx.attention = [AttentionMeta(
            block_tables=dev[o_bt:o_bt + B * MB].view(B, MB), cu_seqlens=ctx.cu_seqlens, ctx_lens=dev_ctx,
            token_seq=ctx.token_seq, slot_mapping=dev[o_slot:o_slot + B], num_seqs=B, max_q_len=1,
            max_ctx_len=ctx_limit or self.max_model_len, page_size=ps, num_decode=B) for (o_slot, o_bt) in group_offsets]
        return ctx

    def step(self, entries: Sequence[StepEntry], late_tokens=None) -> Optional[torch.Tensor]:
        """Run the batch.  Returns float32 logits [wanted places, vocab] in the order of the
        entries and of each entry's `want` (None if nothing is wanted).

        `late_tokens` = (ids, index): ids is an int32 tensor on the device (what the previous step
        sampled), index has one number per entry; an entry with index j >= 0 brings one token whose
        value is ids[j] and is not known on the host yet (its `tokens` holds a stand-in)."""
        if not entries:
            return None
        self.validate(entries)
        if late_tokens is not None:
            if len(late_tokens[1]) != len(entries):
                raise SchedulerError(f"{len(entries)} entries but {len(late_tokens[1])} late-token indices")
            for e, j in zip(entries, late_tokens[1]):
                if j >= 0 and len(e.tokens) != 1:
                    raise SchedulerError(f"request {e.req_id!r}: a late token stands for exactly one token")
            if all(j < 0 for j in late_tokens[1]):
                late_tokens = None
        starts = self.reserve(entries)
        bucket = self._graph_bucket(entries)
        if bucket is not None:
            logits = self._step_graph(entries, starts, bucket, late_tokens)
        else:
            ctx = self.pack(entries, starts, late=late_tokens)
            hidden = self.model.forward(ctx, self.cache)
            logits = self.model.compute_logits(hidden, ctx) if ctx.logit_rows.numel() else None
        for e in entries:
            self.cache.release_passed(e.req_id)
        self.steps_run += 1
        return logits

    # ---- decode steps replayed from CUDA graphs -------------------------------------------------
    def _graph_bucket(self, entries: Sequence[StepEntry]) -> Optional[int]:
        """The batch-size bucket whose graph can run this step: every entry brings one token and
        wants its logits, and a bucket is large enough."""
        if not self.graph_batch_sizes or self.device.type != "cuda":
            return None
        if not getattr(self.model, "graph_safe", True):
            return None                       # a part of this model cannot be captured: every step runs eagerly
        for e in entries:
            if len(e.tokens) != 1 or len(e.want) != 1:
                return None
        for b in self.graph_batch_sizes:
            if b >= len(entries):
                return b
        return None

    def _ctx_bucket(self, longest: int) -> int:
        """The context length a graph is laid out for: 512, 768, 1024, 1536, 2048, ... (the attention
        kernel's split of the keys depends on it), at most max_model_len."""
        b = 512
        while b < longest:
            b = b * 3 // 2 if (b & (b - 1)) == 0 else b // 3 * 4
        return min(b, self.max_model_len)

    def _step_graph(self, entries, starts, bucket: int, late=None) -> torch.Tensor:
        ctx_limit = self._ctx_bucket(max(starts) + 1)
        bucket = (bucket, ctx_limit)
        state = self._graphs.get(bucket)
        if state is None:
            # the first step of a bucket runs eagerly: it loads every kernel library and lets the
            # GEMM library set itself up; the graph is captured right after it for later steps
            ctx = self.pack(entries, starts, late=late)
            hidden = self.model.forward(ctx, self.cache)
            logits = self.model.compute_logits(hidden, ctx)
            self._graphs[bucket] = self._capture(*bucket)
            return logits
        host, dev, graph, out, launches = state
        self._graph_event.synchronize()
        self.pack(entries, starts, pad_to=bucket[0], buffers=(host, dev), late=late, ctx_limit=ctx_limit)
        self._graph_event.record()
        graph.replay()
        COUNTERS["launches"] += launches       # the kernels of this project inside the replayed graph
        return out[:len(entries)]

    def _capture(self, bucket: int, ctx_limit: int):
        G = len(self.cache.groups)
        n_ints = 3 * bucket + (bucket + 1) + 2 * bucket + bucket + G * (bucket + bucket * self.max_blocks) + bucket + 16
        host = torch.empty((n_ints,), dtype=torch.int32, pin_memory=True)
        dev = torch.empty((n_ints,), dtype=torch.int32, device=self.device)
        ctx = self.pack([], [], pad_to=bucket, buffers=(host, dev), ctx_limit=ctx_limit)   # all rows padded: writes nothing
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        before = COUNTERS["launches"]
        with torch.cuda.graph(graph, pool=self._graph_pool):
            hidden = self.model.forward(ctx, self.cache)
            out = self.model.compute_logits(hidden, ctx)
        launches = COUNTERS["launches"] - before
        COUNTERS["launches"] = before          # captured, not run
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        if self._graph_event is None:
            self._graph_event = torch.cuda.Event()
            self._graph_event.record()
        return host, dev, graph, out, launches

    def capture_decode_graphs(self, max_context: Optional[int] = None, batch_sizes: Optional[Sequence[int]] = None) -> int:
        """Capture the decode graphs ahead of time, for every batch bucket (or the given ones) and
        every context bucket up to `max_context` (default: max_model_len), so that no step of a
        running service pays for a capture.  A graph is captured on a batch of padding rows, which
        write nothing, so live requests are not disturbed.  Returns the number of graphs captured."""
        if not self.graph_batch_sizes or self.device.type != "cuda" or not getattr(self.model, "graph_safe", True):
            return 0
        limit = min(max_context or self.max_model_len, self.max_model_len)
        ctx_buckets, b = [], self._ctx_bucket(1)
        while True:
            ctx_buckets.append(b)
            if b >= limit:
                break
            b = self._ctx_bucket(b + 1)
        made = 0
        for bucket in (batch_sizes or self.graph_batch_sizes):
            if bucket not in self.graph_batch_sizes:
                raise SchedulerError(f"{bucket} is not one of the graph batch sizes {self.graph_batch_sizes}")
            for ctx_limit in ctx_buckets:
                if (bucket, ctx_limit) not in self._graphs:
                    # a first, uncaptured run of the padded batch: it loads the kernel libraries
                    # and lets the GEMM library choose its algorithms outside the capture
                    G = len(self.cache.groups)
                    n_ints = 3 * bucket + (bucket + 1) + 2 * bucket + bucket + G * (bucket + bucket * self.max_blocks) + bucket + 16
                    host = torch.empty((n_ints,), dtype=torch.int32, pin_memory=True)
                    dev = torch.empty((n_ints,), dtype=torch.int32, device=self.device)
                    ctx = self.pack([], [], pad_to=bucket, buffers=(host, dev), ctx_limit=ctx_limit)
                    self.model.compute_logits(self.model.forward(ctx, self.cache), ctx)
                    self._graphs[(bucket, ctx_limit)] = self._capture(bucket, ctx_limit)
                    made += 1
        return made

    def finish(self, req_id: Hashable) -> None:
        """Give back everything the request holds."""
        if self.cache.has(req_id):
            self.cache.free(req_id)
