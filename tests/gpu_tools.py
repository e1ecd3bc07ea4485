"""Helpers of the GPU tests: a paged cache built from whole-sequence keys and values."""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from rvllm_b200.kernels import AttentionMeta


def paged_setup(k_seqs: Sequence[torch.Tensor], v_seqs: Sequence[torch.Tensor], q_lens: Sequence[int],
                page_size: int, dtype, seed: int = 0, spare_pages: int = 3, window: Optional[int] = None):
    """Scatter whole-sequence keys/values [ctx, nkv, hd] into shuffled pages.

    Returns (cache layer [pages, 2, nkv, page, hd], AttentionMeta).  The last q_len tokens of every
    sequence are the step's tokens.  With `window`, the pages that lie wholly below the window of a
    sequence's first query have been given back, as the cache manager does while a request runs:
    their block-table entries are -1 and their keys are nowhere in the cache."""
    dev = "cuda"
    B = len(k_seqs)
    nkv, hd = k_seqs[0].shape[1:]
    ctx_lens = [k.shape[0] for k in k_seqs]
    blocks = [(c + page_size - 1) // page_size for c in ctx_lens]
    MB = max(blocks)
    n_pages = sum(blocks) + spare_pages
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g).tolist()
    cache = torch.full((n_pages, 2, nkv, page_size, hd), float("nan"), dtype=torch.float32)
    table = torch.full((B, MB), -1, dtype=torch.int32)
    nxt = 0
    for b in range(B):
        first_seen = (ctx_lens[b] - q_lens[b]) - window + 1 if window else 0      # first key the first query sees
        for blk in range(blocks[b]):
            if (blk + 1) * page_size <= first_seen:
                continue                                                           # given back: the entry stays -1
            page = perm[nxt]
            nxt += 1
            table[b, blk] = page
            lo, hi = blk * page_size, min(ctx_lens[b], (blk + 1) * page_size)
            cache[page, 0, :, :hi - lo] = k_seqs[b][lo:hi].transpose(0, 1)
            cache[page, 1, :, :hi - lo] = v_seqs[b][lo:hi].transpose(0, 1)
    # unused slots hold finite junk, as a reused page would (NaN here would also catch a read
    # past ctx_len, but 0 * NaN in the masked part of a tile is not a fault of the kernel)
    cache = torch.where(torch.isnan(cache), torch.full_like(cache, 3.0), cache)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    token_seq = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(q_lens)])
    meta = AttentionMeta(table.to(dev), torch.tensor(cu, dtype=torch.int32, device=dev),
                         torch.tensor(ctx_lens, dtype=torch.int32, device=dev), token_seq.to(dev), None, B,
                         max(q_lens), max(ctx_lens), page_size, sum(1 for n in q_lens if n == 1))
    return cache.to(dev).to(dtype), meta


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    return float((got.double().cpu() - ref.double().cpu()).abs().max() / ref.double().abs().max())
