"""Run one kernel of the engine alone on a given shape and print its time and throughput.

    python -m rvllm_b200.kernels.microbench decode_gemm  --m 8 --n 28672 --k 4096 [--gated]
    python -m rvllm_b200.kernels.microbench prefill_gemm --m 2048 --n 6144 --k 4096 [--gated]
    python -m rvllm_b200.kernels.microbench decode_attention  --batch 32 --ctx 2048
    python -m rvllm_b200.kernels.microbench prefill_attention --tokens 2048 [--past 2048]
    python -m rvllm_b200.kernels.microbench sampling --batch 8 --n 128256

Used for timing a kernel in isolation (CUDA events, warm-up, inputs rotated so that L2 does not
help) and as the small, self-ending workload of a profiler capture.
"""
from __future__ import annotations

import argparse
import json

import torch


def timed(fns, iters: int, warmup: int = 3):
    for i in range(warmup):
        fns[i % len(fns)]()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        fns[i % len(fns)]()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def main(argv=None) -> int:
    from . import AttentionMeta, get_library
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["decode_gemm", "prefill_gemm", "decode_attention", "prefill_attention", "sampling"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=28672)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--gated", action="store_true")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--past", type=int, default=0, help="prefill_attention: keys already in the cache before the portion")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--splits", type=int, default=0, help="key splits of the decode attention (0: the library's choice)")
    ap.add_argument("--variant", default="", help="decode_attention: tma | cpasync | balanced | balanced_cpasync (default: the library's choice)")
    args = ap.parse_args(argv)
    K = get_library("cuda:0")
    torch.manual_seed(0)
    dev = "cuda"
    out = {"kernel": args.kernel}
    if args.kernel == "sampling":
        # temperature + top-k + top-p over `--batch` rows of `--n` logits; several sets of logits in turn
        R, V = args.batch, args.n
        sets = [torch.randn(R, V, device=dev) * 4 for _ in range(max(2, int(300e6 // (R * V * 4)) + 1))]
        t = torch.full((R,), 0.8, device=dev); tk = torch.full((R,), 50, device=dev, dtype=torch.int32)
        tp = torch.full((R,), 0.95, device=dev)
        seeds = torch.arange(R, device=dev, dtype=torch.int64); di = torch.zeros(R, device=dev, dtype=torch.int64)
        graphs = []
        for lg in sets:                       # one CUDA graph per set: device time without the host's launch cost
            K.sample(lg, t, tk, tp, seeds, di)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                K.sample(lg, t, tk, tp, seeds, di)
            graphs.append(g)
        ms = timed([g.replay for g in graphs], args.iters)
        out.update(rows=R, vocab=V, us=round(ms * 1e3, 2))
        print(json.dumps(out))
        return 0
    if args.kernel in ("decode_gemm", "prefill_gemm"):
        copies = max(2, int(300e6 // (args.n * args.k * 2)) + 1)
        ws = [(torch.randn(args.n, args.k, device=dev) * 0.02).bfloat16() for _ in range(copies)]
        x = torch.randn(args.m, args.k, device=dev).bfloat16()
        if args.kernel == "decode_gemm":
            fns = [(lambda w=w: K.linear_decode(x, w, gated=args.gated)) for w in ws]
        else:
            fns = [(lambda w=w: K.linear_tcgen05(x, w, gated=args.gated)) for w in ws]
        graphs = []
        for fn in fns:                        # one CUDA graph per copy of the weights: device time without the host's launch cost
            fn()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            graphs.append(g)
        ms = timed([g.replay for g in graphs], max(args.iters, 2 * len(graphs)))
        out.update(m=args.m, n=args.n, k=args.k, gated=args.gated, us=round(ms * 1e3, 2),
                   weight_gb_s=round(args.n * args.k * 2 / ms / 1e6, 1),
                   tflops=round(2 * args.m * args.n * args.k / ms / 1e9, 1))
    else:
        nh, nkv, hd, ps = args.heads, args.kv_heads, args.head_dim, args.page
        if args.kernel == "decode_attention":
            B, q_lens, ctx = args.batch, [1] * args.batch, args.ctx
        else:
            B, q_lens, ctx = 1, [args.tokens], args.tokens + args.past
        MB = (ctx + ps - 1) // ps
        # several copies of the cache in one layer, used in turn, so that L2 does not serve the keys
        kv_one = B * ctx * 2 * nkv * hd * 2
        copies = 1 if args.kernel != "decode_attention" else max(2, int(300e6 // kv_one) + 1)
        cache = torch.randn(copies * B * MB, 2, nkv, ps, hd, device=dev).bfloat16()
        bts = [(torch.arange(B * MB, dtype=torch.int32, device=dev) + c * B * MB).view(B, MB) for c in range(copies)]
        bt = bts[0]
        T = sum(q_lens)
        q = torch.randn(T, nh * hd, device=dev).bfloat16()
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev)
        ctxs = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        seq = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(q_lens)]).to(dev)
        meta = AttentionMeta(bt, cu, ctxs, seq, None, B, max(q_lens), ctx, ps, sum(1 for n in q_lens if n == 1))
        metas = [AttentionMeta(b, cu, ctxs, seq, None, B, max(q_lens), ctx, ps, sum(1 for n in q_lens if n == 1)) for b in bts]
        if args.kernel == "decode_attention" and (args.splits > 0 or args.variant):
            o = torch.empty_like(q)
            splits = args.splits or K.decode_splits(meta, nh, nkv)
            if args.variant == "balanced":
                fn = lambda m: K.flash_decode_balanced(q, cache, m, o, nh, nkv, hd, hd ** -0.5, None)
            elif args.variant == "balanced_cpasync":
                fn = lambda m: K.flash_decode_balanced(q, cache, m, o, nh, nkv, hd, hd ** -0.5, None, tma=False)
            else:
                fn = lambda m: K.decode_attention(q, cache, m, o, nh, nkv, hd, hd ** -0.5, None, num_splits=splits,
                                                  tma=args.variant != "cpasync")
        else:
            fn = lambda m: K.paged_attention(q, cache, m, nh, nkv, hd, hd ** -0.5, None)
        # one CUDA graph of several launches: device time without the host's launch cost
        for _ in range(2):
            fn(metas[0])
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(4):
                fn(metas[i % len(metas)])
        ms = timed([graph.replay], args.iters) / 4
        kv_bytes = B * ctx * 2 * nkv * hd * 2
        out.update(batch=B, ctx=ctx, heads=nh, kv_heads=nkv, head_dim=hd, us=round(ms * 1e3, 2))
        if args.kernel == "decode_attention":
            out.update(kv_gb_s=round(kv_bytes / ms / 1e6, 1), splits=args.splits or K.decode_splits(meta, nh, nkv))
        else:
            out.update(past=args.past, tflops=round(4 * nh * hd * (args.tokens * args.past + args.tokens * args.tokens / 2) / ms / 1e9, 1))
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
