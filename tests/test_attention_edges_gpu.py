"""Attention kernels where random inputs would hide a fault: one key made to dominate, placed at
page edges, tile edges and the edges of every query's window, for the kernels that serve real
prompts (tcgen05 prefill attention at head sizes 64 and 128, the flash tilings, the evenly cut
decode kernel), with the pages below the window given back (block-table entries of -1) - and long
contexts: tens of thousands of keys, block tables too long for the kernels' shared-memory copy,
up to 64 key splits, hundreds of (sequence, kv head) pairs of unequal length."""
import math

import pytest
import torch

from gpu_tools import paged_setup, rel_err

pytestmark = pytest.mark.gpu

BF16_TOL = 1e-2


@pytest.fixture(scope="module")
def K():
    from rvllm_b200.kernels import get_library
    return get_library("cuda:0")


def marked_sequence(ctx, nkv, hd, target, seed, strength=12.0):
    """Keys and values of one sequence in which key `target` points along a direction that every
    query of the test uses (as `direction * strength`): its score is strength^2 * scale against
    scores near zero (144 / sqrt(hd) is enough among hundreds of keys; tens of thousands need more)."""
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(ctx, nkv, hd, generator=g) * 0.1
    v = torch.randn(ctx, nkv, hd, generator=g)
    direction = torch.randn(hd, generator=g)
    direction /= direction.norm()
    k[target] = direction * strength
    return k, v, direction


def hits(out, v_target, nh, nkv):
    """Per (token, head): whether the output is the marked key's value row."""
    T = out.shape[0]
    want = v_target.repeat_interleave(nh // nkv, dim=0)                   # [nh, hd]
    return ((out.view(T, nh, -1).float().cpu() - want.float()[None]).abs().amax(-1) < 0.1)


PREFILL_EDGE_CASES = [
    # nh, nkv, hd, page, ctx, q_len, window, targets
    (8, 2, 128, 16, 900, 200, None, (0, 15, 16, 63, 64, 511, 512, 699, 700, 731, 732, 899)),
    (8, 2, 128, 16, 900, 200, 128, (573, 574, 604, 605, 636, 637, 640, 700, 772, 899)),
    (4, 4, 64, 8, 400, 130, 200, (71, 72, 127, 128, 199, 200, 270, 271, 399)),
    (16, 1, 128, 32, 300, 24, 64, (213, 214, 235, 236, 276, 299)),
    (2, 2, 64, 64, 1200, 16, 1000, (185, 186, 200, 1183, 1184, 1199)),
]


@pytest.mark.parametrize("case", PREFILL_EDGE_CASES)
def test_prompt_portions_see_exactly_the_keys_of_their_windows(K, case):
    """Query i of the portion (position p) must return the marked key's value if and only if
    p - window < target <= p.  The targets put that edge on the first and last query of the 128-row
    tiles of the tcgen05 kernel and of the 64-row tiles of the flash kernel, and the key itself on
    page and 64-key tile edges."""
    nh, nkv, hd, page, ctx, q_len, window, targets = case
    scale = 1 / math.sqrt(hd)
    first = ctx - q_len
    for target in targets:
        k, v, direction = marked_sequence(ctx, nkv, hd, target, seed=target)
        cache, meta = paged_setup([k], [v], [q_len], page, torch.bfloat16, seed=target, window=window)
        if window:
            freed = int((meta.block_tables[0] < 0).sum())
            assert freed == max(0, (first - window + 1)) // page, "pages below the first window are given back"
        q = (direction * 12.0).repeat(q_len, nh, 1).reshape(q_len, nh * hd).cuda().bfloat16()
        pos = torch.arange(first, ctx)
        expect = (target <= pos) & ((pos - window < target) if window else torch.ones_like(pos, dtype=torch.bool))
        expect = expect[:, None].expand(q_len, nh)
        vt = v[target].bfloat16()
        outs = {"dispatch": K.paged_attention(q, cache, meta, nh, nkv, hd, scale, window),
                "plain": K.paged_attention_plain(q, cache, meta, nh, nkv, hd, scale, window)}
        o = torch.zeros_like(q)
        outs["flash, prefill tiling"] = K.flash_attention(q, cache, meta, o, nh, nkv, hd, scale, window, mode=0)
        if 128 % (nh // nkv) == 0 and page >= 8:
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            o = torch.zeros_like(q)
            outs["tcgen05"] = K.attention_tcgen05(q, cache, meta, o, nh, nkv, hd, scale, window, status=status)
            assert int(status.item()) == 0
        for name, out in outs.items():
            got = hits(out, vt, nh, nkv)
            wrong = (got != expect).nonzero()
            assert wrong.numel() == 0, (f"{name}, key {target}: query {int(wrong[0, 0])} (position {first + int(wrong[0, 0])}), "
                                        f"head {int(wrong[0, 1])} {'missed' if bool(expect[wrong[0, 0], wrong[0, 1]]) else 'saw'} it")
            assert torch.isfinite(out.float()).all()


DECODE_EDGE_CASES = [
    # nh, nkv, hd, page, window, contexts
    (32, 8, 128, 16, None, (1, 64, 65, 777, 1500, 2049)),
    (32, 8, 128, 16, 256, (1, 255, 256, 257, 300, 1024, 2049)),
    (8, 2, 64, 8, 100, (99, 100, 101, 164, 165, 900)),
]


@pytest.mark.parametrize("case", DECODE_EDGE_CASES)
def test_decoding_tokens_see_exactly_the_keys_of_their_windows(K, case):
    """One-token sequences of many lengths in one batch; in each the marked key sits once on the
    near and once on the far side of the window's edge (or, without a window, on the first key, a
    page edge and a tile edge).  Through the dispatch, the split kernel with several split counts
    and the evenly cut kernel with several grids; pages below the windows given back."""
    nh, nkv, hd, page, window, contexts = case
    scale = 1 / math.sqrt(hd)
    for variant in range(3):
        ks, vs, qs, expect, vts = [], [], [], [], []
        for i, ctx in enumerate(contexts):
            p = ctx - 1
            if window:
                target = max(0, p - window + 1) if variant == 0 else (p - window if variant == 1 and p - window >= 0 else p)
            else:
                target = (0, (ctx // 2) // page * page, max(0, ctx - 1 - (ctx - 1) % 64))[variant]
            k, v, d = marked_sequence(ctx, nkv, hd, target, seed=100 * variant + i)
            ks.append(k); vs.append(v); qs.append((d * 12.0).repeat(nh, 1).reshape(1, nh * hd))
            expect.append(target <= p and (not window or p - window < target))
            vts.append(v[target].bfloat16())
        B = len(contexts)
        cache, meta = paged_setup(ks, vs, [1] * B, page, torch.bfloat16, seed=variant, window=window)
        q = torch.cat(qs).cuda().bfloat16()
        outs = {"dispatch": K.paged_attention(q, cache, meta, nh, nkv, hd, scale, window),
                "plain": K.paged_attention_plain(q, cache, meta, nh, nkv, hd, scale, window)}
        for splits in (1, 2, 7, 33):
            o = torch.zeros_like(q)
            outs[f"split in {splits}"] = K.flash_attention(q, cache, meta, o, nh, nkv, hd, scale, window, mode=1, num_splits=splits)
        for ctas in (0, 5, 148):
            o = torch.zeros_like(q)
            outs[f"evenly cut over {ctas or 'all'} CTAs"] = K.flash_decode_balanced(q, cache, meta, o, nh, nkv, hd, scale, window, ctas=ctas)
        for name, out in outs.items():
            for i in range(B):
                got = bool(hits(out[i:i + 1], vts[i], nh, nkv).all())
                none = not bool(hits(out[i:i + 1], vts[i], nh, nkv).any())
                assert (got if expect[i] else none), f"{name}, variant {variant}: the sequence of {contexts[i]} keys {'missed' if expect[i] else 'saw'} its marked key"


def rows_reference(k, v, q_rows, positions, scale, window, nh):
    """float64 attention of a few query rows [n, nh, hd] at the given positions over the whole
    sequence k, v [ctx, nkv, hd] (computed on the GPU: torch as an array library)."""
    k, v, q_rows = k.cuda().double(), v.cuda().double(), q_rows.cuda().double()
    nkv = k.shape[1]
    out = torch.zeros_like(q_rows)
    idx = torch.arange(k.shape[0], device="cuda")
    for i, p in enumerate(positions):
        ok = idx <= p
        if window:
            ok &= idx > p - window
        for h in range(nh):
            g = h * nkv // nh
            s = (k[:, g] @ q_rows[i, h]) * scale
            s = s.masked_fill(~ok, float("-inf"))
            out[i, h] = torch.softmax(s, 0) @ v[:, g]
    return out.cpu()


@pytest.mark.parametrize("ctx,page,window", [(8192, 16, None), (20000, 16, None), (32768, 16, None), (32768, 16, 4096),
                                             (5000, 4, None), (9000, 4, 3000)])
def test_decode_attention_over_long_contexts(K, ctx, page, window):
    """One and two sequences of up to 32,768 keys: block tables of more than 1,024 pages (not kept
    in shared memory), up to 64 key splits by the policy, and a dominating key far back."""
    nh, nkv, hd = 8, 2, 128
    scale = 1 / math.sqrt(hd)
    torch.manual_seed(ctx + page)
    contexts = [ctx, ctx // 3 + 1]
    bf = lambda t: t.bfloat16().float()
    ks = [bf(torch.randn(c, nkv, hd)) for c in contexts]
    vs = [bf(torch.randn(c, nkv, hd)) for c in contexts]
    q = bf(torch.randn(2, nh, hd))
    cache, meta = paged_setup(ks, vs, [1, 1], page, torch.bfloat16, window=window)
    assert (meta.max_blocks > 1024) == (ctx > 1024 * page)      # most cases: a block table too long for shared memory
    qd = q.reshape(2, nh * hd).cuda().bfloat16()
    ref = torch.cat([rows_reference(ks[i], vs[i], q[i:i + 1], [contexts[i] - 1], scale, window, nh) for i in range(2)])
    plain = K.paged_attention_plain(qd, cache, meta, nh, nkv, hd, scale, window)
    assert rel_err(plain.view(2, nh, hd), ref) < BF16_TOL
    assert K.decode_splits(meta, nh, nkv) > 16 or ctx < 20000
    out = K.paged_attention(qd, cache, meta, nh, nkv, hd, scale, window)
    assert rel_err(out.view(2, nh, hd), ref) < BF16_TOL
    for splits in (1, 16, 41, 64):
        o = torch.zeros_like(qd)
        K.flash_attention(qd, cache, meta, o, nh, nkv, hd, scale, window, mode=1, num_splits=splits)
        assert rel_err(o.view(2, nh, hd), ref) < BF16_TOL, f"{splits} splits"
    for ctas in (0, 31):
        o = torch.zeros_like(qd)
        K.flash_decode_balanced(qd, cache, meta, o, nh, nkv, hd, scale, window, ctas=ctas)
        assert rel_err(o.view(2, nh, hd), ref) < BF16_TOL, f"evenly cut over {ctas} CTAs"
    # a dominating key far back: the very first key seen, a page edge beyond the first 1,024 pages
    # (where the context has that many), a tile edge near the end
    p = ctx - 1
    first_seen = (p - window + 1) if window else 0
    far_edge = -(-max(first_seen, min(1030 * page, p - 200)) // page) * page
    for target in (first_seen, far_edge, p - 64):
        k, v, d = marked_sequence(ctx, nkv, hd, target, seed=target, strength=16.0)
        cache, meta = paged_setup([k], [v], [1], page, torch.bfloat16, seed=1, window=window)
        q1 = (d * 16.0).repeat(nh, 1).reshape(1, nh * hd).cuda().bfloat16()
        for name, out in (("dispatch", K.paged_attention(q1, cache, meta, nh, nkv, hd, scale, window)),
                          ("evenly cut", K.flash_decode_balanced(q1, cache, meta, torch.zeros_like(q1), nh, nkv, hd, scale, window))):
            assert bool(hits(out, v[target].bfloat16(), nh, nkv).all()), f"{name}: key {target} of {ctx} was not found"


def test_evenly_cut_decode_kernel_with_hundreds_of_uneven_pairs(K):
    """40 sequences x 8 kv heads = 320 (sequence, kv head) pairs of 1 to 3,000 keys: the kernel the
    engine takes from 256 pairs on, against the plain kernel and, for some rows, float64."""
    nh, nkv, hd, page = 32, 8, 128, 16
    scale = 1 / math.sqrt(hd)
    g = torch.Generator().manual_seed(9)
    contexts = [1, 2, 63, 64, 65, 3000] + torch.randint(1, 3000, (34,), generator=g).tolist()
    bf = lambda t: t.bfloat16().float()
    ks = [bf(torch.randn(c, nkv, hd, generator=g)) for c in contexts]
    vs = [bf(torch.randn(c, nkv, hd, generator=g)) for c in contexts]
    B = len(contexts)
    q = bf(torch.randn(B, nh, hd, generator=g))
    cache, meta = paged_setup(ks, vs, [1] * B, page, torch.bfloat16)
    qd = q.reshape(B, nh * hd).cuda().bfloat16()
    assert K._balanced_ok(meta, nh // nkv, nkv), "the engine would take the evenly cut kernel here"
    out = K.paged_attention(qd, cache, meta, nh, nkv, hd, scale, None)
    plain = K.paged_attention_plain(qd, cache, meta, nh, nkv, hd, scale, None)
    assert rel_err(out, plain.double()) < BF16_TOL
    for i in (0, 3, 5, 17, 39):
        ref = rows_reference(ks[i], vs[i], q[i:i + 1], [contexts[i] - 1], scale, None, nh)
        assert rel_err(out[i].view(1, nh, hd), ref) < BF16_TOL


@pytest.mark.parametrize("q_len,ctx,window", [(8192, 8192, None), (2048, 8048, None), (2048, 8048, 4096)])
def test_prefill_attention_over_long_contexts(K, q_len, ctx, window):
    """The tcgen05 kernel over 8,192 tokens at once, and over a 2,048-token portion behind a prefix
    of 6,000 tokens: against the plain kernel everywhere and float64 at chosen rows."""
    nh, nkv, hd, page = 8, 2, 128, 16
    scale = 1 / math.sqrt(hd)
    g = torch.Generator().manual_seed(q_len + ctx)
    bf = lambda t: t.bfloat16().float()
    k, v = bf(torch.randn(ctx, nkv, hd, generator=g)), bf(torch.randn(ctx, nkv, hd, generator=g))
    q = bf(torch.randn(q_len, nh, hd, generator=g))
    cache, meta = paged_setup([k], [v], [q_len], page, torch.bfloat16, window=window)
    qd = q.reshape(q_len, nh * hd).cuda().bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = K.attention_tcgen05(qd, cache, meta, torch.zeros_like(qd), nh, nkv, hd, scale, window, status=status)
    assert int(status.item()) == 0
    plain = K.paged_attention_plain(qd, cache, meta, nh, nkv, hd, scale, window)
    assert rel_err(out, plain.double()) < BF16_TOL
    assert torch.equal(out, K.paged_attention(qd, cache, meta, nh, nkv, hd, scale, window))    # what the engine runs
    rows = [0, 1, 31, 32, 127, 128, q_len // 2, q_len - 2, q_len - 1]
    ref = rows_reference(k, v, q[rows], [ctx - q_len + r for r in rows], scale, window, nh)
    assert rel_err(out.view(q_len, nh, hd)[rows], ref) < BF16_TOL


@pytest.mark.parametrize("nh,nkv,hd,page,window", [(32, 8, 128, 16, None), (8, 2, 64, 8, 100), (28, 4, 128, 64, None),
                                                  (6, 6, 64, 128, 333), (16, 1, 128, 32, None)])
def test_tma_fed_decode_attention_gives_the_bits_of_the_cp_async_kernel(K, nh, nkv, hd, page, window):
    """The decode kernel whose tiles come by TMA against the one that copies them with cp.async:
    the same arithmetic in the same order, so the same bits - for every split count, with and
    without requesting keys before the wait for the preceding kernel, with pages given back below
    the window, for one-token sequences among longer ones (q_filter), and with far more CTAs than
    stay resident at once, so that later CTAs inherit the shared memory of earlier ones."""
    scale = 1 / math.sqrt(hd)
    g = torch.Generator().manual_seed(hd + page)
    contexts = [1, 7, 64, 65, 500, 1027, 2049, 130]
    ks = [torch.randn(c, nkv, hd, generator=g) for c in contexts]
    vs = [torch.randn(c, nkv, hd, generator=g) for c in contexts]
    B = len(contexts)
    cache, meta = paged_setup(ks, vs, [1] * B, page, torch.bfloat16, window=window)
    q = torch.randn(B, nh * hd, generator=g).cuda().bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    plain = K.paged_attention_plain(q, cache, meta, nh, nkv, hd, scale, window)
    for splits in (1, 2, 5, 16, 40):
        want = K.decode_attention(q, cache, meta, torch.zeros_like(q), nh, nkv, hd, scale, window, num_splits=splits, tma=False)
        for early in (False, True):
            got = K.decode_attention(q, cache, meta, torch.full_like(q, 9.0), nh, nkv, hd, scale, window, num_splits=splits,
                                     tma=True, early=early, status=status)
            assert torch.equal(got, want), f"{splits} splits, early={early}"
        assert rel_err(want, plain.double()) < BF16_TOL
    assert int(status.item()) == 0
    # one-token sequences among longer ones: only they are touched
    q_lens = [1, 20, 1, 3, 1]
    ctxs = [300, 20, 64, 700, 1]
    ks = [torch.randn(c, nkv, hd, generator=g) for c in ctxs]
    vs = [torch.randn(c, nkv, hd, generator=g) for c in ctxs]
    cache, meta = paged_setup(ks, vs, q_lens, page, torch.bfloat16, window=window)
    q = torch.randn(sum(q_lens), nh * hd, generator=g).cuda().bfloat16()
    want = K.decode_attention(q, cache, meta, torch.full_like(q, 9.0), nh, nkv, hd, scale, window, q_filter=1, tma=False)
    got = K.decode_attention(q, cache, meta, torch.full_like(q, 9.0), nh, nkv, hd, scale, window, q_filter=1, tma=True, status=status)
    assert torch.equal(got, want) and float((got[1:21].float() - 9.0).abs().max()) == 0.0
    # 2,000 CTAs of two to three tiles each: several waves on every SM
    many = 250 if nkv >= 4 else 600
    ctxs = [130 + (37 * i) % 60 for i in range(many)]
    ks = [torch.randn(c, nkv, hd, generator=g) for c in ctxs]
    cache, meta = paged_setup(ks, ks, [1] * many, page, torch.bfloat16)
    q = torch.randn(many, nh * hd, generator=g).cuda().bfloat16()
    want = K.decode_attention(q, cache, meta, torch.zeros_like(q), nh, nkv, hd, scale, None, tma=False)
    for _ in range(3):
        got = K.decode_attention(q, cache, meta, torch.full_like(q, 9.0), nh, nkv, hd, scale, None, tma=True, status=status)
        assert torch.equal(got, want)
    assert int(status.item()) == 0
