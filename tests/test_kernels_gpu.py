"""Each CUDA kernel alone against its plain reference (tests/plain_impl.py), in float32 and
bfloat16, at sizes other than the engine's own tests use."""
import math

import pytest
import torch

import plain_impl as P
from gpu_tools import paged_setup, rel_err

pytestmark = pytest.mark.gpu

from rvllm_b200.kernels.library import COUNTERS

F32_TOL = 2e-6
BF16_TOL = 1e-2      # a bfloat16 result carries half an ulp (2^-9) of its own rounding


@pytest.fixture(scope="module")
def K():
    from rvllm_b200.kernels import get_library
    return get_library("cuda:0")


def tol(dtype):
    return F32_TOL if dtype == torch.float32 else BF16_TOL


DTYPES = [torch.float32, torch.bfloat16]


def same_up_to_an_ulp(a, b):
    """Two bfloat16 results of the same float sums, rounded once each: equal except where an
    FMA contracted differently moved a value across a rounding boundary (one ulp, rarely)."""
    a, b = a.float(), b.float()
    diff = (a - b).abs()
    # (where a rotation cancels, a result near zero inherits the float ulps of its much larger terms)
    ulp = torch.maximum(a.abs(), b.abs()) * 2.0 ** -7 + 1e-5 * float(a.abs().mean())
    return bool((diff <= ulp).all()) and float((diff > 0).float().mean()) < 0.02


def rounded_once(got, exact):
    """The rms error of a bfloat16 result against float64 is that of one rounding (two roundings
    in a row, e.g. a product rounded before it is rotated, give 1.41 times as much)."""
    exact = exact.double().cpu()
    once = (exact.bfloat16().double() - exact).pow(2).mean().sqrt()
    return float((got.double().cpu() - exact).pow(2).mean().sqrt()) < 1.15 * float(once)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width", [(7, 100), (300, 4096), (1, 13)])
def test_gather_rows(K, dtype, rows, width):
    torch.manual_seed(0)
    table = torch.randn(rows, width, device="cuda").to(dtype)
    ids = torch.randint(0, rows, (37,), device="cuda", dtype=torch.int32)
    out = K.gather_rows(table, ids)
    assert torch.equal(out.cpu(), P.embedding(ids.tolist(), table.cpu()))
    ids[3] = rows + 5                                   # the host refuses such ids; the kernel writes zeros
    assert float(K.gather_rows(table, ids)[3].abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width,eps", [(5, 100, 1e-5), (3, 4100, 1e-6), (64, 24, 1e-2)])
def test_rmsnorm(K, dtype, rows, width, eps):
    torch.manual_seed(1)
    x = (torch.randn(rows, width, device="cuda") * 3).to(dtype)
    gamma = (1 + 0.1 * torch.randn(width, device="cuda")).to(dtype)
    ref = P.rms_norm(x.double().cpu(), gamma.double().cpu(), eps)
    assert rel_err(K.rmsnorm(x, gamma, eps), ref) < tol(dtype)
    g32 = gamma.float()                                 # a weight the checkpoint stores in 32 bits stays so
    assert rel_err(K.rmsnorm(x, g32, eps), P.rms_norm(x.double().cpu(), g32.double().cpu(), eps)) < tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,inter", [(3, 172), (17, 1000), (1, 7)])
def test_silu_mul(K, dtype, rows, inter):
    torch.manual_seed(2)
    gu = (torch.randn(rows, 2 * inter, device="cuda") * 4).to(dtype)
    g, u = gu[:, :inter].double().cpu(), gu[:, inter:].double().cpu()
    assert rel_err(K.silu_mul(gu), g / (1 + torch.exp(-g)) * u) < tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,page,bias", [(5, 1, 48, 4, True), (8, 8, 16, 32, False), (6, 3, 128, 16, True)])
def test_rope_bias_cache_write(K, dtype, nh, nkv, hd, page, bias):
    from rvllm_b200.parts import RotaryEncoding
    torch.manual_seed(3)
    T, n_pages = 23, 9
    rope = RotaryEncoding(hd, 50000.0, None)
    rope.prepare(300, "cuda")
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device="cuda").to(dtype)
    b = torch.randn((nh + 2 * nkv) * hd, device="cuda").to(dtype) if bias else None
    positions = torch.randint(0, 300, (T,), dtype=torch.int32)
    slots = torch.randperm(n_pages * page)[:T].to(torch.int32)
    slots[5] = -1                                       # a padded row writes nothing
    cache = torch.zeros(n_pages, 2, nkv, page, hd, device="cuda", dtype=dtype)
    q = K.rope_cache_write(qkv, b, positions.cuda(), rope.cos, rope.sin, slots.cuda(), cache, nh, nkv, hd)
    x = qkv.double().cpu() + (b.double().cpu() if bias else 0)
    inv = P.rope_inv_freq(hd, 50000.0, None)
    q_ref = P.apply_rope(x[:, :nh * hd].view(T, nh, hd), positions.tolist(), inv)
    k_ref = P.apply_rope(x[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd), positions.tolist(), inv)
    v_ref = x[:, (nh + nkv) * hd:].view(T, nkv, hd)
    assert rel_err(q.view(T, nh, hd), q_ref) < tol(dtype)
    want = torch.zeros(n_pages, 2, nkv, page, hd, dtype=torch.float64)
    for t in range(T):
        s = int(slots[t])
        if s >= 0:
            want[s // page, 0, :, s % page] = k_ref[t]
            want[s // page, 1, :, s % page] = v_ref[t]
    assert rel_err(cache, want) < tol(dtype)
    assert float(cache.double().cpu()[want == 0].abs().max()) == 0.0     # nothing else was touched
    # q alone (a layer that reads another layer's cache)
    q_only = K.rope_cache_write(qkv[:, :nh * hd].contiguous(), b[:nh * hd] if bias else None, positions.cuda(),
                                rope.cos, rope.sin, None, None, nh, nkv, hd, write_kv=False)
    assert torch.equal(q_only, q)
    # no position encoding: bias only
    q_plain = K.rope_cache_write(qkv, b, positions.cuda(), None, None, slots.cuda(), cache, nh, nkv, hd)
    assert rel_err(q_plain.view(T, nh, hd), x[:, :nh * hd].view(T, nh, hd)) < tol(dtype)
    # a rotation of the leading part of every head only (tables of rotary_dim / 2 columns)
    for rot in (hd // 2 // 2 * 2, 2):
        part = RotaryEncoding(hd, 50000.0, None, rotary_dim=rot)
        part.prepare(300, "cuda")
        assert part.cos.shape == (300, rot // 2)
        cache2 = torch.zeros_like(cache)
        q2 = K.rope_cache_write(qkv, b, positions.cuda(), part.cos, part.sin, slots.cuda(), cache2, nh, nkv, hd)
        inv2 = P.rope_inv_freq(rot, 50000.0, None)
        turn = lambda t: torch.cat([P.apply_rope(t[..., :rot], positions.tolist(), inv2), t[..., rot:]], -1)
        assert rel_err(q2.view(T, nh, hd), turn(x[:, :nh * hd].view(T, nh, hd))) < tol(dtype)
        k2 = turn(x[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd))
        for t in range(T):
            sl = int(slots[t])
            if sl >= 0:
                assert rel_err(cache2[sl // page, 0, :, sl % page], k2[t]) < tol(dtype)
                assert rel_err(cache2[sl // page, 1, :, sl % page], v_ref[t]) < tol(dtype)
        # the dispatching entry point leaves such tables to this kernel, whatever the number of rows
        w = torch.eye((nh + 2 * nkv) * hd, device="cuda").to(dtype)
        cache3 = torch.zeros_like(cache)
        q3 = K.qkv_rope_cache_write(qkv, w, b, positions.cuda(), part.cos, part.sin, slots.cuda(), cache3, nh, nkv, hd)
        assert rel_err(q3.view(T, nh, hd), turn(x[:, :nh * hd].view(T, nh, hd))) < tol(dtype)
    with pytest.raises(Exception, match="rotary_dim"):
        RotaryEncoding(hd, 50000.0, None, rotary_dim=hd + 2)


def _attention_case(nh, nkv, hd, page, q_lens, ctx_lens, window, seed):
    torch.manual_seed(seed)
    ks = [torch.randn(c, nkv, hd) for c in ctx_lens]
    vs = [torch.randn(c, nkv, hd) for c in ctx_lens]
    qs = [torch.randn(n, nh, hd) for n in q_lens]
    return ks, vs, qs


def _attention_ref(ks, vs, qs, ctx_lens, q_lens, scale, window, dtype):
    outs = []
    for k, v, q, c, n in zip(ks, vs, qs, ctx_lens, q_lens):
        k, v, q = (t.to(dtype).double() for t in (k, v, q))
        full_q = torch.zeros(c, q.shape[1], q.shape[2], dtype=torch.float64)
        full_q[c - n:] = q
        outs.append(P.causal_attention(full_q, k, v, scale, window)[c - n:])
    return torch.cat(outs)


ATT_CASES = [
    # nh, nkv, hd, page, q_lens, ctx_lens, window
    (4, 2, 16, 16, [5], [5], None),
    (6, 2, 32, 8, [70, 1, 1, 2], [70, 9, 129, 64], 40),
    (7, 7, 48, 4, [33, 1, 7], [33, 40, 100], None),
    (12, 4, 64, 32, [1, 1, 1], [500, 31, 1], None),
    (10, 2, 80, 16, [64, 65], [64, 200], 64),
    (3, 1, 256, 16, [9, 1], [30, 77], None),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ATT_CASES)
def test_paged_attention_plain_kernel(K, dtype, case):
    nh, nkv, hd, page, q_lens, ctx_lens, window = case
    ks, vs, qs = _attention_case(nh, nkv, hd, page, q_lens, ctx_lens, window, 4)
    cache, meta = paged_setup(ks, vs, q_lens, page, dtype)
    q = torch.cat(qs).reshape(sum(q_lens), nh * hd).cuda().to(dtype)
    scale = 1 / math.sqrt(hd)
    out = K.paged_attention_plain(q, cache, meta, nh, nkv, hd, scale, window)
    ref = _attention_ref(ks, vs, qs, ctx_lens, q_lens, scale, window, dtype)
    assert rel_err(out.view(-1, nh, hd), ref) < (1e-5 if dtype == torch.float32 else BF16_TOL)


@pytest.mark.parametrize("case", ATT_CASES)
def test_flash_attention_kernel(K, case):
    nh, nkv, hd, page, q_lens, ctx_lens, window = case
    ks, vs, qs = _attention_case(nh, nkv, hd, page, q_lens, ctx_lens, window, 5)
    cache, meta = paged_setup(ks, vs, q_lens, page, torch.bfloat16)
    q = torch.cat(qs).reshape(sum(q_lens), nh * hd).cuda().bfloat16()
    scale = 1 / math.sqrt(hd)
    ref = _attention_ref(ks, vs, qs, ctx_lens, q_lens, scale, window, torch.bfloat16)
    out = K.paged_attention(q, cache, meta, nh, nkv, hd, scale, window)        # the product path's dispatch
    assert rel_err(out.view(-1, nh, hd), ref) < BF16_TOL
    plain = K.paged_attention_plain(q, cache, meta, nh, nkv, hd, scale, window)
    assert rel_err(out, plain.double()) < BF16_TOL
    if 1 in q_lens:
        # the kernel that cuts all tiles evenly over a fixed number of CTAs: rows of one-token sequences
        for ctas in (0, 1, 3, 7, 64):
            o3 = torch.full_like(q, 9.0)
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            K.flash_decode_balanced(q, cache, meta, o3, nh, nkv, hd, scale, window, ctas=ctas, status=status)
            assert int(status.item()) == 0, "a bounded wait inside the kernel gave up"
            o4 = torch.full_like(q, 9.0)           # tiles by cp.async instead of TMA (where the sizes allow TMA): the same bits
            K.flash_decode_balanced(q, cache, meta, o4, nh, nkv, hd, scale, window, ctas=ctas, tma=False)
            assert torch.equal(o3, o4)
            row = 0
            for n in q_lens:
                if n == 1:
                    assert rel_err(o3.view(-1, nh, hd)[row], ref[row]) < BF16_TOL
                else:
                    assert bool((o3[row:row + n] == 9.0).all())                # longer sequences are left alone
                row += n
    if max(q_lens) == 1:
        for splits in (2, 5, 19, 40):                                           # keys split over CTAs and merged (more splits than tiles: empty ones)
            o2 = torch.empty_like(q)
            K.flash_attention(q, cache, meta, o2, nh, nkv, hd, scale, window, mode=1, num_splits=splits)
            assert rel_err(o2.view(-1, nh, hd), ref) < BF16_TOL


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_a_far_key_among_hundreds(K, dtype):
    """One key far back is made to dominate: the output must be its value row.  Random scores
    would hide a kernel that drops or misplaces a page of keys."""
    nh, nkv, hd, page = 4, 2, 64, 16
    ctx = 777
    for target in (0, 15, 16, 300, 511, 512, 776):         # first key, page edges, tile edges, the last key
        torch.manual_seed(target)
        k = torch.randn(ctx, nkv, hd) * 0.1
        v = torch.randn(ctx, nkv, hd)
        q = torch.randn(1, nh, hd) * 0.1
        direction = torch.randn(hd)
        direction /= direction.norm()
        k[target] = direction * 12.0
        q[0] = direction * 12.0                             # score 144 * scale = 18: e^18 against 776 keys near e^0
        cache, meta = paged_setup([k], [v], [1], page, dtype, seed=target)
        out = K.paged_attention(q.reshape(1, nh * hd).cuda().to(dtype), cache, meta, nh, nkv, hd, 1 / math.sqrt(hd), None)
        want = v[target][[0, 0, 1, 1]].to(dtype).double()
        got = out.view(nh, hd).double().cpu()
        assert float((got - want).abs().max()) < 0.1, f"key {target} was not found"


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_window_edge(K, dtype):
    """The key just inside the window dominates when it may be seen; the key just outside never does."""
    nh, nkv, hd, page, window = 2, 1, 32, 8, 24
    ctx, q_len = 100, 10
    torch.manual_seed(0)
    direction = torch.randn(hd)
    direction /= direction.norm()
    for which in ("inside", "outside"):
        k = torch.randn(ctx, nkv, hd) * 0.1
        v = torch.randn(ctx, nkv, hd)
        q = direction.repeat(q_len, nh, 1) * 12.0
        p_last = ctx - 1
        marked = p_last - window + 1 if which == "inside" else p_last - window      # edge of the LAST query's window
        k[marked] = direction * 12.0
        cache, meta = paged_setup([k], [v], [q_len], page, dtype)
        out = K.paged_attention(q.reshape(q_len, nh * hd).cuda().to(dtype), cache, meta, nh, nkv, hd,
                                1 / math.sqrt(hd), window).view(q_len, nh, hd).double().cpu()
        hit = float((out[-1, 0] - v[marked, 0].to(dtype).double()).abs().max()) < 0.1
        assert hit == (which == "inside")
        # the earlier queries of the portion have their own windows: the marked key is inside them all
        assert float((out[0, 0] - v[marked, 0].to(dtype).double()).abs().max()) < 0.1


@pytest.mark.parametrize("M,N,Kd,bias,res", [(1, 7, 5, False, False), (33, 261, 172, True, True),
                                             (130, 64, 300, False, True), (5, 1000, 2048, True, False)])
def test_gemm_f32_is_true_32_bit(K, M, N, Kd, bias, res):
    torch.manual_seed(6)
    x = torch.randn(M, Kd, device="cuda")
    w = torch.randn(N, Kd, device="cuda")
    # operands with more mantissa bits than TF32 keeps: a reduced-precision product would be off by 1e-3
    b = torch.randn(N, device="cuda") if bias else None
    r = torch.randn(M, N, device="cuda") if res else None
    ref = x.double().cpu() @ w.double().cpu().t()
    if bias:
        ref += b.double().cpu()
    if res:
        ref += r.double().cpu()
    out = K.linear(x, w, b, r)
    assert out.dtype == torch.float32 and rel_err(out, ref) < 3e-6
    again = K.linear(x[:1].contiguous(), w, b, r[:1].contiguous() if res else None)
    assert torch.equal(again, out[:1])                      # a row does not depend on the rest of the batch


@pytest.mark.parametrize("M,N,Kd,res,f32out", [(200, 300, 172, True, False), (64, 261, 80, False, True),
                                               (2048, 512, 256, True, False)])
def test_linear_bf16_library_path(K, M, N, Kd, res, f32out):
    torch.manual_seed(8)
    x = torch.randn(M, Kd, device="cuda").bfloat16()
    w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    r = torch.randn(M, N, device="cuda").bfloat16() if res else None
    ref = x.double().cpu() @ w.double().cpu().t() + (r.double().cpu() if res else 0)
    out = K.linear(x, w, None, r, torch.float32 if f32out else None)
    assert out.dtype == (torch.float32 if f32out else torch.bfloat16)
    assert rel_err(out, ref) < (1e-5 if f32out else BF16_TOL)
    # a matrix the checkpoint keeps in 32 bits is multiplied in float32
    assert rel_err(K.linear(x, w.float(), None, r), ref) < BF16_TOL


@pytest.mark.parametrize("M,N,Kd", [(128, 256, 64), (100, 200, 72), (257, 520, 4096), (640, 96, 1032), (2048, 1000, 328)])
def test_gemm_tcgen05_bf16(K, M, N, Kd):
    """The tcgen05 kernel: tails in M, N and K, several tiles per CTA, every epilogue."""
    torch.manual_seed(9)
    x = torch.randn(M, Kd, device="cuda").bfloat16()
    w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    r = torch.randn(M, N, device="cuda").bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = x.double().cpu() @ w.double().cpu().t()
    # both builds of the kernel: one CTA per tile of 128 rows, and pairs of CTAs (cta_group::2) per tile of 256 rows
    for pair in (False, True):
        for ctas in (0, 2, 6):                               # 2 and 6: a CTA (a pair) walks many tiles, both accumulators
            assert rel_err(K.linear_tcgen05(x, w, status=status, max_ctas=ctas, pair=pair), ref) < BF16_TOL
        assert rel_err(K.linear_tcgen05(x, w, r, status=status, pair=pair), ref + r.double().cpu()) < BF16_TOL
        assert rel_err(K.linear_tcgen05(x, w, None, torch.float32, status=status, pair=pair), ref) < 1e-5
        if N % 2 == 0:
            g, u = ref[:, :N // 2], ref[:, N // 2:]
            want = g / (1 + torch.exp(-g)) * u
            assert rel_err(K.linear_tcgen05(x, w, gated=True, status=status, pair=pair), want) < BF16_TOL
            assert rel_err(K.linear_tcgen05(x, w, None, torch.float32, gated=True, status=status, max_ctas=2, pair=pair), want) < 1e-5
    assert torch.equal(K.linear_tcgen05(x, w, r, pair=True), K.linear_tcgen05(x, w, r, pair=False))    # the same sums
    # K cut over a cluster of 2 or 4 CTAs per tile (partials through the cluster's shared memory, added in part order):
    # the same bits in every run, every epilogue but the gated one
    for splits in (2, 4):
        if splits > (Kd + 63) // 64:
            continue
        outs = [K.linear_tcgen05(x, w, r, status=status, splits=splits) for _ in range(3)]
        assert all(torch.equal(outs[0], o) for o in outs[1:]) and rel_err(outs[0], ref + r.double().cpu()) < BF16_TOL
        assert rel_err(K.linear_tcgen05(x, w, None, torch.float32, status=status, splits=splits), ref) < 1e-5
        assert rel_err(K.linear_tcgen05(x, w, status=status, splits=splits), ref) < BF16_TOL
    assert int(status.item()) == 0, "a bounded wait inside the kernel gave up"
    # the product path picks it where its tiles fill the GPU, and the library's GEMM elsewhere
    if K._tcgen05_fills(M, N):
        assert torch.equal(K.linear(x, w, None, r), K.linear_tcgen05(x, w, r))
    else:
        assert rel_err(K.linear(x, w, None, r), ref + r.double().cpu()) < BF16_TOL
    assert K._tcgen05_fills(2048, 4096) and K._tcgen05_fills(2048, 28672, True) and not K._tcgen05_fills(64, 4096)


@pytest.mark.parametrize("M,N,Kd", [(1, 128, 64), (3, 100, 200), (8, 520, 4096), (17, 261, 1032), (64, 1000, 328), (128, 384, 2048)])
def test_gemm_tcgen05_decode_bf16(K, M, N, Kd):
    """The weight-streaming tcgen05 kernel: every padded batch width, K split over CTAs and merged
    by the last arrival, every epilogue; counters are left ready for the next launch."""
    torch.manual_seed(10)
    x = torch.randn(M, Kd, device="cuda").bfloat16()
    w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    b = torch.randn(N, device="cuda").bfloat16()
    r = torch.randn(M, N, device="cuda").bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = x.double().cpu() @ w.double().cpu().t()
    for splits in (1, 2, 5, None):
        assert rel_err(K.linear_decode(x, w, splits=splits, status=status), ref) < BF16_TOL
    full = ref + b.double().cpu() + r.double().cpu()
    for _ in range(2):                                       # twice: the tile counters were reset
        assert rel_err(K.linear_decode(x, w, b, r, splits=3, status=status), full) < BF16_TOL
    assert rel_err(K.linear_decode(x, w, b.float(), None, torch.float32, splits=4, status=status), ref + b.double().cpu()) < 1e-5
    if N % 2 == 0:
        g, u = ref[:, :N // 2], ref[:, N // 2:]
        want = g / (1 + torch.exp(-g)) * u
        for splits in (1, 3):
            assert rel_err(K.linear_decode(x, w, gated=True, splits=splits, status=status), want) < BF16_TOL
    assert int(status.item()) == 0, "a bounded wait inside the kernel gave up"
    one = K.linear_decode(x[:1].contiguous(), w, out_dtype=torch.float32, splits=4)
    assert torch.equal(one, K.linear_decode(x, w, out_dtype=torch.float32, splits=4)[:1])     # batch-invariant
    if K._decode_counters is not None:
        assert int(K._decode_counters.abs().sum().item()) == 0


@pytest.mark.parametrize("M,N,Kd", [(1, 4096, 4096), (8, 520, 1032), (3, 101, 200), (5, 1024, 14336),
                                    (9, 384, 4096), (17, 520, 1032), (32, 4096, 4096), (33, 256, 2048), (64, 1000, 1032)])
def test_split_k_added_up_inside_a_cluster(K, M, N, Kd):
    """The CTAs of a tile as a thread-block cluster that adds its partials in the first CTA's shared
    memory: the same bits as the merge through scratch memory (both add in split order), for every
    cluster size, with bias, residual, float output and the fused norm; launches alternate so that a
    cluster launch follows a plain one and the other way round."""
    torch.manual_seed(14)
    x = torch.randn(M, Kd, device="cuda").bfloat16()
    w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    b = torch.randn(N, device="cuda").bfloat16()
    r = torch.randn(M, N, device="cuda").bfloat16()
    gamma = (1 + 0.1 * torch.randn(Kd, device="cuda")).bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = x.double().cpu() @ w.double().cpu().t() + b.double().cpu() + r.double().cpu()
    for splits in range(2, 9):
        if splits > (Kd + 63) // 64:
            break
        a = K.linear_decode(x, w, b, r, splits=splits, status=status, cluster=True)
        c = K.linear_decode(x, w, b, r, splits=splits, status=status, cluster=False)
        assert torch.equal(a, c) and rel_err(a, ref) < BF16_TOL
        a = K.linear_decode(x, w, None, None, torch.float32, splits=splits, status=status, cluster=True)
        c = K.linear_decode(x, w, None, None, torch.float32, splits=splits, status=status, cluster=False)
        assert torch.equal(a, c)
        if Kd <= 8128 and M <= 16:
            a = K.linear_decode(x, w, None, r, splits=splits, status=status, norm=(gamma, 1e-5), cluster=True)
            c = K.linear_decode(x, w, None, r, splits=splits, status=status, norm=(gamma, 1e-5), cluster=False)
            assert torch.equal(a, c)
    # what a cluster cannot serve falls back to the merge through scratch memory: many rows, many splits
    many = torch.cat([x] * (65 // M + 1))
    assert torch.equal(K.linear_decode(many, w, splits=2, cluster=True)[:M], K.linear_decode(x, w, splits=2, cluster=False))
    if (Kd + 63) // 64 >= 9:
        assert rel_err(K.linear_decode(x, w, b, r, splits=9, status=status, cluster=True), ref) < BF16_TOL
    assert int(status.item()) == 0
    if K._decode_counters is not None:
        assert int(K._decode_counters.abs().sum().item()) == 0


@pytest.mark.parametrize("M,N,Kd", [(100, 520, 1032), (128, 384, 4096), (129, 1000, 520), (300, 4096, 1024), (512, 256, 2048)])
def test_decode_gemm_in_blocks_of_128_rows(K, M, N, Kd):
    """More than 64 rows through the weight-streaming kernel: blocks of 128 rows (the last one cut), K whole or
    split inside a cluster, every epilogue; a row's sums do not depend on the block it falls into or on what
    else the batch holds."""
    torch.manual_seed(21)
    x = torch.randn(M, Kd, device="cuda").bfloat16()
    w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    b = torch.randn(N, device="cuda").bfloat16()
    r = torch.randn(M, N, device="cuda").bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = x.double().cpu() @ w.double().cpu().t()
    full = ref + b.double().cpu() + r.double().cpu()
    for splits in (None, 1, 2, 4, 7):
        if splits and splits > (Kd + 63) // 64:
            continue
        assert rel_err(K.linear_decode(x, w, splits=splits, status=status), ref) < BF16_TOL
        assert rel_err(K.linear_decode(x, w, b, r, splits=splits, status=status), full) < BF16_TOL
        got = K.linear_decode(x, w, b.float(), None, torch.float32, splits=splits, status=status)
        assert rel_err(got, ref + b.double().cpu()) < 1e-5
        if splits in (1, 2):
            # the last rows alone, and the first, with K cut at the same places: the same bits as inside the batch
            tail = K.linear_decode(x[-3:].contiguous(), w, b.float(), None, torch.float32, splits=splits, status=status)
            head = K.linear_decode(x[:70].contiguous(), w, b.float(), None, torch.float32, splits=splits, status=status)
            assert torch.equal(tail, got[-3:]) and torch.equal(head, got[:70])
    g, u = ref[:, :N // 2], ref[:, N // 2:]
    assert rel_err(K.linear_decode(x, w, gated=True, splits=1, status=status), g / (1 + torch.exp(-g)) * u) < BF16_TOL
    assert int(status.item()) == 0, "a bounded wait inside the kernel gave up"
    # the dispatch takes this kernel where tiles x row blocks leave SMs idle, and not beyond
    assert K._use_decode_gemm(M, N, Kd, False) == (M <= K.DECODE_BLOCK_MAX_ROWS and -(-N // 128) * -(-M // 128) <= K.num_sms)
    assert not K._use_decode_gemm(K.DECODE_BLOCK_MAX_ROWS + 1, N, Kd, False) and not K._use_decode_gemm(M, 2 * N, Kd, True)
    assert torch.equal(K.linear(x, w, b, r), K.linear_decode(x, w, b, r)) or not K._use_decode_gemm(M, N, Kd, False)


@pytest.mark.parametrize("M,nh,nkv,hd,Kd,page,bias", [(100, 6, 2, 64, 264, 16, True), (200, 8, 2, 128, 1024, 16, False),
                                                      (384, 4, 4, 32, 520, 8, True)])
def test_qkv_rotation_and_cache_write_in_blocks_of_128_rows(K, M, nh, nkv, hd, Kd, page, bias):
    """The rotary epilogue for more than 64 rows: every block of 128 rows takes its own positions and slots."""
    torch.manual_seed(22)
    N = (nh + 2 * nkv) * hd
    x = torch.randn(M, Kd, device="cuda").bfloat16()
    w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    b = torch.randn(N, device="cuda").bfloat16() if bias else None
    positions = torch.randint(0, 500, (M,), device="cuda", dtype=torch.int32)
    ang = torch.arange(512, dtype=torch.float64)[:, None] * (10000.0 ** (-torch.arange(hd // 2, dtype=torch.float64) * 2 / hd))[None]
    cos, sin = ang.cos().float().cuda(), ang.sin().float().cuda()
    pages = 2 * M // page + 3
    slots = torch.randperm(pages * page)[:M].to(torch.int32).cuda()
    slots[M // 2] = -1
    slots[M - 1] = -1
    cache_a = torch.full((pages, 2, nkv, page, hd), 7.0, device="cuda").bfloat16()
    cache_b = cache_a.clone()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for splits in (None, 1, 2, 3):
        if splits and splits > (Kd + 63) // 64 // 4:
            continue
        cache_a.fill_(7.0)
        cache_b.fill_(7.0)
        qa = K._qkv_rope_fused(x, w, b, positions, cos, sin, slots, cache_a, nh, nkv, hd, splits=splits, status=status)
        qkv = K.linear_decode(x, w, splits=splits, out_dtype=torch.float32)
        qb = K.rope_cache_write(qkv, b, positions, cos, sin, slots, cache_b, nh, nkv, hd, out_dtype=torch.bfloat16)
        assert same_up_to_an_ulp(qa, qb) and same_up_to_an_ulp(cache_a, cache_b)
    assert int(status.item()) == 0
    y = x.double().cpu() @ w.double().cpu().t()
    if bias:
        y = y + b.double().cpu()
    y = y.view(M, nh + 2 * nkv, hd)
    c, s_ = ang.cos()[positions.cpu().long()][:, None, :], ang.sin()[positions.cpu().long()][:, None, :]
    rot = lambda t: torch.cat([t[..., :hd // 2] * c - t[..., hd // 2:] * s_, t[..., :hd // 2] * s_ + t[..., hd // 2:] * c], -1)
    assert rounded_once(qa, rot(y[:, :nh]).reshape(M, nh * hd))
    kref, vref = rot(y[:, nh:nh + nkv]), y[:, nh + nkv:]
    for m in (0, 63, 64, 127, 128, M - 2):
        if m >= M:
            continue
        sl = int(slots[m])
        if sl >= 0:
            assert rel_err(cache_a[sl // page, 0, :, sl % page], kref[m]) < BF16_TOL
            assert rel_err(cache_a[sl // page, 1, :, sl % page], vref[m]) < BF16_TOL
    # rows without a slot wrote nothing: as many untouched slots as the cache has beyond the written ones
    written = int((slots >= 0).sum())
    assert int((cache_a.float().permute(0, 3, 1, 2, 4).reshape(pages * page, -1) != 7.0).any(1).sum()) == written


@pytest.mark.parametrize("M,nh,nkv,hd,Kd,page,bias", [(1, 32, 8, 128, 4096, 16, False), (5, 6, 2, 32, 96, 8, True),
                                                      (16, 5, 5, 16, 80, 16, True), (3, 4, 1, 64, 264, 4, False)])
def test_qkv_product_with_rotation_and_cache_write_in_one_kernel(K, M, nh, nkv, hd, Kd, page, bias):
    """The decode GEMM's rotary epilogue against the two-kernel path (a float32 product, then the
    rotary kernel: the same float sums, rounded once in both) and against plain float64 arithmetic,
    where its error must be that of ONE rounding to bfloat16; rows with slot -1 write nothing; other
    cache slots stay untouched."""
    torch.manual_seed(12)
    N = (nh + 2 * nkv) * hd
    x = torch.randn(M, Kd, device="cuda").bfloat16()
    w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    b = torch.randn(N, device="cuda").bfloat16() if bias else None
    positions = torch.randint(0, 500, (M,), device="cuda", dtype=torch.int32)
    ang = torch.arange(512, dtype=torch.float64)[:, None] * (10000.0 ** (-torch.arange(hd // 2, dtype=torch.float64) * 2 / hd))[None]
    cos, sin = ang.cos().float().cuda(), ang.sin().float().cuda()
    pages = 2 * M + 3
    slots = torch.randperm(pages * page)[:M].to(torch.int32).cuda()
    if M > 2:
        slots[1] = -1
    cache_a = torch.full((pages, 2, nkv, page, hd), 7.0, device="cuda").bfloat16()
    cache_b = cache_a.clone()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for splits in (None, 1, 3):
        cache_a.fill_(7.0)
        qa = K._qkv_rope_fused(x, w, b, positions, cos, sin, slots, cache_a, nh, nkv, hd, splits=splits, status=status)
        qkv = K.linear_decode(x, w, splits=splits, out_dtype=torch.float32)
        cache_b.fill_(7.0)
        qb = K.rope_cache_write(qkv, b, positions, cos, sin, slots, cache_b, nh, nkv, hd, out_dtype=torch.bfloat16)
        assert same_up_to_an_ulp(qa, qb) and same_up_to_an_ulp(cache_a, cache_b)
    if Kd >= 128:                           # the cluster's merge and the one through scratch memory
        for cluster in (True, False):
            cache_b.fill_(7.0)
            qc = K._qkv_rope_fused(x, w, b, positions, cos, sin, slots, cache_b, nh, nkv, hd, splits=2, status=status, cluster=cluster)
            qkv = K.linear_decode(x, w, splits=2, cluster=False, out_dtype=torch.float32)
            cache_a.fill_(7.0)
            qb = K.rope_cache_write(qkv, b, positions, cos, sin, slots, cache_a, nh, nkv, hd, out_dtype=torch.bfloat16)
            assert same_up_to_an_ulp(qc, qb) and same_up_to_an_ulp(cache_a, cache_b)
        cache_a.fill_(7.0)
        qa = K._qkv_rope_fused(x, w, b, positions, cos, sin, slots, cache_a, nh, nkv, hd, splits=3, status=status)
    assert int(status.item()) == 0
    # plain arithmetic
    y = x.double().cpu() @ w.double().cpu().t()
    if bias:
        y = y + b.double().cpu()
    y = y.view(M, nh + 2 * nkv, hd)
    c, s_ = ang.cos()[positions.cpu().long()][:, None, :], ang.sin()[positions.cpu().long()][:, None, :]
    rot = lambda t: torch.cat([t[..., :hd // 2] * c - t[..., hd // 2:] * s_, t[..., :hd // 2] * s_ + t[..., hd // 2:] * c], -1)
    assert rel_err(qa, rot(y[:, :nh]).reshape(M, nh * hd)) < BF16_TOL
    assert rounded_once(qa, rot(y[:, :nh]).reshape(M, nh * hd))
    kref, vref = rot(y[:, nh:nh + nkv]), y[:, nh + nkv:]
    written = torch.zeros(pages, page, dtype=torch.bool)
    for m in range(M):
        sl = int(slots[m])
        if sl < 0:
            continue
        written[sl // page, sl % page] = True
        assert rel_err(cache_a[sl // page, 0, :, sl % page], kref[m]) < BF16_TOL
        assert rel_err(cache_a[sl // page, 1, :, sl % page], vref[m]) < BF16_TOL
    untouched = cache_a.cpu().float().permute(0, 3, 1, 2, 4)[~written]
    assert bool((untouched == 7.0).all())
    # with the layer's input norm inside the kernel
    gamma = (1 + 0.1 * torch.randn(Kd, device="cuda")).bfloat16()
    cache_a.fill_(7.0)
    cache_b.fill_(7.0)
    qn = K._qkv_rope_fused(x, w, b, positions, cos, sin, slots, cache_a, nh, nkv, hd, norm=(gamma, 1e-6), status=status)
    qm = K._qkv_rope_fused(K.rmsnorm(x, gamma, 1e-6), w, b, positions, cos, sin, slots, cache_b, nh, nkv, hd)
    assert rel_err(qn, qm.double().cpu()) < 4e-3 and rel_err(cache_a, cache_b.double().cpu()) < 4e-3
    assert int(status.item()) == 0
    # the dispatching entry point runs the fused kernel (with its own choice of splits) for few rows
    cache_a.fill_(7.0)
    cache_b.fill_(7.0)
    qa = K._qkv_rope_fused(x, w, b, positions, cos, sin, slots, cache_a, nh, nkv, hd)
    before = COUNTERS["launches"]
    qd = K.qkv_rope_cache_write(x, w, b, positions, cos, sin, slots, cache_b, nh, nkv, hd)
    if M <= K.FUSED_QKV_MAX_ROWS:
        assert COUNTERS["launches"] == before + 1 and torch.equal(qd, qa) and torch.equal(cache_a, cache_b)
    else:                                   # more rows: the product and the rotation kernel, one after the other
        assert COUNTERS["launches"] == before + 2
        assert rel_err(qd, qa.double().cpu()) < BF16_TOL and rel_err(cache_b, cache_a.double().cpu()) < BF16_TOL


@pytest.mark.parametrize("M,N,Kd,gamma_dtype", [(1, 4096, 4096, torch.bfloat16), (8, 512, 328, torch.float32),
                                                (5, 200, 1032, torch.bfloat16), (16, 384, 64, torch.bfloat16)])
def test_rmsnorm_inside_the_decode_gemm(K, M, N, Kd, gamma_dtype):
    """RMSNorm applied to the activation tiles in shared memory (the consuming GEMM's own warps)
    against the norm kernel followed by the same GEMM, for the plain, gated and rotary epilogues,
    with and without a split of K; and against plain float64 arithmetic."""
    torch.manual_seed(13)
    x = (torch.randn(M, Kd, device="cuda") * 3).bfloat16()
    w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    gamma = (1 + 0.1 * torch.randn(Kd, device="cuda")).to(gamma_dtype)
    eps = 1e-5
    r = torch.randn(M, N, device="cuda").bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    h = K.rmsnorm(x, gamma, eps)
    xd = x.double().cpu()
    hd_ = xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + eps) * gamma.double().cpu()
    ref = hd_ @ w.double().cpu().t()
    for splits in (1, 3, None):
        a = K.linear_decode(x, w, None, r, splits=splits, status=status, norm=(gamma, eps))
        b = K.linear_decode(h, w, None, r, splits=splits, status=status)
        assert rel_err(a, b.double().cpu()) < 4e-3            # the two round the normalised row alike up to the last bit of 1/rms
        assert rel_err(a, ref + r.double().cpu()) < BF16_TOL
        g = K.linear_decode(x, w, gated=True, splits=splits, status=status, norm=(gamma, eps))
        assert rel_err(g, K.linear_decode(h, w, gated=True, splits=splits, status=status).double().cpu()) < 4e-3
    one = K.linear_decode(x[:1].contiguous(), w, out_dtype=torch.float32, splits=2, norm=(gamma, eps))
    assert torch.equal(one, K.linear_decode(x, w, out_dtype=torch.float32, splits=2, norm=(gamma, eps))[:1])   # batch-invariant
    assert int(status.item()) == 0
    # dispatching entry points: fused for few rows, norm kernel first otherwise - same numbers within rounding
    y = K.linear(x, w, None, r, norm=(gamma, eps))
    assert rel_err(y, ref + r.double().cpu()) < BF16_TOL
    many = torch.cat([x] * 5)
    y5 = K.linear(many, w, None, None, norm=(gamma, eps))
    assert rel_err(y5[:M], ref) < BF16_TOL
    gref = ref[:, :N // 2] / (1 + torch.exp(-ref[:, :N // 2])) * ref[:, N // 2:]
    assert rel_err(K.gate_up_silu(x, w, norm=(gamma, eps)), gref) < 2 * BF16_TOL
    assert rel_err(K.gate_up_silu(many, w, norm=(gamma, eps))[:M], gref) < 2 * BF16_TOL


@pytest.mark.parametrize("M,nh,nkv,hd,Kd,page,bias", [(2048, 32, 8, 128, 512, 16, False), (300, 6, 2, 64, 264, 8, True),
                                                      (129, 2, 1, 256, 128, 16, True), (640, 5, 5, 128, 96, 4, False)])
def test_qkv_product_with_rotation_and_cache_write_for_many_rows(K, M, nh, nkv, hd, Kd, page, bias):
    """The prefill GEMM's rotary epilogue against a float32 product followed by the rotary kernel (same
    sums, same formula, one rounding: equal up to the last bit of a contracted multiply-add) and against
    float64 arithmetic, where its error must be that of ONE rounding to bfloat16; rows with slot -1
    write nothing; other cache slots stay untouched; several tiles per CTA."""
    torch.manual_seed(14)
    N = (nh + 2 * nkv) * hd
    x = torch.randn(M, Kd, device="cuda").bfloat16()
    w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    b = torch.randn(N, device="cuda").bfloat16() if bias else None
    positions = torch.randint(0, 500, (M,), device="cuda", dtype=torch.int32)
    ang = torch.arange(512, dtype=torch.float64)[:, None] * (10000.0 ** (-torch.arange(hd // 2, dtype=torch.float64) * 2 / hd))[None]
    cos, sin = ang.cos().float().cuda(), ang.sin().float().cuda()
    pages = (2 * M) // page + 3
    slots = torch.randperm(pages * page)[:M].to(torch.int32).cuda()
    slots[1] = -1
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cache_b = torch.full((pages, 2, nkv, page, hd), 7.0, device="cuda").bfloat16()
    qb = K.rope_cache_write(K.linear_tcgen05(x, w, out_dtype=torch.float32), b, positions, cos, sin, slots, cache_b, nh, nkv, hd,
                            out_dtype=torch.bfloat16)
    for ctas, pair, splits in ((0, False, 1), (2, False, 1), (0, True, 1), (4, True, 1), (0, False, 2), (0, False, 4), (0, None, None)):
        if splits and splits > 1 and ((256 // splits) % hd or (Kd + 63) // 64 < splits):
            continue
        cache_a = torch.full((pages, 2, nkv, page, hd), 7.0, device="cuda").bfloat16()
        qa = K._qkv_rope_tcgen05(x, w, b, positions, cos, sin, slots, cache_a, nh, nkv, hd, status=status, max_ctas=ctas, pair=pair,
                                 splits=splits)
        assert same_up_to_an_ulp(qa, qb) and same_up_to_an_ulp(cache_a, cache_b)         # nearly every element bit-equal
    assert int(status.item()) == 0
    y = x.double().cpu() @ w.double().cpu().t()
    if bias:
        y = y + b.double().cpu()
    y = y.view(M, nh + 2 * nkv, hd)
    c, s_ = ang.cos()[positions.cpu().long()][:, None, :], ang.sin()[positions.cpu().long()][:, None, :]
    rot = lambda t: torch.cat([t[..., :hd // 2] * c - t[..., hd // 2:] * s_, t[..., :hd // 2] * s_ + t[..., hd // 2:] * c], -1)
    assert rel_err(qa, rot(y[:, :nh]).reshape(M, nh * hd)) < BF16_TOL
    assert rounded_once(qa, rot(y[:, :nh]).reshape(M, nh * hd))
    kref, vref = rot(y[:, nh:nh + nkv]), y[:, nh + nkv:]
    written = torch.zeros(pages, page, dtype=torch.bool)
    for m in range(0, M, 7):
        sl = int(slots[m])
        if sl >= 0:
            assert rel_err(cache_a[sl // page, 0, :, sl % page], kref[m]) < BF16_TOL
            assert rel_err(cache_a[sl // page, 1, :, sl % page], vref[m]) < BF16_TOL
    for m in range(M):
        sl = int(slots[m])
        if sl >= 0:
            written[sl // page, sl % page] = True
    untouched = cache_a.cpu().float().permute(0, 3, 1, 2, 4)[~written]
    assert bool((untouched == 7.0).all())
    # the dispatching entry point takes this kernel where its tiles fill the GPU, else a product and the rotary kernel
    cache_c = torch.full((pages, 2, nkv, page, hd), 7.0, device="cuda").bfloat16()
    before = COUNTERS["launches"]
    qc = K.qkv_rope_cache_write(x, w, b, positions, cos, sin, slots, cache_c, nh, nkv, hd)
    if K._use_decode_gemm(M, N, Kd, False):          # few tiles: the weight-streaming kernel in blocks of 128 rows
        assert COUNTERS["launches"] == before + 1 and same_up_to_an_ulp(qc, qa) and same_up_to_an_ulp(cache_c, cache_a)
    elif K._tcgen05_fills(M, N):
        assert COUNTERS["launches"] == before + 1 and torch.equal(qc, qa) and torch.equal(cache_c, cache_a)
    else:
        assert same_up_to_an_ulp(qc, qa) and same_up_to_an_ulp(cache_c, cache_a)


TC_ATT_CASES = [
    # nh, nkv, hd, page, q_lens, ctx_lens, window
    (4, 1, 128, 16, [32], [32], None),
    (8, 2, 128, 16, [200], [500], None),
    (8, 2, 64, 8, [70, 1, 33], [70, 9, 129], 40),
    (2, 2, 64, 32, [300], [300], None),
    (16, 1, 128, 64, [40, 50], [300, 50], 100),
    (32, 8, 128, 16, [333, 1, 64], [777, 100, 64], None),
    (8, 8, 128, 128, [17], [400], 256),
    # groups that do not divide the 128 rows of a tile: 18 tokens of 7 heads, 25 of 5, 42 of 3, 21 of 6, one of 100
    (28, 4, 128, 16, [300, 1, 19], [700, 50, 19], None),
    (10, 2, 64, 16, [127, 26], [127, 400], 60),
    (3, 1, 128, 32, [85, 43], [200, 43], None),
    (12, 2, 64, 8, [64], [1000], None),
    (100, 1, 64, 16, [5], [70], None),
]


@pytest.mark.parametrize("case", TC_ATT_CASES)
def test_attention_tcgen05_kernel(K, case):
    """The tcgen05 attention kernel for prompt portions (sequences of one token are left alone),
    through the product path's dispatch and directly, with its status word."""
    nh, nkv, hd, page, q_lens, ctx_lens, window = case
    ks, vs, qs = _attention_case(nh, nkv, hd, page, q_lens, ctx_lens, window, 11)
    cache, meta = paged_setup(ks, vs, q_lens, page, torch.bfloat16)
    q = torch.cat(qs).reshape(sum(q_lens), nh * hd).cuda().bfloat16()
    scale = 1 / math.sqrt(hd)
    ref = _attention_ref(ks, vs, qs, ctx_lens, q_lens, scale, window, torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros_like(q)
    K.attention_tcgen05(q, cache, meta, out, nh, nkv, hd, scale, window, status=status)
    rows = torch.cat([torch.full((n,), n > 1) for n in q_lens])
    assert rel_err(out.view(-1, nh, hd)[rows.cuda()], ref[rows]) < BF16_TOL
    assert float(out.view(-1, nh, hd)[(~rows).cuda()].abs().sum()) == 0.0        # one-token sequences untouched
    assert int(status.item()) == 0, "a bounded wait inside the kernel gave up"
    full = K.paged_attention(q, cache, meta, nh, nkv, hd, scale, window)          # with the decode kernel for the rest
    assert rel_err(full.view(-1, nh, hd), ref) < BF16_TOL


def test_fill_normal_kernel_is_counter_based_and_normal(K):
    """The random-weights fill: element i is a function of (seed, stream, i) - checked against the
    plain Philox and Box-Muller for the first elements -, the same whatever the size of the launch,
    different for another seed or stream, and normal in its first four moments."""
    n = 1_000_004
    a = K.fill_normal((n,), torch.float32, 0.0, 1.0, seed=7, stream=3)
    assert torch.equal(a[:1001], K.fill_normal((1001,), torch.float32, 0.0, 1.0, seed=7, stream=3))
    assert not torch.equal(a[:1000], K.fill_normal((1000,), torch.float32, 0.0, 1.0, seed=8, stream=3))
    assert not torch.equal(a[:1000], K.fill_normal((1000,), torch.float32, 0.0, 1.0, seed=7, stream=4))
    for qd in (0, 1, 250_000):
        w = P.philox4x32([qd, 0, 3, 0], [7, 0])
        for h in range(2):
            u1, u2 = ((w[2 * h] >> 8) + 0.5) / 16777216.0, (w[2 * h + 1] >> 8) / 16777216.0
            r = math.sqrt(-2.0 * math.log(u1))
            assert abs(float(a[4 * qd + 2 * h]) - r * math.cos(2 * math.pi * u2)) < 1e-5
            assert abs(float(a[4 * qd + 2 * h + 1]) - r * math.sin(2 * math.pi * u2)) < 1e-5
    d = a.double()
    assert abs(float(d.mean())) < 5e-3 and abs(float(d.std()) - 1) < 5e-3
    assert abs(float((d ** 3).mean())) < 2e-2 and abs(float((d ** 4).mean()) - 3) < 5e-2
    b = K.fill_normal((300, 1000), torch.bfloat16, 1.0, 0.1, seed=1, stream=0).double()
    assert b.shape == (300, 1000) and abs(float(b.mean()) - 1) < 2e-3 and abs(float(b.std()) - 0.1) < 2e-3
