"""The sampling kernel against the plain sampler."""
import pytest
import torch

import plain_impl as P

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from rvllm_b200.kernels import get_library
    return get_library("cuda:0")


def test_greedy_ties_and_nan(K):
    logits = torch.randn(6, 1000)
    logits[0, 17] = logits[0, 900] = 9.0                 # a tie: the lowest index wins
    logits[1, 0] = 50.0
    logits[2, 999] = 50.0
    logits[3, 5] = float("nan")                           # NaN never wins
    logits[3, 6] = 40.0
    logits[4] = -3.0                                      # all equal: index 0
    out = K.sample(logits.cuda()).tolist()
    assert out[:5] == [17, 0, 999, 6, 0]
    assert out[5] == P.argmax_lowest(logits[5])
    big = torch.randn(3, 128256)
    assert K.sample(big.cuda()).tolist() == [P.argmax_lowest(r) for r in big]


@pytest.mark.parametrize("vocab", [383, 5000, 128256])
@pytest.mark.parametrize("top_k,top_p", [(0, 1.0), (20, 1.0), (0, 0.8), (50, 0.9)])
def test_draws_match_the_plain_sampler(K, vocab, top_k, top_p):
    torch.manual_seed(vocab + top_k)
    R = 24
    logits = torch.randn(R, vocab) * (2.5 if vocab < 10000 else 8.0)    # peaked, so that steps of the CDF are wide
    temps = torch.tensor([0.7 + 0.05 * (i % 5) for i in range(R)])
    temps[3] = 0.0                                        # a greedy row among sampled ones
    seeds = torch.arange(100, 100 + R, dtype=torch.int64)
    draws = torch.arange(R, dtype=torch.int64) * 7
    out = K.sample(logits.cuda(), temps.cuda(), torch.full((R,), top_k, dtype=torch.int32).cuda() if top_k else None,
                   torch.full((R,), top_p).cuda() if top_p < 1 else None, seeds.cuda(), draws.cuda()).tolist()
    checked = 0
    for r in range(R):
        tok, margin = P.sample(logits[r], float(temps[r]), int(seeds[r]), int(draws[r]), top_k, top_p)
        if margin < 1e-4:
            continue          # u sits on a step of the CDF: float rounding may pick the neighbour
        if top_p < 1.0:
            p = torch.softmax(logits[r].double() / float(temps[r]), 0) if temps[r] > 0 else None
            if p is not None:
                sp = torch.sort(p, descending=True).values
                cs = torch.cumsum(sp, 0)
                n = int((cs < top_p).sum()) + 1
                if abs(float(cs[n - 1]) - top_p) < 3e-6 or (n > 1 and abs(float(cs[n - 2]) - top_p) < 3e-6):
                    continue  # the top-p cut itself sits on a rounding edge
        assert out[r] == tok, f"row {r}: kernel {out[r]}, plain {tok} (margin {margin:.2e})"
        checked += 1
    assert checked >= R // 2


def test_distribution_and_batch_independence(K):
    z = torch.tensor([0.5, 1.5, 0.0, 1.0, -1.0, 2.0])
    n = 6000
    logits = z.repeat(n, 1).cuda()
    temps = torch.full((n,), 0.8).cuda()
    seeds = torch.full((n,), 77, dtype=torch.int64).cuda()
    draws = torch.arange(n, dtype=torch.int64).cuda()
    out = K.sample(logits, temps, None, None, seeds, draws)
    counts = torch.bincount(out.long().cpu(), minlength=6).double()
    want = torch.softmax(z.double() / 0.8, 0) * n
    assert float(((counts - want) ** 2 / want).sum()) < 20.5          # 5 degrees of freedom, p = 0.001
    # the same (seed, output index) gives the same token whatever else is in the batch
    sub = K.sample(logits[100:103].contiguous(), temps[:3].contiguous(), None, None, seeds[:3].contiguous(),
                   draws[100:103].contiguous())
    assert sub.tolist() == out[100:103].tolist()


def test_sampler_object_and_parameter_checks(K):
    from rvllm_b200 import Sampler, SamplingError, SamplingParams
    s = Sampler(K)
    logits = torch.randn(3, 500).cuda()
    greedy = s.sample(logits, [SamplingParams()] * 3, [0, 0, 0], [0, 0, 0])
    assert greedy.tolist() == [P.argmax_lowest(r) for r in logits.cpu()]
    mixed = s.sample(logits, [SamplingParams(), SamplingParams(temperature=1.0, top_k=1), SamplingParams(temperature=0.5, top_p=0.01)],
                     [1, 2, 3], [0, 0, 0])
    assert mixed.tolist() == greedy.tolist()                          # top_k = 1 and a tiny top_p are greedy too
    for bad in (dict(temperature=-1.0), dict(top_p=0.0), dict(top_p=1.5), dict(top_k=-2), dict(max_tokens=0)):
        with pytest.raises(SamplingError):
            SamplingParams(**bad)
    with pytest.raises(SamplingError):
        s.sample(logits, [SamplingParams()], [0], [0])


@pytest.mark.parametrize("vocab", [5, 31, 383, 5000, 128256])
def test_the_token_does_not_depend_on_how_many_ctas_share_a_row(K, vocab):
    """A row is cut into eight slices whatever the launch; one, two, four or eight CTAs (a thread-block
    cluster, results exchanged through distributed shared memory) work through them: the same
    arithmetic in the same order, so the same tokens bit for bit - greedy, temperature, top-k, top-p,
    rows of NaN and rows of equal logits included."""
    from ctypes import c_int
    torch.manual_seed(vocab)
    R = 7
    logits = torch.randn(R, vocab) * 4
    logits[1] = 2.0                                       # all equal
    logits[2] = float("nan")                              # nothing to keep: the arg-max rule (index 0)
    if vocab > 20:
        logits[3, 7] = logits[3, vocab - 2] = 30.0        # a tie across slices
    temps = torch.tensor([0.8, 1.0, 0.9, 0.7, 0.0, 1.3, 0.6])
    seeds = torch.arange(5, 5 + R, dtype=torch.int64)
    draws = torch.arange(R, dtype=torch.int64) * 3
    tk = torch.tensor([0, 3, 2, 0, 5, min(40, vocab - 1), 1], dtype=torch.int32)
    tp = torch.tensor([1.0, 0.9, 0.5, 0.95, 0.8, 0.7, 1.0])
    lib = K._lib("sampling.cu")
    results = []
    try:
        for cl in (1, 2, 4, 8):
            lib.rv_sample_set_cluster(c_int(cl))
            g = logits.cuda()
            results.append((K.sample(g).tolist(),
                            K.sample(g, temps.cuda(), None, None, seeds.cuda(), draws.cuda()).tolist(),
                            K.sample(g, temps.cuda(), tk.cuda(), None, seeds.cuda(), draws.cuda()).tolist(),
                            K.sample(g, temps.cuda(), tk.cuda(), tp.cuda(), seeds.cuda(), draws.cuda()).tolist()))
    finally:
        lib.rv_sample_set_cluster(c_int(0))
    assert all(r == results[0] for r in results[1:]), results
    greedy = results[0][0]
    assert greedy[1] == 0 and greedy[2] == 0 and (vocab <= 20 or greedy[3] == 7)
    assert results[0][3][6] == greedy[6]                  # top-k of one: the most likely token
    assert results[0][1][4] == greedy[4]                  # temperature 0 among sampled rows


@pytest.mark.parametrize("vocab,spread", [(128256, 8.0), (128256, 1.0), (5000, 3.0), (383, 0.2)])
def test_the_short_way_and_the_general_search_draw_the_same_tokens(K, vocab, spread):
    """Top-k / top-p rows first try one histogram and a sort of the few candidates; flat distributions
    (too many candidates) fall back to the general digit-by-digit search.  Both must keep the same
    set and draw the same token: compared row by row with the short way switched off, over peaked and
    flat rows, k from 1 to beyond the candidate limit, p from 0.1 to 0.999, ties and NaN."""
    from ctypes import c_int
    torch.manual_seed(vocab + int(spread * 10))
    R = 48
    logits = torch.randn(R, vocab) * spread
    logits[1, 5] = logits[1, vocab - 3] = logits[1].max() + 1.0          # a tie at the top
    logits[2, ::7] = float("nan")
    logits[3] = 1.5                                                       # all equal
    temps = torch.tensor([0.5 + 0.03 * i for i in range(R)])
    ks = torch.tensor([(0, 1, 2, 5, 50, 300, 2047, 2048, 5000, 100000)[i % 10] for i in range(R)], dtype=torch.int32)
    ps = torch.tensor([(1.0, 0.1, 0.5, 0.9, 0.95, 0.999, 0.7)[i % 7] for i in range(R)])
    seeds = torch.arange(900, 900 + R, dtype=torch.int64)
    draws = torch.arange(R, dtype=torch.int64) * 5
    lib = K._lib("sampling.cu")
    g = logits.cuda()
    try:
        assert lib.rv_sample_set_short_way(c_int(0)) == 0
        general = K.sample(g, temps.cuda(), ks.cuda(), ps.cuda(), seeds.cuda(), draws.cuda()).tolist()
        general_k = K.sample(g, temps.cuda(), ks.cuda(), None, seeds.cuda(), draws.cuda()).tolist()
    finally:
        assert lib.rv_sample_set_short_way(c_int(1)) == 0
    short = K.sample(g, temps.cuda(), ks.cuda(), ps.cuda(), seeds.cuda(), draws.cuda()).tolist()
    short_k = K.sample(g, temps.cuda(), ks.cuda(), None, seeds.cuda(), draws.cuda()).tolist()
    # the two ways add the masses up in different orders; a draw within rounding of a step of the CDF may differ
    differ = [r for r in range(R) if short[r] != general[r]] + [r for r in range(R) if short_k[r] != general_k[r]]
    for r in differ:
        _, margin = P.sample(logits[r].nan_to_num(float("-inf")), float(temps[r]), int(seeds[r]), int(draws[r]),
                             int(ks[r]) if 0 < int(ks[r]) < vocab else 0, float(ps[r]))
        assert margin < 1e-4, f"row {r}: short way {short[r]}, general search {general[r]}, margin {margin:.2e}"
    assert len(differ) <= 3
    assert all(0 <= t < vocab for t in short + short_k)
