"""The plain implementation itself: hand-computed values and properties that must hold."""
import math

import pytest
import torch

import plain_impl as P
import tiny_configs
from model_tools import model_folder


def test_rms_norm_hand_value():
    # own numbers: x = [3, 4], gamma = [1, 2]: mean square 12.5
    y = P.rms_norm(torch.tensor([[3.0, 4.0]], dtype=torch.float64), torch.tensor([1.0, 2.0], dtype=torch.float64), 0.0)
    r = 1.0 / math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([[3 * r, 8 * r]], dtype=torch.float64))


def test_the_reference_s_own_literal_vectors():
    """The only literal numbers the reference's code carries: the unit tests of its float oracle
    (v3/crates/rvllm-fused/src/reference.rs:247-304), restated here."""
    # rmsnorm_matches_hand_calc (:247-259): x = [1, 2, 3], gamma = 1, eps = 0 -> x / sqrt(14 / 3)
    x = torch.tensor([[1.0, 2.0, 3.0]], dtype=torch.float64)
    y = P.rms_norm(x, torch.ones(3, dtype=torch.float64), 0.0)
    assert (y - x / math.sqrt(14.0 / 3.0)).abs().max() < 1e-6
    # argmax_returns_largest (:261-268): rows [0.1, 0.9, 0.3] -> 1 and [0.5, -1.0, 0.8] -> 2
    assert P.argmax_lowest(torch.tensor([0.1, 0.9, 0.3])) == 1
    assert P.argmax_lowest(torch.tensor([0.5, -1.0, 0.8])) == 2
    # embedding_gather_picks_row (:284-293): a 3 x 2 table, ids [2, 0]
    table = torch.tensor([[10.0, 11.0], [20.0, 21.0], [30.0, 31.0]], dtype=torch.float64)
    assert P.embedding([2, 0], table).tolist() == [[30.0, 31.0], [10.0, 11.0]]
    # rope_is_orthogonal_preserving (:295-304): one token at position 0, one head of 4 (cos 1, sin 0)
    q = torch.tensor([[[1.0, 0.0, 0.0, 1.0]]], dtype=torch.float64)
    assert P.apply_rope(q, [0], P.rope_inv_freq(4, 10000.0, None)).tolist() == q.tolist()
    # silu_mul (:270-282 gives gate [0, 1, -1, 2], up 1 and checks only that something is non-zero):
    # silu(0) = 0, silu(1) = 1 / (1 + e^-1)
    g = torch.tensor([[0.0, 1.0, -1.0, 2.0]], dtype=torch.float64)
    eye = torch.eye(4, dtype=torch.float64)
    h = P.gated_mlp(torch.ones(1, 4, dtype=torch.float64) , torch.diag(g[0]), eye, eye)
    assert abs(float(h[0, 0])) == 0.0 and abs(float(h[0, 1]) - 1.0 / (1.0 + math.exp(-1.0))) < 1e-12


def test_rope_pairs_are_half_split_and_keep_norms():
    x = torch.randn(5, 2, 8, dtype=torch.float64)
    inv = P.rope_inv_freq(8, 10000.0, None)
    y = P.apply_rope(x, [0, 1, 2, 3, 40], inv)
    assert torch.allclose(y[0], x[0])                                   # position 0: no rotation
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    a = float(inv.float()[1]) * 3                                        # pair (1, 5) at position 3
    want1 = x[3, 0, 1] * math.cos(a) - x[3, 0, 5] * math.sin(a)
    want5 = x[3, 0, 1] * math.sin(a) + x[3, 0, 5] * math.cos(a)
    assert abs(float(y[3, 0, 1] - want1)) < 1e-12 and abs(float(y[3, 0, 5] - want5)) < 1e-12
    # relative property: q.k depends on the distance only
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    d1 = (P.apply_rope(q, [7], inv) * P.apply_rope(k, [3], inv)).sum()
    d2 = (P.apply_rope(q, [104], inv) * P.apply_rope(k, [100], inv)).sum()
    assert abs(float(d1 - d2)) < 1e-9


def test_llama3_scaling_has_three_bands():
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 32}
    base = P.rope_inv_freq(16, 10000.0, None)
    inv = P.rope_inv_freq(16, 10000.0, sc)
    ratio = (inv / base).tolist()
    assert ratio[0] == 1.0                                               # short wavelengths are kept
    assert abs(ratio[-1] - 1 / 8) < 1e-12                                # long ones are divided by the factor
    assert any(1 / 8 + 1e-6 < r < 1 - 1e-6 for r in ratio)               # and some are blended
    assert all(a >= b for a, b in zip(ratio, ratio[1:]))


def test_attention_is_causal_and_windowed():
    torch.manual_seed(0)
    q, k, v = (torch.randn(12, 4, 8, dtype=torch.float64) for _ in range(3))
    k, v = k[:, :2], v[:, :2]
    o = P.causal_attention(q, k, v, 0.3)
    k2, v2 = k.clone(), v.clone()
    k2[8:], v2[8:] = 9.0, -9.0
    assert torch.allclose(P.causal_attention(q, k2, v2, 0.3)[:8], o[:8])      # the future is not seen
    assert torch.allclose(o[0], v[0, [0, 0, 1, 1]])                            # first token sees itself; heads 0,1 -> kv 0
    w = P.causal_attention(q, k, v, 0.3, window=3)
    assert torch.allclose(w[:3], o[:3])                                       # window not yet full
    k3, v3 = k.clone(), v.clone()
    k3[:7], v3[:7] = 5.0, 5.0
    assert torch.allclose(P.causal_attention(q, k3, v3, 0.3, window=3)[9:], w[9:])   # keys <= p - 3 are out
    assert not torch.allclose(P.causal_attention(q, k3, v3, 0.3, window=4)[9], w[9])


def test_whole_model_prefix_property_and_tying():
    for name in ("tiny_llama", "tiny_qwen2"):
        cfg, w = P.read_model_folder(model_folder(name))
        toks = list(range(3, 60))
        full = P.forward(cfg, w, toks)
        assert full.shape == (57, cfg["vocab_size"]) and torch.isfinite(full).all()
        assert torch.allclose(P.forward(cfg, w, toks[:20]), full[:20], atol=1e-10)
    cfg, w = P.read_model_folder(model_folder("tiny_qwen2"))
    assert "lm_head.weight" not in w and P.has_qkv_bias(cfg)
    assert P.layer_windows(cfg) == [None, 40, 40]


def test_window_matters_in_the_tiny_qwen2_model():
    cfg, w = P.read_model_folder(model_folder("tiny_qwen2"))
    toks = [(7 * i) % cfg["vocab_size"] for i in range(80)]
    a = P.forward(cfg, w, toks)
    cfg2 = dict(cfg, use_sliding_window=False)
    b = P.forward(cfg2, w, toks)
    assert torch.allclose(a[:40], b[:40], atol=1e-10)                   # up to 40 keys the window hides nothing
    assert (a[60:] - b[60:]).abs().max() > 1e-6


def test_philox_known_answers():
    # test vectors published with the Random123 library for philox4x32-10
    assert P.philox4x32([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert P.philox4x32([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert P.philox4x32([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]
    us = [P.uniform_for(5, i) for i in range(2000)]
    assert all(0.0 <= u < 1.0 for u in us) and abs(sum(us) / len(us) - 0.5) < 0.03


def test_sampling_rules():
    logits = torch.tensor([1.0, 3.0, 3.0, -2.0])
    assert P.argmax_lowest(logits) == 1                                  # lowest index wins ties
    assert P.sample(logits, 0.0, 0, 0)[0] == 1
    p = P.filtered_probs(torch.tensor([0.0, 1.0, 2.0, 3.0]), 1.0, top_k=2)
    assert p[0] == 0 and p[1] == 0 and abs(float(p[2] + p[3]) - 1) < 1e-12
    p = P.filtered_probs(torch.tensor([0.0, 1.0, 2.0, 3.0]), 1.0, top_p=0.5)
    assert (p > 0).tolist() == [False, False, False, True]               # the top token alone has mass 0.64 >= 0.5
    p = P.filtered_probs(torch.tensor([0.0, 1.0, 2.0, 3.0]), 1.0, top_p=0.7)
    assert (p > 0).tolist() == [False, False, True, True]
    counts = torch.zeros(4)
    z = torch.tensor([0.5, 1.5, 0.0, 1.0])
    for i in range(4000):
        counts[P.sample(z, 0.8, 11, i)[0]] += 1
    want = torch.softmax(z.double() / 0.8, 0) * 4000
    chi2 = float(((counts - want) ** 2 / want).sum())
    assert chi2 < 16.3                                                   # 3 degrees of freedom, p = 0.001
