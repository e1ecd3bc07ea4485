"""Each part of a layer alone on the GPU against the plain function of the same part."""
import math

import pytest
import torch

import plain_impl as P
from gpu_tools import rel_err

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}
DTYPES = [torch.float32, torch.bfloat16]


class Harness:
    """A cache manager and a step packer around parts that are not inside a model."""

    def __init__(self, needs, dtype, page=8, pages=64, max_len=512):
        from rvllm_b200.cache import CacheManager
        from rvllm_b200.engine import ModelRunner
        from rvllm_b200.kernels import get_library
        self.kernels = get_library("cuda:0")
        self.cache = CacheManager(needs, pages, page, 4, dtype, "cuda:0")
        self.runner = ModelRunner(None, self.cache, self.kernels, max_len, "cuda:0")

    def ctx(self, entries):
        from rvllm_b200.engine import StepEntry
        es = [StepEntry(rid, toks, ()) for rid, toks in entries]
        starts = self.runner.reserve(es)
        return self.runner.pack(es, starts)


def bind_random(part, dtype, seed=0):
    from rvllm_b200.weights.random_init import random_tensors
    specs = part.tensor_specs()
    tensors = random_tensors(specs, seed, dtype)
    part.bind(lambda n: tensors[n].cuda())
    return {k: v.double() for k, v in tensors.items()}


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from rvllm_b200.parts import NORMS
    norm = NORMS.build("rmsnorm", size=200, eps=3e-4)
    w = bind_random(norm, dtype)
    h = Harness({}, dtype)
    x = torch.randn(11, 200, device="cuda").to(dtype)
    out = norm(x, h.ctx([("a", [1] * 11)]))
    assert rel_err(out, P.rms_norm(x.double().cpu(), w["weight"], 3e-4)) < TOL[dtype]


def test_rotary_tables_match_float64():
    from rvllm_b200.parts import POSITION_ENCODINGS
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    for scaling in (None, sc):
        rope = POSITION_ENCODINGS.build("rotary", head_dim=48, theta=500000.0, scaling=scaling)
        rope.prepare(3000, "cuda")
        inv = P.rope_inv_freq(48, 500000.0, scaling).float().double()
        ang = torch.arange(3000, dtype=torch.float64)[:, None] * inv[None]
        assert float((rope.cos.double().cpu() - torch.cos(ang)).abs().max()) < 1e-7
        assert float((rope.sin.double().cpu() - torch.sin(ang)).abs().max()) < 1e-7
        assert torch.equal(rope.inv_freq.double(), inv)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,bias,window", [(6, 2, 32, True, None), (5, 5, 16, False, 24), (8, 1, 64, True, 100)])
def test_attention_mixer(dtype, nh, nkv, hd, bias, window):
    """The mixer over a cache it filled in earlier steps: a whole sequence fed in three cuts."""
    from rvllm_b200.parts import MIXERS, POSITION_ENCODINGS
    H, T = 72, 90
    rope = POSITION_ENCODINGS.build("rotary", head_dim=hd, theta=10000.0, scaling=None)
    rope.prepare(512, "cuda")
    att = MIXERS.build("paged_attention", hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                       scale=0.37, qkv_bias=bias, window=window, position=rope)
    w = bind_random(att, dtype, seed=3)
    h = Harness({0: att.cache_need()}, dtype)
    torch.manual_seed(0)
    x = torch.randn(T, H).to(dtype)
    res = torch.randn(T, H).to(dtype)
    outs = []
    pos = 0
    for n in (41, 2, 47):
        ctx = h.ctx([("a", [0] * n)])
        outs.append(att(x[pos:pos + n].cuda(), ctx, h.cache.view(0), residual=res[pos:pos + n].cuda()))
        h.cache.release_passed("a")
        pos += n
    got = torch.cat(outs)
    xd = x.double()
    q = P.linear(xd, w["q_proj.weight"], w.get("q_proj.bias")).view(T, nh, hd)
    k = P.linear(xd, w["k_proj.weight"], w.get("k_proj.bias")).view(T, nkv, hd)
    v = P.linear(xd, w["v_proj.weight"], w.get("v_proj.bias")).view(T, nkv, hd)
    inv = P.rope_inv_freq(hd, 10000.0, None)
    q, k = P.apply_rope(q, range(T), inv), P.apply_rope(k, range(T), inv)
    o = P.causal_attention(q, k, v, 0.37, window).reshape(T, nh * hd)
    ref = res.double() + P.linear(o, w["o_proj.weight"])
    assert rel_err(got, ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [3, 150])
def test_gated_mlp(dtype, rows):
    from rvllm_b200.parts import FEED_FORWARDS
    mlp = FEED_FORWARDS.build("gated_mlp", hidden_size=88, intermediate_size=172)
    w = bind_random(mlp, dtype, seed=5)
    h = Harness({}, dtype)
    x = torch.randn(rows, 88).to(dtype)
    res = torch.randn(rows, 88).to(dtype)
    out = mlp(x.cuda(), h.ctx([("a", [1] * rows)]), residual=res.cuda())
    ref = res.double() + P.gated_mlp(x.double(), w["gate_proj.weight"], w["up_proj.weight"], w["down_proj.weight"])
    assert rel_err(out, ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_equals_plain_decoder_layer(dtype):
    """A whole pre-norm block built from registry parts against the plain layer function."""
    from rvllm_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS
    cfg = {"architectures": ["Qwen2ForCausalLM"], "hidden_size": 56, "num_attention_heads": 4, "num_key_value_heads": 2,
           "head_dim": 16, "rms_norm_eps": 2e-5, "rope_theta": 7000.0}
    rope = POSITION_ENCODINGS.build("rotary", head_dim=16, theta=7000.0, scaling=None)
    rope.prepare(256, "cuda")
    att = MIXERS.build("paged_attention", hidden_size=56, num_heads=4, num_kv_heads=2, head_dim=16, scale=0.25,
                       qkv_bias=True, position=rope)
    mlp = FEED_FORWARDS.build("gated_mlp", hidden_size=56, intermediate_size=100)
    n1, n2 = NORMS.build("rmsnorm", size=56, eps=2e-5), NORMS.build("rmsnorm", size=56, eps=2e-5)
    block = BLOCKS.build("prenorm_residual", parts={"mixer": att, "feed_forward": mlp, "mixer_norm": n1, "feed_forward_norm": n2})
    w = {}
    for prefix, part, seed in (("self_attn.", att, 1), ("mlp.", mlp, 2), ("input_layernorm.", n1, 3),
                               ("post_attention_layernorm.", n2, 4)):
        w.update({"L." + prefix + k: v for k, v in bind_random(part, dtype, seed).items()})
    h = Harness({0: att.cache_need()}, dtype)
    x = torch.randn(37, 56).to(dtype)
    out = block(x.cuda(), h.ctx([("a", [0] * 37)]), h.cache.view(0))
    ref = P.decoder_layer(x.double(), list(range(37)), cfg, w, "L.", P.rope_inv_freq(16, 7000.0, None), None)
    assert rel_err(out, ref) < TOL[dtype]


def test_unknown_part_names_the_known_ones():
    from rvllm_b200 import ConfigError
    from rvllm_b200.parts import MIXERS
    with pytest.raises(ConfigError, match="paged_attention"):
        MIXERS.build("mamba", size=3)
