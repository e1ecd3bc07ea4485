"""Toy parts defined here - a mixer with state of its own, a feed-forward with a router, a position
encoding added to the embeddings, a block arrangement with four norms, hooks on the embeddings and
on the logits - are registered, built into a model through a toy architecture, loaded from a
random-weights folder and stepped - prompts cut into portions, decoding, several live requests,
slots used again - without touching the framework's files.  The attention layers of the toy
rotate only the first half of each head (a rotary_dim below head_dim), and the state mixer says
that it cannot be captured in a CUDA graph, so the engine runs the toy's decode steps eagerly
even with graphs switched on.

The toy mixer keeps a running, decayed sum of projected inputs per request:
    s_t = decay * s_{t-1} + x_t W^T ;  y_t = s_t
which has a closed form to compare with.  It is no model of anyone's; it only shows that
state slots, registration and the step function carry a mixer that is not attention.  The
torch operations inside it run on whatever device the engine runs on, so the test exists in a
CPU form (with the emulated kernels for the other parts) and in a GPU form.
"""
import json
import os
from dataclasses import dataclass

import pytest
import torch

from rvllm_b200 import config_from_dict, kernels as kernel_pkg, register_architecture, write_random_model
from rvllm_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry, unregister_architecture
from rvllm_b200.parts import BLOCKS, FEED_FORWARDS, HOOKS, MIXERS, POSITION_ENCODINGS, Part, StateNeed, TensorSpec

DECAY = 0.9
SOFTCAP = 5.0
EMBED_SCALE = 1.5
ROTARY_DIM = 8         # of a head of 16


class RunningSumMixer(Part):
    graph_safe = False     # it reads the state slots on the host: its steps cannot be captured

    def __init__(self, hidden_size: int, state_size: int):
        self.hidden_size, self.state_size = hidden_size, state_size
        self.w_in = self.w_out = None

    def tensor_specs(self):
        return {"in_proj.weight": TensorSpec((self.state_size, self.hidden_size), "matrix"),
                "out_proj.weight": TensorSpec((self.hidden_size, self.state_size), "matrix")}

    def bind(self, get):
        self.w_in, self.w_out = get("in_proj.weight"), get("out_proj.weight")

    def cache_need(self):
        return StateNeed((self.state_size,), "float32")

    def __call__(self, x, ctx, cache, residual=None, write_cache=True):
        u = x.float() @ self.w_in.float().t()                       # [T, state]
        out = torch.empty_like(u)
        slots = ctx.state_slots.tolist()
        start = 0
        for seq, n in enumerate(ctx.q_lens):                        # tokens of a request run in order
            slot = slots[seq]
            if slot < 0:                                            # a padding row of a graph bucket
                out[start:start + n] = 0
                start += n
                continue
            s = cache.state[slot]
            for t in range(start, start + n):
                s = DECAY * s + u[t]
                out[t] = s
            cache.state[slot] = s
            start += n
        y = (out @ self.w_out.float().t()).to(x.dtype)
        return y if residual is None else residual + y


class RoutedExperts(Part):
    """Feed-forward with a router: y = sum_e softmax(x R^T)_e * down_e(relu(up_e x)), the router in
    float32.  Every expert weighs in (no hard choice that a rounding could flip)."""

    def __init__(self, hidden_size: int, expert_size: int, num_experts: int):
        self.hidden_size, self.expert_size, self.num_experts = hidden_size, expert_size, num_experts
        self.router = None
        self.up, self.down = [], []

    def tensor_specs(self):
        specs = {"router.weight": TensorSpec((self.num_experts, self.hidden_size), "matrix")}
        for e in range(self.num_experts):
            specs[f"experts.{e}.up.weight"] = TensorSpec((self.expert_size, self.hidden_size), "matrix")
            specs[f"experts.{e}.down.weight"] = TensorSpec((self.hidden_size, self.expert_size), "matrix")
        return specs

    def bind(self, get):
        self.router = get("router.weight")
        self.up = [get(f"experts.{e}.up.weight") for e in range(self.num_experts)]
        self.down = [get(f"experts.{e}.down.weight") for e in range(self.num_experts)]

    def __call__(self, x, ctx, residual=None):
        xf = x.float()
        gate = torch.softmax(xf @ self.router.float().t() * 8.0, dim=-1)           # [T, E]
        y = torch.zeros_like(xf)
        for e in range(self.num_experts):
            y = y + gate[:, e:e + 1] * (torch.relu(xf @ self.up[e].float().t()) @ self.down[e].float().t())
        y = y.to(x.dtype)
        return y if residual is None else residual + y


class LearnedPositions(Part):
    """A table of position vectors added to the embeddings; no rotation tables."""

    def __init__(self, hidden_size: int, max_len: int):
        self.hidden_size, self.max_len = hidden_size, max_len
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.max_len, self.hidden_size), "matrix")}

    def bind(self, get):
        self.weight = get("weight")

    def prepare(self, max_len, device):
        pass

    def rotation_tables(self):
        return None

    def on_embeddings(self, x, ctx):
        return x + self.weight[ctx.positions.long()].to(x.dtype)


class SandwichBlock:
    """x + norm(mixer(norm(x))), then + norm(feed_forward(norm(.))): four norms, each with a weight
    of its own, around the two parts."""
    ROLES = ("mixer", "feed_forward", "pre_mixer_norm", "post_mixer_norm", "pre_ffn_norm", "post_ffn_norm")

    def __init__(self, parts):
        assert sorted(parts) == sorted(self.ROLES)
        self.p = parts

    def __call__(self, x, ctx, cache, write_cache=True):
        p = self.p
        h = p["mixer"](p["pre_mixer_norm"](x, ctx), ctx, cache, residual=None, write_cache=write_cache)
        x = x + p["post_mixer_norm"](h, ctx)
        h = p["feed_forward"](p["pre_ffn_norm"](x, ctx), ctx, residual=None)
        return x + p["post_ffn_norm"](h, ctx)


class Scale(Part):
    def __init__(self, factor: float):
        self.factor = factor

    def __call__(self, x, ctx):
        return x * self.factor


class SoftCap(Part):
    def __init__(self, cap: float):
        self.cap = cap

    def __call__(self, logits, ctx):
        return torch.tanh(logits / self.cap) * self.cap


@dataclass(frozen=True)
class ToyConfig:
    hidden_size: int
    state_size: int
    vocab_size: int
    num_layers: int
    raw: dict

    @classmethod
    def from_dict(cls, obj, where="config.json"):
        return cls(obj["hidden_size"], obj["state_size"], obj["vocab_size"], obj["num_layers"], dict(obj))

    def to_dict(self):
        return dict(self.raw)

    def to_spec(self):
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": 1e-5})
        layers = []
        for i in range(self.num_layers):
            # odd layers are ordinary attention layers: two kinds of mixer in one model
            if i % 2:
                mixer = PartSpec("paged_attention", {"hidden_size": self.hidden_size, "num_heads": 2, "num_kv_heads": 1,
                                                     "head_dim": 16, "scale": 0.25, "position": "rope"})
            else:
                mixer = PartSpec("running_sum", {"hidden_size": self.hidden_size, "state_size": self.state_size})
            # even layers have the routed feed-forward, odd ones the gated MLP
            ffn = (PartSpec("gated_mlp", {"hidden_size": self.hidden_size, "intermediate_size": 40}) if i % 2 else
                   PartSpec("routed_experts", {"hidden_size": self.hidden_size, "expert_size": 12, "num_experts": 3}))
            if i % 2:
                # the attention layers use the block with four norms, named part by part
                n = PartSpec("rmsnorm", norm.params, "norm")
                layers.append(LayerSpec(prefix=f"layers.{i}.", block=PartSpec("sandwich"),
                                        parts={"mixer": PartSpec(mixer.kind, mixer.params, "mixer"),
                                               "feed_forward": PartSpec(ffn.kind, ffn.params, "feed_forward"),
                                               "pre_mixer_norm": n, "post_mixer_norm": n, "pre_ffn_norm": n, "post_ffn_norm": n},
                                        names={"feed_forward": "ffn.", "pre_mixer_norm": "norm1.", "post_mixer_norm": "norm1b.",
                                               "pre_ffn_norm": "norm2.", "post_ffn_norm": "norm2b."}))
                continue
            layers.append(LayerSpec.standard(prefix=f"layers.{i}.", block=PartSpec("prenorm_residual"), mixer=mixer,
                                             feed_forward=ffn, mixer_norm=norm, feed_forward_norm=norm,
                                             names={"mixer": "mixer.", "feed_forward": "ffn.", "mixer_norm": "norm1.",
                                                    "feed_forward_norm": "norm2."}))
        # the run order names layer 0 twice (its second run has a state of its own) and lets the
        # last entry read the keys and values that layer 1 wrote
        order = (RunEntry(0, 0), RunEntry(1, 1), RunEntry(0, 2), RunEntry(1, 1, writes_cache=False))
        return ModelSpec(architecture="ToyForCausalLM", hidden_size=self.hidden_size, vocab_size=self.vocab_size,
                         max_position_embeddings=256, embedding_name="embed.weight", layers=tuple(layers),
                         run_order=order, final_norm=norm, final_norm_prefix="final_norm.", lm_head_name=None,
                         position_encodings={"rope": PartSpec("rotary", {"head_dim": 16, "theta": 10000.0, "rotary_dim": ROTARY_DIM}),
                                             "abs": PartSpec("learned_positions", {"hidden_size": self.hidden_size, "max_len": 256})},
                         embedding_hooks=(PartSpec("scale", {"factor": EMBED_SCALE}),),
                         logit_hooks=(PartSpec("softcap", {"cap": SOFTCAP}),))


TOY = {"architectures": ["ToyForCausalLM"], "hidden_size": 24, "state_size": 10, "vocab_size": 50, "num_layers": 2}


@pytest.fixture
def toy_registered():
    MIXERS.register("running_sum", RunningSumMixer)
    FEED_FORWARDS.register("routed_experts", RoutedExperts)
    POSITION_ENCODINGS.register("learned_positions", LearnedPositions)
    BLOCKS.register("sandwich", SandwichBlock)
    HOOKS.register("scale", Scale)
    HOOKS.register("softcap", SoftCap)
    register_architecture("ToyForCausalLM", ToyConfig)
    yield
    BLOCKS.unregister("sandwich")
    HOOKS.unregister("scale")
    HOOKS.unregister("softcap")
    MIXERS.unregister("running_sum")
    FEED_FORWARDS.unregister("routed_experts")
    POSITION_ENCODINGS.unregister("learned_positions")
    unregister_architecture("ToyForCausalLM")


def reference_logits(folder, tokens):
    """The toy model, whole sequence, no cache, written out directly."""
    import plain_impl as P
    from safetensors.torch import load_file
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    T = len(tokens)
    x = (w["embed.weight"][torch.tensor(tokens)] + w["position.abs.weight"][:T]) * EMBED_SCALE
    inv = P.rope_inv_freq(ROTARY_DIM, 10000.0, None)
    kv = {}

    def rope(t):       # only the first ROTARY_DIM elements of each head turn
        return torch.cat([P.apply_rope(t[..., :ROTARY_DIM], range(T), inv), t[..., ROTARY_DIM:]], -1)

    def running_sum(h, p):
        u = h @ w[p + "mixer.in_proj.weight"].t()
        s = torch.zeros(u.shape[1], dtype=torch.float64)
        out = []
        for t in range(T):
            s = DECAY * s + u[t]
            out.append(s)
        return torch.stack(out) @ w[p + "mixer.out_proj.weight"].t()

    def attention(h, p, reuse):
        q = (h @ w[p + "mixer.q_proj.weight"].t()).view(T, 2, 16)
        q = rope(q)
        if not reuse:
            k = rope((h @ w[p + "mixer.k_proj.weight"].t()).view(T, 1, 16))
            v = (h @ w[p + "mixer.v_proj.weight"].t()).view(T, 1, 16)
            kv["k"], kv["v"] = k, v
        o = P.causal_attention(q, kv["k"], kv["v"], 0.25).reshape(T, 32)
        return o @ w[p + "mixer.o_proj.weight"].t()

    for layer, reuse in ((0, False), (1, False), (0, False), (1, True)):
        p = f"layers.{layer}."
        h = P.rms_norm(x, w[p + "norm1.weight"], 1e-5)
        if layer == 0:
            x = x + running_sum(h, p)
        else:              # the block with four norms
            x = x + P.rms_norm(attention(h, p, reuse), w[p + "norm1b.weight"], 1e-5)
        h = P.rms_norm(x, w[p + "norm2.weight"], 1e-5)
        if layer == 0:
            gate = torch.softmax(h @ w[p + "ffn.router.weight"].t() * 8.0, dim=-1)
            for e in range(3):
                x = x + gate[:, e:e + 1] * (torch.relu(h @ w[p + f"ffn.experts.{e}.up.weight"].t()) @ w[p + f"ffn.experts.{e}.down.weight"].t())
        else:
            m = P.gated_mlp(h, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"])
            x = x + P.rms_norm(m, w[p + "norm2b.weight"], 1e-5)
    logits = P.rms_norm(x, w["final_norm.weight"], 1e-5) @ w["embed.weight"].t()
    return torch.tanh(logits / SOFTCAP) * SOFTCAP


def run_toy(tmp_path, device, dtype, tol, graphs=False):
    from rvllm_b200.engine import StepEntry
    from rvllm_b200.engine.trace import build_engine
    folder = write_random_model(config_from_dict(TOY), str(tmp_path / "toy"), seed=2, dtype="float32")
    eng = build_engine(folder, dtype, 3 * 64, block_size=8, device=device, max_live=3, graphs=graphs)
    assert not eng.model.graph_safe                 # because of the state mixer
    assert len(eng.cache.groups) == 1 and sorted(eng.cache._state) == [0, 2]        # two states, one kv group
    g = torch.Generator().manual_seed(0)
    seqs = {r: torch.randint(0, 50, (n,), generator=g).tolist() for r, n in (("a", 30), ("b", 21), ("c", 17), ("d", 26))}
    ref = {r: reference_logits(folder, t) for r, t in seqs.items()}
    got = {r: [] for r in seqs}
    pos = {r: 0 for r in seqs}

    def feed(parts):
        entries = [StepEntry(r, seqs[r][pos[r]:pos[r] + n], list(range(n))) for r, n in parts]
        out = eng.runner.step(entries).cpu()
        row = 0
        for r, n in parts:
            got[r].append(out[row:row + n])
            row += n
            pos[r] += n

    feed([("a", 7)])
    feed([("a", 2), ("b", 11)])                     # a portion beside another request's portion
    feed([("a", 1), ("b", 1), ("c", 17)])           # decoded tokens beside a whole prompt
    while pos["a"] < 30 or pos["b"] < 21:
        feed([(r, 1) for r in ("a", "b") if pos[r] < len(seqs[r])])
    eng.runner.finish("a")
    eng.runner.finish("b")
    feed([("d", 5)])                                # d takes a state slot that a or b held: it starts from zero
    feed([("d", 21)])
    for r in seqs:
        full = torch.cat(got[r]).double()
        err = float((full - ref[r]).abs().max() / ref[r].abs().max())
        assert err < tol, f"request {r}: {err:.2e}"
    eng.cache.check()
    assert not eng.runner._graphs                   # no step of this model was captured
    return eng


def test_toy_state_mixer_on_cpu_with_emulated_kernels(tmp_path, toy_registered):
    from emulated_kernels import EmulatedKernels
    kernel_pkg.set_library(EmulatedKernels())
    try:
        run_toy(tmp_path, "cpu", "float32", 1e-5)
    finally:
        kernel_pkg.set_library(None)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_toy_state_mixer_on_gpu(tmp_path, toy_registered, dtype, tol):
    run_toy(tmp_path, "cuda:0", dtype, tol)


@pytest.mark.gpu
def test_a_part_that_cannot_be_captured_keeps_the_model_out_of_cuda_graphs(tmp_path, toy_registered):
    """With graphs switched on, the toy's decode steps (which call .tolist() inside the state
    mixer) still run, eagerly, and give the same logits; a model of the framework's own parts is
    captured as before."""
    eng = run_toy(tmp_path, "cuda:0", "float32", 1e-4, graphs=True)
    assert eng.runner.graph_batch_sizes and eng.runner.capture_decode_graphs() == 0
    from model_tools import model_folder
    from rvllm_b200.engine.trace import build_engine
    plain = build_engine(model_folder("tiny_llama"), "float32", 128, graphs=True)
    assert plain.model.graph_safe and plain.runner.capture_decode_graphs(batch_sizes=(1,)) > 0


def test_the_toy_s_spec_is_checked(toy_registered):
    """Named parts: an unknown family, two mixers in a layer and roles a block does not know are
    refused with a message."""
    from rvllm_b200 import ConfigError
    from rvllm_b200.models import DecoderModel
    spec = config_from_dict(TOY).to_spec()
    layer = spec.layers[1]
    import dataclasses
    two = dataclasses.replace(layer, parts={**layer.parts, "second": layer.parts["mixer"]})
    with pytest.raises(ConfigError, match="more than one mixer"):
        DecoderModel(dataclasses.replace(spec, layers=(spec.layers[0], two)))
    odd = dataclasses.replace(layer, parts={**layer.parts, "mixer": PartSpec("paged_attention", layer.parts["mixer"].params, "gizmo")})
    with pytest.raises(ConfigError, match="family 'gizmo'"):
        DecoderModel(dataclasses.replace(spec, layers=(spec.layers[0], odd)))
    wrong = dataclasses.replace(spec.layers[0], parts={k: v for k, v in spec.layers[0].parts.items() if k != "mixer_norm"})
    with pytest.raises(ConfigError, match="arranges the parts"):
        DecoderModel(dataclasses.replace(spec, layers=(wrong, spec.layers[1])))
