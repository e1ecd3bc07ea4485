"""Toy parts defined here - a mixer with state of its own, a feed-forward with a router, a position
encoding added to the embeddings - are registered, built into a model through a toy architecture,
loaded from a random-weights folder and stepped - prompts cut into portions, decoding, several
live requests, slots used again - without touching the framework's files.

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
from rvllm_b200.parts import FEED_FORWARDS, MIXERS, POSITION_ENCODINGS, Part, StateNeed, TensorSpec

DECAY = 0.9


class RunningSumMixer(Part):
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
            layers.append(LayerSpec(prefix=f"layers.{i}.", block=PartSpec("prenorm_residual"), mixer=mixer,
                                    feed_forward=ffn,
                                    mixer_norm=norm, feed_forward_norm=norm,
                                    names={"mixer": "mixer.", "feed_forward": "ffn.", "mixer_norm": "norm1.", "feed_forward_norm": "norm2."}))
        # the run order names layer 0 twice (its second run has a state of its own) and lets the
        # last entry read the keys and values that layer 1 wrote
        order = (RunEntry(0, 0), RunEntry(1, 1), RunEntry(0, 2), RunEntry(1, 1, writes_cache=False))
        return ModelSpec(architecture="ToyForCausalLM", hidden_size=self.hidden_size, vocab_size=self.vocab_size,
                         max_position_embeddings=256, embedding_name="embed.weight", layers=tuple(layers),
                         run_order=order, final_norm=norm, final_norm_prefix="final_norm.", lm_head_name=None,
                         position_encodings={"rope": PartSpec("rotary", {"head_dim": 16, "theta": 10000.0}),
                                             "abs": PartSpec("learned_positions", {"hidden_size": self.hidden_size, "max_len": 256})})


TOY = {"architectures": ["ToyForCausalLM"], "hidden_size": 24, "state_size": 10, "vocab_size": 50, "num_layers": 2}


@pytest.fixture
def toy_registered():
    MIXERS.register("running_sum", RunningSumMixer)
    FEED_FORWARDS.register("routed_experts", RoutedExperts)
    POSITION_ENCODINGS.register("learned_positions", LearnedPositions)
    register_architecture("ToyForCausalLM", ToyConfig)
    yield
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
    x = w["embed.weight"][torch.tensor(tokens)] + w["position.abs.weight"][:T]
    inv = P.rope_inv_freq(16, 10000.0, None)
    kv = {}

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
        q = P.apply_rope(q, range(T), inv)
        if not reuse:
            k = P.apply_rope((h @ w[p + "mixer.k_proj.weight"].t()).view(T, 1, 16), range(T), inv)
            v = (h @ w[p + "mixer.v_proj.weight"].t()).view(T, 1, 16)
            kv["k"], kv["v"] = k, v
        o = P.causal_attention(q, kv["k"], kv["v"], 0.25).reshape(T, 32)
        return o @ w[p + "mixer.o_proj.weight"].t()

    for layer, reuse in ((0, False), (1, False), (0, False), (1, True)):
        p = f"layers.{layer}."
        h = P.rms_norm(x, w[p + "norm1.weight"], 1e-5)
        x = x + (running_sum(h, p) if layer == 0 else attention(h, p, reuse))
        h = P.rms_norm(x, w[p + "norm2.weight"], 1e-5)
        if layer == 0:
            gate = torch.softmax(h @ w[p + "ffn.router.weight"].t() * 8.0, dim=-1)
            for e in range(3):
                x = x + gate[:, e:e + 1] * (torch.relu(h @ w[p + f"ffn.experts.{e}.up.weight"].t()) @ w[p + f"ffn.experts.{e}.down.weight"].t())
        else:
            x = x + P.gated_mlp(h, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"])
    return P.rms_norm(x, w["final_norm.weight"], 1e-5) @ w["embed.weight"].t()


def run_toy(tmp_path, device, dtype, tol):
    from rvllm_b200.engine import StepEntry
    from rvllm_b200.engine.trace import build_engine
    folder = write_random_model(config_from_dict(TOY), str(tmp_path / "toy"), seed=2, dtype="float32")
    eng = build_engine(folder, dtype, 3 * 64, block_size=8, device=device, max_live=3)
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
