"""Plain, slow implementation of the Llama / Qwen2 dense decoder, used as the oracle.

Whole sequences only, no cache, no batching, one function per part, torch used
purely as an array library (float64; on the CPU, or, for the models of real layer widths whose
float64 products would take minutes there, on the device the weights were read to).  It shares no code with the engine under
``rvllm_b200``: it reads config.json with ``json`` and model.safetensors with the
``safetensors`` package, and restates every formula from the reference's files
(paths are relative to the reference project's root).

This oracle rests on the formulas only: the reference's own oracles are Rust
(v3/crates/rvllm-fused/src/reference.rs) and its array ports import jax; neither
toolchain can be compiled or imported here, so no golden vectors were produced by
running reference code.

Where the reference contradicts itself, the convention of the checkpoints it loads
wins: rotary pairs are (i, i + head_dim/2) as in its f32 oracle
(rvllm-fused/src/reference.rs:177-203), not the interleaved pairs of its CUDA
kernel (v3/kernels/fused_rope_cache_fp8kv.cu:53-69).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

DEFAULT_DTYPE = torch.float64


# --------------------------------------------------------------------------- model folder

def read_model_folder(path: str, dtype=DEFAULT_DTYPE, device="cpu"):
    """config.json as a dict and every tensor of model.safetensors converted to `dtype` on `device`."""
    from safetensors.torch import load_file

    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    raw = load_file(os.path.join(path, "model.safetensors"))
    weights = {k: v.to(device=device, dtype=dtype) for k, v in raw.items()}
    return cfg, weights


# --------------------------------------------------------------------------- parts

def embedding(ids: Sequence[int], table: torch.Tensor) -> torch.Tensor:
    """out[t, :] = E[id[t], :], a pure copy without scaling.

    kernels/embedding_gather_f16.cu:12-39; oracle rvllm-fused/src/reference.rs:157-172
    (which asserts id < vocab; so do we).
    """
    ids = list(ids)
    assert all(0 <= i < table.shape[0] for i in ids), "token id out of vocabulary"
    return table[torch.tensor(ids, dtype=torch.long, device=table.device)]


def rms_norm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    """y_i = x_i / sqrt(mean(x^2) + eps) * gamma_i, plain gamma (no 1 + gamma).

    rvllm-fused/src/reference.rs:12-24; kernels/fused_rmsnorm_fp8_quant.cu:61-84.
    """
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(ms + eps)) * gamma


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T (+ b) with W stored [out, in] as in the checkpoints.

    v3/crates/rvllm-cutlass/src/cublaslt.rs:375-606 (D = A B^T, f32 accumulate);
    bias is a row broadcast (kernels/add_bias_f16.cu:27-30).
    """
    y = x @ w.t()
    if b is not None:
        y = y + b
    return y


def rope_inv_freq(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """inv_freq_i = theta^(-2i/head_dim), i in [0, head_dim/2), in float64.

    rvllm-loader/src/load.rs:876-891.  The reference never reads `rope_scaling`;
    the llama3 rule below is the published one the Llama-3.1 checkpoints are made
    for: wavelengths shorter than orig/high are kept, longer than orig/low are
    divided by `factor`, and the band between is blended linearly.
    """
    half = head_dim // 2
    inv = torch.tensor([theta ** (-2.0 * i / head_dim) for i in range(half)], dtype=torch.float64)
    if scaling is None:
        return inv
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    if kind == "default":
        return inv
    assert kind == "llama3", kind
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = inv.clone()
    for i in range(half):
        wavelen = 2.0 * math.pi / float(inv[i])
        if wavelen < orig / high:
            continue
        if wavelen > orig / low:
            out[i] = inv[i] / factor
        else:
            s = (orig / wavelen - low) / (high - low)
            out[i] = (1.0 - s) * inv[i] / factor + s * inv[i]
    return out


def apply_rope(x: torch.Tensor, positions: Sequence[int], inv_freq: torch.Tensor) -> torch.Tensor:
    """Rotate x [T, heads, head_dim] in pairs (i, i + head_dim/2).

    angle = position * inv_freq_i; x_i' = a cos - b sin, x_{i+half}' = a sin + b cos.
    rvllm-fused/src/reference.rs:177-203.
    """
    half = x.shape[-1] // 2
    pos = torch.tensor(list(positions), dtype=torch.float64, device=x.device)
    # the engine keeps inv_freq as float32; use the same rounded frequencies so that the
    # comparison measures the rotation, not a difference in the table's last bit
    ang = pos[:, None] * inv_freq.to(torch.float32).to(device=x.device, dtype=torch.float64)[None, :]
    cos = torch.cos(ang).to(x.dtype)[:, None, :]
    sin = torch.sin(ang).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: Optional[int] = None, store=None) -> torch.Tensor:
    """GQA attention over one whole sequence.  q [T, nh, hd], k/v [T, nkv, hd].

    kv_head = h * nkv / nh; score = (q . k) * scale; query t sees keys j <= t and,
    with a window of W keys, j > t - W.  Softmax and the weighted sum run in the
    array's own precision.
    v3/kernels/paged_attention_sm89.cu:241-369 (causal rule :277-287, window :300-308
    where window_size_left + 1 keys are kept).
    """
    T, nh, hd = q.shape
    nkv = k.shape[1]
    out = torch.zeros_like(q)
    t_idx = torch.arange(T, device=q.device)
    allowed = t_idx[None, :] <= t_idx[:, None]
    if window is not None:
        allowed = allowed & (t_idx[None, :] > t_idx[:, None] - window)
    for h in range(nh):
        g = h * nkv // nh
        s = (q[:, h, :] @ k[:, g, :].t()) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        p = torch.softmax(s, dim=-1)
        if store is not None:
            # a tensor-core attention multiplies probabilities as 16-bit operands: exp(s - max) is
            # rounded (the row's sum is not), which is the same as rounding p up to the common factor
            e = torch.exp(s - s.amax(dim=-1, keepdim=True))
            p = store(e) / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, g, :]
    return out


def gated_mlp(x: torch.Tensor, w_gate, w_up, w_down) -> torch.Tensor:
    """down( silu(gate(x)) * up(x) ), silu(g) = g / (1 + exp(-g)).

    kernels/fused_silu_fp8_quant.cu:52-56,74-78; rvllm-fused/src/reference.rs:76-100;
    v3/crates/rvllm-runtime/src/layer_exec.rs:476-522.
    """
    g = linear(x, w_gate)
    u = linear(x, w_up)
    h = g / (1.0 + torch.exp(-g)) * u
    return linear(h, w_down)


# --------------------------------------------------------------------------- configuration

def layer_windows(cfg: dict) -> List[Optional[int]]:
    """Per layer: None for full attention, W for a window of W keys (the query included).

    `layer_types` names each layer (rvllm-loader/src/load.rs:122-135); without it a
    Qwen2 configuration with use_sliding_window puts the window on layers from
    max_window_layers upward.  Llama has no window.
    """
    L = cfg["num_hidden_layers"]
    w = cfg.get("sliding_window")
    if cfg["architectures"][0] == "Qwen2ForCausalLM" and not cfg.get("use_sliding_window", False):
        w = None
    if cfg["architectures"][0] == "LlamaForCausalLM":
        w = None
    types = cfg.get("layer_types")
    if types is None:
        start = cfg.get("max_window_layers", L)
        types = ["sliding_attention" if (w is not None and i >= start) else "full_attention"
                 for i in range(L)]
    return [w if t == "sliding_attention" else None for t in types]


def has_qkv_bias(cfg: dict) -> bool:
    """Llama: `attention_bias` (default false, load.rs:120).  Qwen2: always on q, k, v."""
    if cfg["architectures"][0] == "Qwen2ForCausalLM":
        return True
    return bool(cfg.get("attention_bias", False))


def has_out_bias(cfg: dict) -> bool:
    """A Llama checkpoint with `attention_bias` carries a bias on o_proj as well; Qwen2 never does."""
    return cfg["architectures"][0] == "LlamaForCausalLM" and bool(cfg.get("attention_bias", False))


# --------------------------------------------------------------------------- whole model

def _keep(t):
    return t


def decoder_layer(x, positions, cfg, w: Dict[str, torch.Tensor], prefix: str, inv_freq, window, store=_keep):
    """x + attn(norm(x)), then + mlp(norm(.)) — v3/crates/rvllm-runtime/src/layer_exec.rs:162-529.

    `store` is applied to every tensor that an engine would write to memory between two kernels
    (default: nothing); with a rounding to bfloat16 it shows how much error that precision alone
    causes, whatever the kernels (see `forward`)."""
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    eps = cfg["rms_norm_eps"]
    bias = has_qkv_bias(cfg)
    T = x.shape[0]

    a = store(rms_norm(x, w[prefix + "input_layernorm.weight"], eps))
    sa = prefix + "self_attn."
    q = linear(a, w[sa + "q_proj.weight"], w[sa + "q_proj.bias"] if bias else None).view(T, nh, hd)
    k = linear(a, w[sa + "k_proj.weight"], w[sa + "k_proj.bias"] if bias else None).view(T, nkv, hd)
    v = store(linear(a, w[sa + "v_proj.weight"], w[sa + "v_proj.bias"] if bias else None).view(T, nkv, hd))
    q = store(apply_rope(q, positions, inv_freq))
    k = store(apply_rope(k, positions, inv_freq))
    o = store(causal_attention(q, k, v, 1.0 / math.sqrt(hd), window, None if store is _keep else store).reshape(T, nh * hd))
    x = store(x + linear(o, w[sa + "o_proj.weight"], w[sa + "o_proj.bias"] if has_out_bias(cfg) else None))

    m = store(rms_norm(x, w[prefix + "post_attention_layernorm.weight"], eps))
    mp = prefix + "mlp."
    if store is _keep:
        return x + gated_mlp(m, w[mp + "gate_proj.weight"], w[mp + "up_proj.weight"], w[mp + "down_proj.weight"])
    g, u = linear(m, w[mp + "gate_proj.weight"]), linear(m, w[mp + "up_proj.weight"])
    h = store(g / (1.0 + torch.exp(-g)) * u)
    return store(x + linear(h, w[mp + "down_proj.weight"]))


def round_to_bfloat16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(t.dtype)


def forward(cfg: dict, w: Dict[str, torch.Tensor], token_ids: Sequence[int], store=_keep) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence starting at position 0.

    Skeleton: v3/crates/rvllm-runtime/src/bring_up.rs:535-669; the LM head is the
    embedding matrix when `tie_word_embeddings` (rvllm-loader/src/load.rs:310-311,351-363).

    With `store=round_to_bfloat16` every tensor that passes between two parts is rounded to
    bfloat16 while all arithmetic stays float64: the difference to the plain logits is the error
    that storing activations in that precision causes by itself, the yardstick for a bfloat16 engine.
    """
    nh = cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    inv_freq = rope_inv_freq(hd, float(cfg.get("rope_theta", 10000.0)), cfg.get("rope_scaling"))
    windows = layer_windows(cfg)
    positions = list(range(len(token_ids)))
    x = embedding(token_ids, w["model.embed_tokens.weight"])
    for l in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, positions, cfg, w, f"model.layers.{l}.", inv_freq, windows[l], store)
    y = store(rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(y, head)


# --------------------------------------------------------------------------- sampling

def argmax_lowest(logits: torch.Tensor) -> int:
    """Index of the largest value; the lowest index wins ties (reference.rs:131-146)."""
    best, best_v = 0, float(logits[0])
    for j in range(1, logits.shape[0]):
        vj = float(logits[j])
        if vj > best_v:
            best, best_v = j, vj
    return best


_PHILOX_M0, _PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32(counter: Sequence[int], key: Sequence[int], rounds: int = 10) -> List[int]:
    """The published Philox-4x32 block function (Salmon et al., 2011), on Python integers."""
    c = [int(v) & 0xFFFFFFFF for v in counter]
    k = [int(v) & 0xFFFFFFFF for v in key]
    for _ in range(rounds):
        p0 = _PHILOX_M0 * c[0]
        p1 = _PHILOX_M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k[1]) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k = [(k[0] + _PHILOX_W0) & 0xFFFFFFFF, (k[1] + _PHILOX_W1) & 0xFFFFFFFF]
    return c


def uniform_for(seed: int, draw_index: int) -> float:
    """The uniform in [0, 1) that belongs to (request seed, index of the output token)."""
    r = philox4x32([draw_index & 0xFFFFFFFF, (draw_index >> 32) & 0xFFFFFFFF, 0, 0],
                   [seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF])
    return (r[0] >> 8) * (1.0 / 16777216.0)


def filtered_probs(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0):
    """softmax(logits / T), then keep the k most likely and the smallest set reaching top_p.

    Parameters as rvllm-sampling/src/params.rs:7-28 (temperature, top_k, top_p, seed).
    Ties at the cut are kept (every token as likely as the last kept one stays in).
    """
    z = logits.to(torch.float64) / temperature
    p = torch.softmax(z - z.max(), dim=-1)
    keep = torch.ones_like(p, dtype=torch.bool)
    if top_k and top_k < p.numel():
        kth = torch.sort(p, descending=True).values[top_k - 1]
        keep &= p >= kth
    if top_p < 1.0:
        sp = torch.sort(p, descending=True).values
        csum = torch.cumsum(sp, 0)
        n = int((csum < top_p).sum().item()) + 1
        keep &= p >= sp[min(n, p.numel()) - 1]
    p = torch.where(keep, p, torch.zeros_like(p))
    return p / p.sum()


def sample(logits: torch.Tensor, temperature: float, seed: int, draw_index: int,
           top_k: int = 0, top_p: float = 1.0):
    """Inverse-CDF draw in vocabulary order.  Returns (token, margin): margin is the distance of
    u from the nearest CDF step, so a test can skip draws that rounding could flip."""
    if temperature == 0.0:
        return argmax_lowest(logits), 1.0
    p = filtered_probs(logits, temperature, top_k, top_p)
    cdf = torch.cumsum(p, 0)
    u = uniform_for(seed, draw_index)
    tok = int((cdf <= u).sum().item())
    tok = min(tok, p.numel() - 1)
    # never return a token of probability zero (u may fall on a flat stretch of the CDF)
    while p[tok] == 0 and tok > 0:
        tok -= 1
    lo = float(cdf[tok - 1]) if tok > 0 else 0.0
    hi = float(cdf[tok])
    return tok, min(u - lo, hi - u)


def greedy_generate(cfg, w, prompt: Sequence[int], n_new: int) -> List[int]:
    """Greedy continuation by running the whole sequence again for every new token."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(cfg, w, ids)
        t = argmax_lowest(logits[-1])
        out.append(t)
        ids.append(t)
    return out
