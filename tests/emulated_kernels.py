"""Stand-ins for the CUDA kernels, written with torch on the CPU, for tests of the host side.

The product path has no CPU implementation.  These functions exist only so that the tests that
run without a GPU can drive the real step function, cache manager, scheduler and trace replay
and check their bookkeeping (paging, block tables, slot mapping, portions, page reuse) against
the plain implementation.  Each method restates what the kernel of the same name must do; the
GPU tests compare the kernels themselves with their plain references.
"""
from __future__ import annotations

import math

import torch


class EmulatedKernels:
    def gather_rows(self, table, ids):
        return table[ids.long()].clone()

    def late_tokens(self, token_ids, cu_seqlens, source, sampled):
        for i, j in enumerate(source.tolist()):
            if j >= 0:
                token_ids[int(cu_seqlens[i])] = sampled[j]

    def rmsnorm(self, x, gamma, eps):
        xf = x.float()
        r = 1.0 / torch.sqrt((xf * xf).mean(-1, keepdim=True) + eps)
        return (xf * r * gamma.float()).to(x.dtype)

    def silu_mul(self, gate_up):
        inter = gate_up.shape[1] // 2
        g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
        return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)

    def rope_cache_write(self, qkv, bias, positions, cos, sin, slot_mapping, cache_layer,
                         num_heads, num_kv_heads, head_dim, write_kv=True, out_dtype=None):
        out_dtype = out_dtype or qkv.dtype
        T = qkv.shape[0]
        x = qkv.float()
        if bias is not None:
            x = x + bias.float()
        pos = positions.long()

        def rot(t):   # [T, heads, hd]; the tables' width says how much of a head is rotated
            if cos is None:
                return t
            half = cos.shape[1]
            c, s = cos[pos][:, None, :], sin[pos][:, None, :]
            a, b, rest = t[..., :half], t[..., half:2 * half], t[..., 2 * half:]
            return torch.cat([a * c - b * s, a * s + b * c, rest], -1)

        q_dim, kv_dim = num_heads * head_dim, num_kv_heads * head_dim
        q = rot(x[:, :q_dim].view(T, num_heads, head_dim))
        if write_kv:
            k = rot(x[:, q_dim:q_dim + kv_dim].view(T, num_kv_heads, head_dim)).to(out_dtype)
            v = x[:, q_dim + kv_dim:].view(T, num_kv_heads, head_dim).to(out_dtype)
            ps = cache_layer.shape[3]
            for t in range(T):
                slot = int(slot_mapping[t])
                if slot < 0:
                    continue
                cache_layer[slot // ps, 0, :, slot % ps, :] = k[t]
                cache_layer[slot // ps, 1, :, slot % ps, :] = v[t]
        return q.reshape(T, q_dim).to(out_dtype)

    def qkv_rope_cache_write(self, x, weight, bias, positions, cos, sin, slot_mapping, cache_layer,
                             num_heads, num_kv_heads, head_dim, norm=None):
        return self.rope_cache_write(self.linear(x, weight, norm=norm), bias, positions, cos, sin, slot_mapping, cache_layer,
                                     num_heads, num_kv_heads, head_dim)

    def paged_attention(self, q, cache_layer, meta, num_heads, num_kv_heads, head_dim, scale, window):
        T = q.shape[0]
        ps = cache_layer.shape[3]
        out = torch.zeros_like(q).view(T, num_heads, head_dim)
        qv = q.view(T, num_heads, head_dim).float()
        cu = meta.cu_seqlens.tolist()
        for s in range(meta.num_seqs):
            ctx = int(meta.ctx_lens[s])
            if ctx <= 0:
                continue
            q_len = cu[s + 1] - cu[s]
            table = meta.block_tables[s].tolist()
            for i in range(q_len):
                t = cu[s] + i
                pos = ctx - q_len + i
                lo = max(0, pos - window + 1) if window else 0
                keys = list(range(lo, pos + 1))
                pages = [table[j // ps] for j in keys]
                assert all(p >= 0 for p in pages), "attention reads a page that was given back"
                offs = [j % ps for j in keys]
                for h in range(num_heads):
                    g = h * num_kv_heads // num_heads
                    K = cache_layer[pages, 0, g, offs, :].float()
                    V = cache_layer[pages, 1, g, offs, :].float()
                    p = torch.softmax((K @ qv[t, h]) * scale, 0)
                    out[t, h] = (p @ V).to(q.dtype)
        return out.view(T, num_heads * head_dim)

    def linear(self, x, weight, bias=None, residual=None, out_dtype=None, norm=None):
        if norm is not None:
            x = self.rmsnorm(x, *norm)
        y = x.float() @ weight.float().t()
        if bias is not None:
            y = y + bias.float()
        if residual is not None:
            y = y + residual.float()
        return y.to(out_dtype or x.dtype)

    def gate_up_silu(self, x, weight, norm=None):
        return self.silu_mul(self.linear(x, weight, norm=norm))

    def sample(self, logits, temperature=None, top_k=None, top_p=None, seeds=None, draw_index=None):
        from plain_impl import sample as plain_sample
        out = []
        for r in range(logits.shape[0]):
            T = float(temperature[r]) if temperature is not None else 0.0
            k = int(top_k[r]) if top_k is not None else 0
            p = float(top_p[r]) if top_p is not None else 1.0
            tok, _ = plain_sample(logits[r], T, int(seeds[r]) if seeds is not None else 0,
                                  int(draw_index[r]) if draw_index is not None else 0, k, p)
            out.append(tok)
        return torch.tensor(out, dtype=torch.int32)
