"""rv_flash_attention_static, the attention entry point for callers that cannot allocate.

Some users of the kernel library load the shared object straight from a host program that owns
all device memory, or call it where cudaMalloc is off limits; they cannot hand the split-key
attention its scratch buffer.  This entry point keeps the scratch in a fixed array inside the
library.  The test calls it the way such a caller would - through the exported C symbol, with raw
pointers, no wrapper - twice in a row on different inputs (the array keeps the first call's
contents, which must not leak into the second), and compares with the ordinary entry point, which
gets a scratch buffer from the caller.  It also checks that a call too large for the array is
refused with a message.  This file sorts last, so a run that stops at the first failure has
already run everything else; it passes alone in a fresh process as well.
"""
import ctypes
import math
from ctypes import c_char_p, c_float, c_int, c_void_p

import pytest
import torch

from gpu_tools import paged_setup

pytestmark = pytest.mark.gpu

HD = 64
STATIC_FLOATS = 1 << 20


def ptr(t):
    return c_void_p(t.data_ptr() if t is not None else 0)


def call_static(lib, q, cache, meta, out, nh, nkv, scale, window, splits, err, mode=1):
    return lib.rv_flash_attention_static(
        ptr(q), ptr(cache), ptr(meta.block_tables), ptr(meta.cu_seqlens), ptr(meta.ctx_lens), ptr(out),
        c_int(q.shape[0]), c_int(meta.num_seqs), c_int(nh), c_int(nkv), c_int(HD), c_int(cache.shape[3]),
        c_int(meta.max_blocks), c_float(scale), c_int(window), c_int(mode), c_int(meta.max_q_len), c_int(splits),
        c_void_p(torch.cuda.current_stream().cuda_stream), err, c_int(len(err)))


def call_ordinary(lib, q, cache, meta, out, scratch, nh, nkv, scale, window, splits, mode=1):
    return lib.rv_flash_attention(
        ptr(q), ptr(cache), ptr(meta.block_tables), ptr(meta.cu_seqlens), ptr(meta.ctx_lens), ptr(out), ptr(scratch),
        c_int(q.shape[0]), c_int(meta.num_seqs), c_int(nh), c_int(nkv), c_int(HD), c_int(cache.shape[3]),
        c_int(meta.max_blocks), c_float(scale), c_int(window), c_int(mode), c_int(meta.max_q_len), c_int(splits), c_int(0),
        c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from rvllm_b200.kernels import build
    lib = build.load_library("attention_flash.cu", (f"-DHEAD_DIM={HD}",))
    lib.rv_flash_scratch_floats.restype = ctypes.c_longlong
    nh, nkv, page = 8, 2, 16
    scale = 1 / math.sqrt(HD)
    err = ctypes.create_string_buffer(256)
    for call, (ctx_lens, splits, window, seed) in enumerate([((700, 64, 1, 333), 6, 0, 1), ((90, 1000, 257), 4, 128, 2)]):
        torch.manual_seed(seed)
        ks = [torch.randn(c, nkv, HD) for c in ctx_lens]
        vs = [torch.randn(c, nkv, HD) for c in ctx_lens]
        B = len(ctx_lens)
        cache, meta = paged_setup(ks, vs, [1] * B, page, torch.bfloat16, seed=seed)
        q = torch.randn(B, nh * HD, device="cuda").bfloat16()
        need = lib.rv_flash_scratch_floats(c_int(B), c_int(nh), c_int(splits))
        assert 0 < need <= STATIC_FLOATS
        scratch = torch.empty(need, dtype=torch.float32, device="cuda")
        want = torch.zeros_like(q)
        assert call_ordinary(lib, q, cache, meta, want, scratch, nh, nkv, scale, window, splits) == 0
        got = torch.zeros_like(q)
        assert call_static(lib, q, cache, meta, got, nh, nkv, scale, window, splits, err) == 0, err.value.decode()
        torch.cuda.synchronize()
        assert err.value == b""
        assert torch.isfinite(got.float()).all()
        diff = float((got.float() - want.float()).abs().max())
        assert diff <= 1e-2 * float(want.float().abs().max()), f"call {call}: differs by {diff}"
        # and against the plain kernel, so that both being wrong together would show
        from rvllm_b200.kernels import get_library
        plain = get_library("cuda:0").paged_attention_plain(q, cache, meta, nh, nkv, HD, scale, window or None)
        assert float((got.float() - plain.float()).abs().max()) <= 1e-2 * float(plain.float().abs().max())


def test_static_scratch_entry_point_with_the_prefill_tiling():
    """The header offers both tilings: here prompt portions of several tokens (mode 0, 64 rows per
    CTA), their keys split over three CTAs, again twice in a row on different inputs."""
    from rvllm_b200.kernels import build, get_library
    lib = build.load_library("attention_flash.cu", (f"-DHEAD_DIM={HD}",))
    lib.rv_flash_scratch_floats.restype = ctypes.c_longlong
    nh, nkv, page, splits = 8, 2, 16, 3
    scale = 1 / math.sqrt(HD)
    err = ctypes.create_string_buffer(256)
    for call, (q_lens, ctx_lens, window, seed) in enumerate([((40, 7), (100, 300), 0, 5), ((3, 64, 20), (500, 64, 129), 96, 6)]):
        torch.manual_seed(seed)
        ks = [torch.randn(c, nkv, HD) for c in ctx_lens]
        vs = [torch.randn(c, nkv, HD) for c in ctx_lens]
        cache, meta = paged_setup(ks, vs, list(q_lens), page, torch.bfloat16, seed=seed)
        T = sum(q_lens)
        q = torch.randn(T, nh * HD, device="cuda").bfloat16()
        need = lib.rv_flash_scratch_floats(c_int(T), c_int(nh), c_int(splits))
        assert 0 < need <= STATIC_FLOATS
        scratch = torch.empty(need, dtype=torch.float32, device="cuda")
        want = torch.zeros_like(q)
        assert call_ordinary(lib, q, cache, meta, want, scratch, nh, nkv, scale, window, splits, mode=0) == 0
        got = torch.zeros_like(q)
        assert call_static(lib, q, cache, meta, got, nh, nkv, scale, window, splits, err, mode=0) == 0, err.value.decode()
        torch.cuda.synchronize()
        assert err.value == b"" and torch.isfinite(got.float()).all()
        assert float((got.float() - want.float()).abs().max()) <= 1e-2 * float(want.float().abs().max()), f"call {call}"
        plain = get_library("cuda:0").paged_attention_plain(q, cache, meta, nh, nkv, HD, scale, window or None)
        assert float((got.float() - plain.float()).abs().max()) <= 1e-2 * float(plain.float().abs().max())


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from rvllm_b200.kernels import build
    lib = build.load_library("attention_flash.cu", (f"-DHEAD_DIM={HD}",))
    nh, nkv, page, B, splits = 64, 8, 16, 64, 8          # 8 * 64 * 64 * 66 floats > 2^20
    ks = [torch.randn(40, nkv, HD) for _ in range(B)]
    cache, meta = paged_setup(ks, ks, [1] * B, page, torch.bfloat16)
    q = torch.randn(B, nh * HD, device="cuda").bfloat16()
    out = torch.full_like(q, 7.0)
    err = ctypes.create_string_buffer(256)
    st = call_static(lib, q, cache, meta, out, nh, nkv, 0.125, 0, splits, err)
    torch.cuda.synchronize()
    assert st == -5
    msg = err.value.decode()
    assert "needs" in msg and str(1 << 20) in msg and "scratch" in msg
    assert float((out.float() - 7.0).abs().max()) == 0.0   # nothing ran
    # without splits no scratch is needed, whatever the batch
    assert call_static(lib, q, cache, meta, out, nh, nkv, 0.125, 0, 1, err) == 0
    torch.cuda.synchronize()
