"""The kernels of the product path, as methods that take torch tensors.

`CudaKernels` launches the hand-written sm_100a kernels of csrc/ on torch's current stream
through their exported C launchers.  bfloat16 matrix products with at least `TCGEN05_MIN_ROWS` rows
run on this project's tcgen05 / TMEM / TMA kernel (on pairs of CTAs where the rows fill its tiles);
with up to 32 rows, and with up to 64 where K need not be split, on its weight-streaming tcgen05
kernel; what lies between goes to the library GEMM behind `torch` (the reference calls cuBLASLt for
all its linear layers, v3/crates/rvllm-cutlass/src/cublaslt.rs).  Everything else is this project's
own code.  There is no CPU implementation: without a CUDA device, or when a kernel library cannot be
built, construction raises `KernelError`.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_void_p, c_int, c_float
from typing import Optional

import torch

from ..errors import KernelError
from . import build

_DT = {torch.float32: 0, torch.bfloat16: 1}
COUNTERS = {'launches': 0}   # kernels of this project launched so far (library GEMMs are not counted)
_STATUS = {-1: "a size is out of range", -2: "unsupported dtype", -3: "misaligned pointer or stride",
           -4: "size not supported by this kernel"}


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _check(name: str, status: int):
    if status == 0:
        COUNTERS['launches'] += 1
        return
    if status < 0:
        raise KernelError(f"{name}: refused, {_STATUS.get(status, 'code %d' % status)}")
    raise KernelError(f"{name}: CUDA launch failed with error {status}")


def _need(t: torch.Tensor, name: str, dtype=None, dims=None):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous, got strides {t.stride()} for shape {tuple(t.shape)}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, got shape {tuple(t.shape)}")


class AttentionMeta:
    """Per-step, per-cache-group arguments of the attention kernels (device int32 tensors) and
    the few host-side numbers that size their launches."""
    __slots__ = ("block_tables", "cu_seqlens", "ctx_lens", "token_seq", "slot_mapping", "num_seqs",
                 "max_q_len", "max_ctx_len", "max_blocks", "page_size", "num_decode")

    def __init__(self, block_tables, cu_seqlens, ctx_lens, token_seq, slot_mapping, num_seqs,
                 max_q_len, max_ctx_len, page_size, num_decode=0):
        self.num_decode = num_decode       # sequences that bring exactly one token
        self.block_tables, self.cu_seqlens, self.ctx_lens = block_tables, cu_seqlens, ctx_lens
        self.token_seq, self.slot_mapping = token_seq, slot_mapping
        self.num_seqs, self.max_q_len, self.max_ctx_len = num_seqs, max_q_len, max_ctx_len
        self.max_blocks = block_tables.shape[1]
        self.page_size = page_size


class CudaKernels:
    TCGEN05_MIN_ROWS = 128  # rows from which the tcgen05 GEMM of this project is used for bfloat16 ...
    TCGEN05_MIN_FILL = 0.0  # ... where its tiles keep its persistent workers busy for this share of their rounds
                            # (0: always.  With 0.8 the library's GEMM takes the partly filled shapes and is 20-140 %
                            # faster there, but its sums depend on the operands' addresses: the same request no longer
                            # gives the same bits in every run)
    PREFILL_SPLIT_MIN_KB = 32          # ... k blocks that a part keeps at least
    PREFILL_SPLIT_K = True             # ... or, where 2 or 4 CTAs per tile still fit the SMs, with K cut over a cluster of CTAs per tile
    NARROW_TILES = True                # ... with tiles of 128 columns where those of 256 would occupy at most half of the SMs
    PAIR_GEMM = True                   # the tcgen05 GEMM runs on pairs of CTAs (cta_group::2) where the rows fill its 256-row tiles
    TCGEN05_ATTENTION = True           # prompt portions go to the tcgen05 attention kernel when it fits
    TCGEN05_ATTENTION_MIN_TOKENS = 16  # ... from this many tokens in the longest portion of the step
    DECODE_MAX_ROWS = 64    # rows up to which the weight-streaming tcgen05 GEMM may be used
    DECODE_SPLIT_ROWS = 8   # ... when K has to be split over CTAs, only up to this many rows
    DECODE_BLOCK_MAX_ROWS = 256   # ... and, in blocks of 128 rows, for products of up to this many rows whose 128-feature
                                  # tiles x row blocks do not fill the SMs (q/k/v, o, down of a short prompt: the 256-row
                                  # tiles of the prefill GEMM would keep a fraction of the GPU busy)
    CLUSTER_REDUCE = True        # split-K partials of few rows are added up inside a thread-block cluster
    DECODE_K_ROTATE = 13         # tile t of a decode GEMM starts its K loop at block (t * this) mod its count, so that the CTAs of a
                                 # wave do not all read the same columns of the weights at a time (0: all start at the first block)
    DECODE_L2_AHEAD = 6          # k blocks of weights, beyond its stages, that a decode GEMM's CTA asks into L2 before its wait
    CLUSTER_MAX_ROWS = 64        # ... of up to this many rows (the whole range of the weight-streaming GEMM)
    CLUSTER_TARGET_CTAS = 225    # of such a product, tiles x splits (measured best at 8B, 7B and 32B layer sizes)
    TMA_DECODE = True       # decode attention's tiles come by TMA (head sizes 64 / 128, pages of 8 keys or more) ...
    TMA_DECODE_EARLY = True   # ... and keys older than the step's own are requested before the wait for the kernel before
    BALANCED_DECODE = True  # decode attention by the kernel that cuts all tiles evenly over resident CTAs ...
    BALANCED_MIN_PAIRS = 256  # ... from this many (sequence, kv head) pairs on
    FUSED_QKV_PREFILL = True  # from TCGEN05_MIN_ROWS rows on the prefill GEMM rotates and writes the cache in its epilogue
    FUSED_NORM_MAX_ROWS = 0 # rows up to which an RMSNorm is applied inside the decode GEMM that consumes it
    FUSED_QKV_MAX_ROWS = 64 # rows up to which q/k/v product, rotation and cache write are one kernel
    pdl = os.environ.get("RVLLM_NO_PDL") != "1"   # programmatic dependent launch between kernels
    num_sms = 148           # SMs of the device; asked from the device when the library is made

    def __init__(self, device="cuda:0"):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine has no CPU path")
        self.device = torch.device(device)
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(f"the kernels are built for sm_100a; device {device} has compute capability {major}.{minor}")
        # the float32 path must never round operands to TF32 inside a library product
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._libs = {}
        self._decode_counters = None
        # one status word for every tcgen05 launch of the engine: a kernel whose bounded wait on an
        # mbarrier gave up writes a non-zero code here instead of hanging (see `raise_on_abort`)
        self._status = torch.zeros((1,), dtype=torch.int32, device=self.device)

    # ------------------------------------------------------------------ plumbing
    def _lib(self, source: str, defines=()):
        key = (source, tuple(defines))
        lib = self._libs.get(key)
        if lib is None:
            lib = build.load_library(source, defines)
            lib.rv_set_pdl(c_int(1 if self.pdl else 0))
            if source == "gemm_tcgen05_decode.cu":
                lib.rv_gemm_decode_set_l2_ahead(c_int(self.DECODE_L2_AHEAD if self.pdl else 0))
                lib.rv_gemm_decode_set_k_rotate(c_int(self.DECODE_K_ROTATE))
            self._libs[key] = lib
        return lib

    @staticmethod
    def _stream():
        return c_void_p(torch.cuda.current_stream().cuda_stream)

    @staticmethod
    def _dt(t: torch.Tensor, name: str) -> int:
        try:
            return _DT[t.dtype]
        except KeyError:
            raise KernelError(f"{name}: dtype {t.dtype} is not supported (float32, bfloat16)") from None

    # ------------------------------------------------------------------ aborted kernels
    @property
    def status_word(self) -> torch.Tensor:
        """int32 [1] on the device: 0, or the code of the first bounded wait that gave up in a tcgen05
        kernel launched without a status tensor of the caller's own."""
        return self._status

    def raise_on_abort(self, value: Optional[int] = None) -> None:
        """Raise `KernelError` if a kernel gave up a bounded wait since the last check: what it
        wrote is then not a result.  `value` is the status word as the caller has already read it
        (for instance copied to the host beside a step's sampled ids); None reads it now, which
        waits for the device.  After a non-zero value the word and the arrival counters of the
        split-K products are cleared, so that the next launches start clean (an aborted CTA skips
        its arrival, which would make a later launch take the wrong CTA for the last one)."""
        if value is None:
            value = int(self._status.item())
        if value == 0:
            return
        self._status.zero_()
        if self._decode_counters is not None:
            self._decode_counters.zero_()
        raise KernelError(f"a tcgen05 kernel gave up a bounded wait on an mbarrier (wait number {value} of the kernel's "
                          "source); what that step wrote is not a result")

    # ------------------------------------------------------------------ row kernels
    def gather_rows(self, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """out[t] = table[ids[t]]; ids int32.  Used for the embedding and for picking logit rows."""
        _need(table, "table", dims=2); _need(ids, "ids", torch.int32, 1)
        out = torch.empty((ids.shape[0], table.shape[1]), dtype=table.dtype, device=table.device)
        st = self._lib("elementwise.cu").rv_gather_rows(
            _ptr(table), _ptr(ids), _ptr(out), c_int(ids.shape[0]), c_int(table.shape[1]),
            c_int(table.shape[0]), c_int(self._dt(table, "table")), self._stream())
        _check("gather_rows", st)
        return out

    def fill_normal(self, shape, dtype: torch.dtype, mean: float, std: float, seed: int, stream: int) -> torch.Tensor:
        """A new tensor of N(mean, std) values from the counter-based generator: element i depends
        on (seed, stream, i) only.  The engine's random-weights mode gives every tensor a stream of
        its own (its index among the sorted tensor names)."""
        out = torch.empty(tuple(shape), dtype=dtype, device=self.device)
        st = self._lib("elementwise.cu").rv_fill_normal(
            _ptr(out), ctypes.c_longlong(out.numel()), c_float(mean), c_float(std), ctypes.c_ulonglong(seed & (2 ** 64 - 1)),
            ctypes.c_ulonglong(stream), c_int(self._dt(out, "out")), self._stream())
        _check("fill_normal", st)
        return out

    def late_tokens(self, token_ids: torch.Tensor, cu_seqlens: torch.Tensor, source: torch.Tensor,
                    sampled: torch.Tensor) -> None:
        """token_ids[cu_seqlens[i]] = sampled[source[i]] for every sequence i with source[i] >= 0:
        tokens that the previous step sampled and the host has not read yet."""
        _need(token_ids, "token_ids", torch.int32, 1); _need(cu_seqlens, "cu_seqlens", torch.int32, 1)
        _need(source, "source", torch.int32, 1); _need(sampled, "sampled", torch.int32, 1)
        if cu_seqlens.shape[0] < source.shape[0]:
            raise KernelError(f"late_tokens: {source.shape[0]} sequences but {cu_seqlens.shape[0]} sequence starts")
        st = self._lib("elementwise.cu").rv_late_tokens(_ptr(token_ids), _ptr(cu_seqlens), _ptr(source), _ptr(sampled),
                                                        c_int(source.shape[0]), c_int(sampled.shape[0]), self._stream())
        _check("late_tokens", st)

    def rmsnorm(self, x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
        _need(x, "x", dims=2); _need(gamma, "gamma", dims=1)
        if gamma.shape[0] != x.shape[1]:
            raise KernelError(f"rmsnorm: gamma has {gamma.shape[0]} entries for rows of {x.shape[1]}")
        out = torch.empty_like(x)
        st = self._lib("elementwise.cu").rv_rmsnorm(
            _ptr(x), _ptr(gamma), c_int(self._dt(gamma, "gamma")), _ptr(out), c_int(x.shape[0]),
            c_int(x.shape[1]), c_float(eps), c_int(self._dt(x, "x")), self._stream())
        _check("rmsnorm", st)
        return out

    def silu_mul(self, gate_up: torch.Tensor) -> torch.Tensor:
        """rows [gate | up] -> silu(gate) * up."""
        _need(gate_up, "gate_up", dims=2)
        inter = gate_up.shape[1] // 2
        if inter * 2 != gate_up.shape[1]:
            raise KernelError(f"silu_mul: row width {gate_up.shape[1]} is odd")
        out = torch.empty((gate_up.shape[0], inter), dtype=gate_up.dtype, device=gate_up.device)
        st = self._lib("elementwise.cu").rv_silu_mul(_ptr(gate_up), _ptr(out), c_int(gate_up.shape[0]),
                                                    c_int(inter), c_int(self._dt(gate_up, "gate_up")), self._stream())
        _check("silu_mul", st)
        return out

    def rope_cache_write(self, qkv, bias, positions, cos, sin, slot_mapping, cache_layer,
                         num_heads, num_kv_heads, head_dim, write_kv=True, out_dtype=None) -> torch.Tensor:
        """Add the q/k/v bias, rotate q and k, write k and v into their cache pages, return q
        [T, num_heads * head_dim].  qkv rows are [q | k | v], or q alone when `write_kv` is False.
        cache_layer: [num_pages, 2, num_kv_heads, page_size, head_dim].  `out_dtype` bfloat16 with
        float32 rows: the product stays in float until it has been biased and rotated."""
        _need(qkv, "qkv", dims=2); _need(positions, "positions", torch.int32, 1)
        out_dtype = out_dtype or qkv.dtype
        T = qkv.shape[0]
        width = (num_heads + (2 * num_kv_heads if write_kv else 0)) * head_dim
        if qkv.shape[1] != width:
            raise KernelError(f"rope_cache_write: qkv rows have {qkv.shape[1]} columns, expected {width}")
        if write_kv:
            _need(cache_layer, "cache_layer", out_dtype, 5); _need(slot_mapping, "slot_mapping", torch.int32, 1)
            if tuple(cache_layer.shape[1:3]) != (2, num_kv_heads) or cache_layer.shape[4] != head_dim:
                raise KernelError(f"rope_cache_write: cache layer of shape {tuple(cache_layer.shape)} does not "
                                  f"fit {num_kv_heads} kv heads of {head_dim}")
        rot = head_dim
        if cos is not None:
            _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
            rot = 2 * cos.shape[1]            # the leading `rot` elements of a head are rotated, the rest pass through
            if not 0 < rot <= head_dim or sin.shape != cos.shape:
                raise KernelError(f"rope_cache_write: cos/sin tables must be [rows, rotary_dim/2] with rotary_dim <= "
                                  f"head_dim {head_dim}, got {tuple(cos.shape)} and {tuple(sin.shape)}")
        if bias is not None:
            _need(bias, "bias", dims=1)
        q = torch.empty((T, num_heads * head_dim), dtype=out_dtype, device=qkv.device)
        page = cache_layer.shape[3] if write_kv else 1
        st = self._lib("elementwise.cu").rv_rope_cache_write(
            _ptr(qkv), _ptr(bias), c_int(self._dt(bias, "bias") if bias is not None else 0), _ptr(positions),
            _ptr(cos), _ptr(sin), _ptr(slot_mapping if write_kv else None), _ptr(cache_layer if write_kv else None),
            _ptr(q), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(page),
            c_int(1 if write_kv else 0), c_int(cos.shape[0] if cos is not None else 1), c_int(qkv.shape[1]),
            c_int(_DT[out_dtype]), c_int(rot), c_int(self._dt(qkv, "qkv")), self._stream())
        _check("rope_cache_write", st)
        return q

    # ------------------------------------------------------------------ attention
    def paged_attention(self, q, cache_layer, meta: AttentionMeta, num_heads, num_kv_heads, head_dim,
                        scale: float, window: Optional[int]) -> torch.Tensor:
        """Attention of the step's tokens over the paged cache (keys of this step included).

        bfloat16 with a head size that is a multiple of 16 and pages of a power of two go to the
        tensor-core flash kernel (one token per sequence: the decode tiling, keys split over CTAs
        when the batch alone cannot fill the GPU); everything else goes to the plain kernel."""
        page = cache_layer.shape[3]
        if q.dtype != torch.bfloat16 or head_dim % 16 or head_dim > 256 or (page & (page - 1)):
            return self.paged_attention_plain(q, cache_layer, meta, num_heads, num_kv_heads, head_dim, scale, window)
        out = torch.empty_like(q)
        group = num_heads // num_kv_heads
        if self.TCGEN05_ATTENTION and meta.max_q_len >= self.TCGEN05_ATTENTION_MIN_TOKENS and head_dim in (64, 128) \
                and group <= 128 and page >= 8:
            self.attention_tcgen05(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window)
            if meta.num_decode:
                if self._balanced_ok(meta, group, num_kv_heads):
                    self.flash_decode_balanced(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window)
                else:
                    self.decode_attention(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window, q_filter=1)
            return out
        if meta.max_q_len == 1:
            if self._balanced_ok(meta, group, num_kv_heads):
                self.flash_decode_balanced(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window)
            else:
                self.decode_attention(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window,
                                      num_splits=self.decode_splits(meta, num_heads, num_kv_heads))
        elif meta.num_decode == 0:
            self.flash_attention(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window, mode=0)
        else:
            self.flash_attention(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window,
                                 mode=0, q_filter=2)
            self.decode_attention(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window, q_filter=1)
        return out

    def decode_attention(self, q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window,
                         num_splits=1, q_filter=0, status=None, tma=None, early=None):
        """Attention of the step's one-token sequences (all of them, or with q_filter 1 those among
        longer ones) with the decode tiling, the keys split over `num_splits` CTAs: the tiles come by
        TMA where the kernel is built for the sizes (head size 64 or 128, pages of 8 keys or more),
        by cp.async otherwise; both give the same bits."""
        tma = self.TMA_DECODE if tma is None else tma
        if not tma or head_dim not in (64, 128) or cache_layer.shape[3] < 8:
            return self.flash_attention(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window,
                                        mode=1, num_splits=num_splits, q_filter=q_filter, max_q_len=1)
        _need(q, "q", torch.bfloat16, 2); _need(cache_layer, "cache_layer", torch.bfloat16, 5)
        lib = self._lib("attention_flash.cu", (f"-DHEAD_DIM={head_dim}",))
        T = q.shape[0]
        scratch = None
        if num_splits > 1:
            scratch = torch.empty((num_splits * T * num_heads * (head_dim + 2),), dtype=torch.float32, device=q.device)
        early = self.TMA_DECODE_EARLY if early is None else early
        st = lib.rv_flash_decode_tma(
            _ptr(q), _ptr(cache_layer), ctypes.c_longlong(cache_layer.shape[0]), _ptr(meta.block_tables), _ptr(meta.cu_seqlens),
            _ptr(meta.ctx_lens), _ptr(out), _ptr(scratch), c_int(T), c_int(meta.num_seqs), c_int(num_heads), c_int(num_kv_heads),
            c_int(head_dim), c_int(cache_layer.shape[3]), c_int(meta.max_blocks), c_float(scale), c_int(window or 0), c_int(1),
            c_int(num_splits), c_int(q_filter), _ptr(status if status is not None else self._status),
            c_int(1 if (early and self.pdl) else 0), self._stream())
        _check("flash_decode_tma", st)
        return out

    def decode_splits(self, meta: AttentionMeta, num_heads: int, num_kv_heads: int) -> int:
        """Into how many CTAs the keys of a sequence are split in a decode step.  Three CTAs of
        the kernel fit an SM (444 on a GPU of 148 SMs) and run in waves; a CTA costs about 4 us plus 2.25 us
        per 64-key tile (measured with all slots busy, where the tiles' bytes arrive at the speed
        of the memory), the merge kernel 2.5 us.  The split count with the least modelled time is
        taken: it fills one wave when the batch is small and keeps the last wave full when it is
        large."""
        self_max_splits = 64          # a long context at a small batch still fills the GPU (one sequence of 32,768 keys: 55)
        group = num_heads // num_kv_heads
        ctas = meta.num_seqs * num_kv_heads * ((group + 15) // 16)
        tiles = max(1, (meta.max_ctx_len + 63) // 64)
        best, best_t = 1, float("inf")
        for s in range(1, min(self_max_splits, tiles) + 1):
            per = -(-tiles // s)
            if s > 1 and per < 2:
                break
            # (the merge kernel reads eight splits per round trip)
            t = -(-ctas * s // (3 * self.num_sms)) * (4.0 + 2.25 * per) + (2.0 + 0.5 * -(-s // 8) if s > 1 else 0.0)
            if t < best_t - 1e-9:
                best, best_t = s, t
        return best

    def _balanced_tma_ctas(self, lib, num_heads: int, num_kv_heads: int) -> int:
        """CTAs of the TMA-fed evenly cut kernel that stay resident (asked from the device once per shape)."""
        key = (id(lib), num_heads, num_kv_heads)
        cache = self.__dict__.setdefault("_balanced_ctas", {})
        if key not in cache:
            cache[key] = int(lib.rv_flash_balanced_tma_ctas(c_int(num_heads), c_int(num_kv_heads)))
        return cache[key]

    def _balanced_ok(self, meta, group: int, num_kv_heads: int) -> bool:
        """The evenly cut decode kernel serves batches whose (sequence, kv head) pairs alone fill more
        than half of the resident CTAs: there the split kernel leaves waves half empty, and sequences
        of unequal length (continuous batching) unbalance it; smaller batches are faster split."""
        return (self.BALANCED_DECODE and group <= 16 and meta.num_seqs <= 256
                and meta.num_decode * num_kv_heads >= self.BALANCED_MIN_PAIRS)

    def flash_decode_balanced(self, q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window, ctas=0,
                              tma=None, status=None):
        """Decode attention for the sequences of the step that bring one token, the 64-key tiles of
        all (sequence, kv head) pairs cut evenly over a fixed number of resident CTAs; sequences
        with more tokens are left alone.  The tiles come by TMA where the kernel is built for the
        sizes (head size 64 or 128, pages of 8 keys or more, up to 240 sequences), by cp.async
        otherwise; both give the same bits."""
        _need(q, "q", torch.bfloat16, 2); _need(cache_layer, "cache_layer", torch.bfloat16, 5)
        lib = self._lib("attention_flash.cu", (f"-DHEAD_DIM={head_dim}",))
        T = q.shape[0]
        tma = self.TMA_DECODE if tma is None else tma
        if tma and head_dim in (64, 128) and cache_layer.shape[3] >= 8 and meta.num_seqs <= 240:
            grid = ctas or self._balanced_tma_ctas(lib, num_heads, num_kv_heads)
            if grid > 0:
                pieces = lib.rv_flash_balanced_max_pieces(c_int(meta.max_ctx_len), c_int(num_kv_heads), c_int(grid))
                scratch = torch.empty((pieces * T * num_heads * (head_dim + 2),), dtype=torch.float32, device=q.device)
                counts = torch.empty((meta.num_seqs * num_kv_heads,), dtype=torch.int32, device=q.device)
                st = lib.rv_flash_decode_balanced_tma(
                    _ptr(q), _ptr(cache_layer), ctypes.c_longlong(cache_layer.shape[0]), _ptr(meta.block_tables),
                    _ptr(meta.cu_seqlens), _ptr(meta.ctx_lens), _ptr(out), _ptr(scratch), _ptr(counts), c_int(pieces), c_int(T),
                    c_int(meta.num_seqs), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(cache_layer.shape[3]),
                    c_int(meta.max_blocks), c_float(scale), c_int(window or 0), c_int(grid),
                    _ptr(status if status is not None else self._status), self._stream())
                _check("flash_decode_balanced_tma", st)
                return out
        grid = ctas or 3 * self.num_sms
        pieces = lib.rv_flash_balanced_max_pieces(c_int(meta.max_ctx_len), c_int(num_kv_heads), c_int(grid))
        scratch = torch.empty((pieces * T * num_heads * (head_dim + 2),), dtype=torch.float32, device=q.device)
        counts = torch.empty((meta.num_seqs * num_kv_heads,), dtype=torch.int32, device=q.device)
        st = lib.rv_flash_decode_balanced(
            _ptr(q), _ptr(cache_layer), _ptr(meta.block_tables), _ptr(meta.cu_seqlens), _ptr(meta.ctx_lens), _ptr(out),
            _ptr(scratch), _ptr(counts), c_int(pieces), c_int(T), c_int(meta.num_seqs), c_int(num_heads),
            c_int(num_kv_heads), c_int(head_dim), c_int(cache_layer.shape[3]), c_int(meta.max_blocks), c_float(scale),
            c_int(window or 0), c_int(grid), self._stream())
        _check("flash_decode_balanced", st)
        return out

    def flash_attention(self, q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window,
                        mode=0, num_splits=1, q_filter=0, max_q_len=None):
        _need(q, "q", torch.bfloat16, 2); _need(cache_layer, "cache_layer", torch.bfloat16, 5)
        lib = self._lib("attention_flash.cu", (f"-DHEAD_DIM={head_dim}",))
        T = q.shape[0]
        scratch = None
        if num_splits > 1:
            scratch = torch.empty((num_splits * T * num_heads * (head_dim + 2),), dtype=torch.float32, device=q.device)
        st = lib.rv_flash_attention(
            _ptr(q), _ptr(cache_layer), _ptr(meta.block_tables), _ptr(meta.cu_seqlens), _ptr(meta.ctx_lens),
            _ptr(out), _ptr(scratch), c_int(T), c_int(meta.num_seqs), c_int(num_heads), c_int(num_kv_heads),
            c_int(head_dim), c_int(cache_layer.shape[3]), c_int(meta.max_blocks), c_float(scale), c_int(window or 0),
            c_int(mode), c_int(max_q_len or meta.max_q_len), c_int(num_splits), c_int(q_filter), self._stream())
        _check("flash_attention", st)
        return out

    def attention_tcgen05(self, q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window, status=None):
        """The tcgen05 flash-attention kernel for the sequences of a step that bring more than one
        token (bfloat16, head size 64 or 128, groups of up to 128 heads, pages of at least 8 keys)."""
        _need(q, "q", torch.bfloat16, 2); _need(cache_layer, "cache_layer", torch.bfloat16, 5)
        lib = self._lib("attention_tcgen05.cu", (f"-DHEAD_DIM={head_dim}",))
        st = lib.rv_attention_tcgen05(
            _ptr(q), _ptr(cache_layer), ctypes.c_longlong(cache_layer.shape[0]), _ptr(meta.block_tables),
            _ptr(meta.cu_seqlens), _ptr(meta.ctx_lens), _ptr(out), c_int(q.shape[0]), c_int(meta.num_seqs),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(cache_layer.shape[3]), c_int(meta.max_blocks),
            c_float(scale), c_int(window or 0), c_int(meta.max_q_len), _ptr(status if status is not None else self._status), self._stream())
        _check("attention_tcgen05", st)
        return out

    def paged_attention_plain(self, q, cache_layer, meta, num_heads, num_kv_heads, head_dim, scale, window):
        _need(q, "q", dims=2); _need(cache_layer, "cache_layer", q.dtype, 5)
        out = torch.empty_like(q)
        st = self._lib("attention_ref.cu").rv_paged_attention_ref(
            _ptr(q), _ptr(cache_layer), _ptr(meta.block_tables), _ptr(meta.cu_seqlens), _ptr(meta.ctx_lens),
            _ptr(meta.token_seq), _ptr(out), c_int(q.shape[0]), c_int(num_heads), c_int(num_kv_heads),
            c_int(head_dim), c_int(cache_layer.shape[3]), c_int(meta.max_blocks), c_float(scale),
            c_int(window or 0), c_int(self._dt(q, "q")), self._stream())
        _check("paged_attention_plain", st)
        return out

    # ------------------------------------------------------------------ linear layers
    def linear(self, x, weight, bias=None, residual=None, out_dtype=None, norm=None) -> torch.Tensor:
        """x [M, K] . weight [N, K]^T (+ bias) (+ residual), accumulated in float.
        norm = (gamma, eps): x is normalised first (RMSNorm); few bfloat16 rows get it inside the GEMM.

        float32 operands: this project's FFMA kernel (no TF32 anywhere).  bfloat16 operands: the
        library GEMM; the residual is added in its float epilogue (beta = 1).  A weight kept in
        32 bits under a bfloat16 engine is multiplied in float32."""
        _need(x, "x", dims=2); _need(weight, "weight", dims=2)
        M, K = x.shape
        N = weight.shape[0]
        if weight.shape[1] != K:
            raise KernelError(f"linear: x has {K} columns, weight has {weight.shape[1]}")
        out_dtype = out_dtype or x.dtype
        if norm is not None:
            fuse = (self._can_fuse_norm(x, norm) and weight.dtype == torch.bfloat16 and self._use_decode_gemm(M, N, K, False)
                    and out_dtype in (torch.bfloat16, torch.float32)
                    and (residual is None or (residual.dtype == torch.bfloat16 and out_dtype == torch.bfloat16)))
            if fuse:
                return self.linear_decode(x, weight, bias, residual, out_dtype, norm=norm)
            x = self.rmsnorm(x, *norm)
        if weight.dtype == torch.float32:
            xf = x if x.dtype == torch.float32 else x.float()
            rf = None
            if residual is not None:
                rf = residual if residual.dtype == torch.float32 else residual.float()
                _need(rf, "residual", dims=2)
            if bias is not None:
                _need(bias, "bias", dims=1)
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
            st = self._lib("gemm_f32.cu").rv_gemm_f32(
                _ptr(xf), _ptr(weight), _ptr(bias), c_int(self._dt(bias, "bias") if bias is not None else 0),
                _ptr(rf), _ptr(out), c_int(M), c_int(N), c_int(K), self._stream())
            _check("gemm_f32", st)
            return out if out_dtype == torch.float32 else out.to(out_dtype)
        if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
            raise KernelError(f"linear: unsupported operand types {x.dtype} x {weight.dtype}")
        return self._linear_bf16(x, weight, bias, residual, out_dtype)

    def _linear_bf16(self, x, weight, bias, residual, out_dtype):
        M, K = x.shape
        if self._use_decode_gemm(M, weight.shape[0], K, False) and out_dtype in (torch.bfloat16, torch.float32) \
                and (residual is None or (residual.dtype == torch.bfloat16 and out_dtype == torch.bfloat16)):
            return self.linear_decode(x, weight, bias, residual, out_dtype)
        if self._tcgen05_fills(M, weight.shape[0]) and K % 8 == 0 and bias is None and out_dtype in (torch.bfloat16, torch.float32) \
                and (residual is None or (residual.dtype == torch.bfloat16 and out_dtype == torch.bfloat16)):
            return self.linear_tcgen05(x, weight, residual, out_dtype)
        if out_dtype == torch.float32:
            out = torch.mm(x, weight.t(), out_dtype=torch.float32)
            if bias is not None:
                out += bias.float()
            if residual is not None:
                out += residual.float()
            return out
        if residual is not None and bias is None:
            return torch.addmm(residual, x, weight.t())
        if residual is not None:
            # bias and residual: the sum is formed in float and rounded once
            out = torch.mm(x, weight.t(), out_dtype=torch.float32)
            out += bias.float()
            out += residual.float()
            return out.to(out_dtype)
        return torch.nn.functional.linear(x, weight, bias.to(x.dtype) if bias is not None else None)

    def _tcgen05_fills(self, M: int, N: int, gated: bool = False) -> bool:
        """Whether this project's tcgen05 GEMM is the one to use for M rows and N weight rows: from
        `TCGEN05_MIN_ROWS` rows on, and only where its persistent workers (one CTA per SM, or one pair per two SMs on
        tiles of 256 rows) are busy for at least `TCGEN05_MIN_FILL` of their rounds.  Where a last
        round stays mostly empty the library's GEMM, which cuts such shapes differently, measured
        20 to 140 % faster (o_proj at 512 rows: 22.6 against 41 us)."""
        if M < self.TCGEN05_MIN_ROWS:
            return False
        pair = self.PAIR_GEMM and (M % 256 == 0 or M % 256 > 128)
        rows, workers = (256, self.num_sms // 2) if pair else (128, self.num_sms)
        tiles = -(-M // rows) * (-(-(N // 2) // 128) if gated else -(-N // 256))
        rounds = -(-tiles // workers)
        return tiles >= self.TCGEN05_MIN_FILL * rounds * workers

    def _prefill_splits(self, M: int, N: int, K: int, gated: bool = False, head_dim: int = 0) -> int:
        """Into how many parts (1, 2 or 4) the prefill GEMM cuts K over a cluster of CTAs per tile of 128 rows x 256
        columns: as many as keep all CTAs within the SMs, with 32 k blocks each at least (the exchange of the partials
        through the cluster's shared memory costs about 7 us, as much as 16 k blocks); with the rotary epilogue only
        while a CTA's share of the columns holds whole heads."""
        if gated or not self.PREFILL_SPLIT_K or M < self.TCGEN05_MIN_ROWS:
            return 1
        tiles = -(-M // 128) * -(-N // 256)
        for s in (4, 2):
            if tiles * s <= self.num_sms and ((K + 63) // 64) // s >= self.PREFILL_SPLIT_MIN_KB and (head_dim == 0 or (256 // s) % head_dim == 0):
                return s
        return 1

    def _prefill_gemm_lib(self, M: int, pair=None, N: int = 0, gated: bool = False, head_dim: int = 0):
        """The tcgen05 GEMM library for M rows: built for pairs of CTAs (tiles of 256 rows) unless the
        last tile's second half would be empty, or for one CTA per tile (tiles of 128 rows); with
        tiles of 128 columns instead of 256 where the wide ones would leave half of the workers without
        a tile (N given: a few hundred rows of a product with few weight rows)."""
        if pair is None:
            pair = self.PAIR_GEMM and (M % 256 == 0 or M % 256 > 128)
        defines = ("-DRV_PAIR=1",) if pair else ()
        if N and self.NARROW_TILES and head_dim <= 128:        # (a head's rotation pairs lie in one tile)
            rows, workers = (256, self.num_sms // 2) if pair else (128, self.num_sms)
            tiles = -(-M // rows) * (-(-(N // 2) // 128) if gated else -(-N // 256))
            if 2 * tiles <= workers + workers // 8:
                defines = defines + ("-DBN=128",)
        return self._lib("gemm_tcgen05.cu", defines)

    def linear_tcgen05(self, x, weight, residual=None, out_dtype=None, gated=False, status=None, max_ctas=0, pair=None,
                       splits=None):
        """The tcgen05 / TMEM / TMA GEMM for bfloat16 (any M; K a multiple of 8).  gated: weight rows
        are [gate | up] and the result is silu(x gate^T) * (x up^T).  `status`: optional int32 device
        tensor that receives a non-zero code if a bounded wait inside the kernel gave up.  `pair`:
        the build on pairs of CTAs (cta_group::2) or on single CTAs; default: by the number of rows."""
        _need(x, "x", torch.bfloat16, 2); _need(weight, "weight", torch.bfloat16, 2)
        M, K = x.shape
        N = weight.shape[0]
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
        if residual is not None:
            _need(residual, "residual", torch.bfloat16, 2)
        epilogue = 2 if gated else (1 if residual is not None else 0)
        if splits is None:
            splits = self._prefill_splits(M, N, K, gated) if (max_ctas == 0 and pair is None) else 1
        if splits > 1:
            lib = self._lib("gemm_tcgen05.cu", ())          # K over a cluster: the build on single CTAs, wide tiles
        else:
            lib = self._prefill_gemm_lib(M, pair, N, gated)
        st = lib.rv_gemm_tcgen05_bf16(
            _ptr(x), _ptr(weight), _ptr(residual), _ptr(out), c_int(1 if out_dtype == torch.float32 else 0),
            c_int(M), c_int(N), c_int(K), c_int(epilogue), _ptr(status if status is not None else self._status), c_int(max_ctas),
            c_int(splits), self._stream())
        _check("gemm_tcgen05", st)
        return out

    def _use_decode_gemm(self, M: int, N: int, K: int, gated: bool) -> bool:
        """Whether the weight-streaming tcgen05 GEMM serves this product: few rows, and either
        enough 128-feature tiles to fill the GPU without splitting K, or so few rows that the
        split reduction is cheap."""
        if M <= 0 or K % 8:
            return False
        tiles = ((N // 2 + 63) // 64) if gated else (N + 127) // 128
        if M > self.DECODE_MAX_ROWS:
            return (not gated and self.CLUSTER_REDUCE and M <= self.DECODE_BLOCK_MAX_ROWS
                    and tiles * ((M + 127) // 128) <= self.num_sms)
        split_rows = self.CLUSTER_MAX_ROWS if (self.CLUSTER_REDUCE and not gated) else self.DECODE_SPLIT_ROWS
        return M <= max(split_rows, self.DECODE_SPLIT_ROWS) or self.gemm_splits(tiles, K) == 1

    def gemm_splits(self, n_tiles: int, K: int) -> int:
        """Into how many CTAs the K dimension of a decode GEMM is cut: about two CTAs per SM with
        at least four 64-wide k blocks each, three per SM where that still leaves sixteen (measured:
        cutting finer costs more in the merge than it gains in bandwidth)."""
        num_kb = (K + 63) // 64
        two, three = 2 * self.num_sms // max(n_tiles, 1), 3 * self.num_sms // max(n_tiles, 1)
        if three > two and num_kb // three >= 16:
            return min(three, 32)
        return max(1, min(two, num_kb // 4, 32))

    def _norm_args(self, norm, K):
        """ctypes arguments for a fused RMSNorm (gamma [K], eps), or the three nulls."""
        if norm is None:
            return c_void_p(0), c_int(0), c_float(0.0)
        gamma, eps = norm
        _need(gamma, "norm weight", dims=1)
        if gamma.shape[0] != K:
            raise KernelError(f"fused norm: gamma has {gamma.shape[0]} entries for rows of {K}")
        return _ptr(gamma), c_int(self._dt(gamma, "norm weight")), c_float(eps)

    def _can_fuse_norm(self, x, norm) -> bool:
        return (norm is not None and x.dtype == torch.bfloat16 and 0 < x.shape[0] <= self.FUSED_NORM_MAX_ROWS
                and x.shape[1] <= 8128)       # the kernel keeps gamma of its K range in shared memory

    def _cluster_policy(self, M, gated, splits, cluster, tiles, K, chosen):
        """(splits, cluster) of a decode GEMM.  Up to `CLUSTER_MAX_ROWS` rows of a product that is not
        gated are cut into at most 8 CTAs per tile, which add their partials up inside a cluster; where
        the caller left the cut open, about `CLUSTER_TARGET_CTAS` CTAs in all (measured: more CTAs
        than that delay the next kernel's first loads by more than they gain)."""
        if M > self.DECODE_MAX_ROWS and not gated:
            # blocks of 128 rows, one CTA per SM (four stages of 32 KB and the cluster's buffers fill one): K is
            # split so that tiles x row blocks x splits stay within the SMs, inside a cluster or not at all
            if not chosen:         # (clusters do not fill the last SMs of every GPC: an eighth of the SMs is left out of the count)
                splits = (self.num_sms - self.num_sms // 8) // max(tiles * ((M + 127) // 128), 1)
            splits = max(1, min(splits, 8, ((K + 63) // 64) // 4))
            return splits, splits >= 2 and cluster is not False
        if cluster is None:
            cluster = self.CLUSTER_REDUCE and not gated and 0 < M <= self.CLUSTER_MAX_ROWS and splits >= 2
            if cluster:
                if not chosen:
                    splits = max(2, min(self.CLUSTER_TARGET_CTAS // max(tiles, 1), ((K + 63) // 64) // 4))
                splits = min(splits, 8)
        return splits, bool(cluster)

    def linear_decode(self, x, weight, bias=None, residual=None, out_dtype=None, gated=False, splits=None, status=None,
                      norm=None, cluster=None):
        """The weight-streaming tcgen05 GEMM for few rows of bfloat16 activations (beyond 128 rows:
        in blocks of 128, K split inside a cluster or not at all).
        norm = (gamma, eps): RMSNorm applied to x inside the kernel (at most 16 rows)."""
        _need(x, "x", torch.bfloat16, 2); _need(weight, "weight", torch.bfloat16, 2)
        M, K = x.shape
        N = weight.shape[0]
        lib = self._lib("gemm_tcgen05_decode.cu")
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
        tiles = lib.rv_gemm_decode_tiles(c_int(N), c_int(1 if gated else 0))
        chosen = splits is not None
        if splits is None:
            splits = self.gemm_splits(tiles, K)
        splits = max(1, min(splits, (K + 63) // 64))
        splits, cluster = self._cluster_policy(M, gated, splits, cluster, tiles, K, chosen)
        scratch = None
        if splits > 1 and not (cluster and M > self.DECODE_MAX_ROWS):
            if self._decode_counters is None or self._decode_counters.numel() < tiles:
                self._decode_counters = torch.zeros((max(tiles, 4096),), dtype=torch.int32, device=x.device)
            mb = lib.rv_gemm_decode_padded_rows(c_int(M))
            scratch = torch.empty((tiles * splits * mb * 128,), dtype=torch.float32, device=x.device)
        if bias is not None:
            _need(bias, "bias", dims=1)
        if residual is not None:
            _need(residual, "residual", torch.bfloat16, 2)
        st = lib.rv_gemm_tcgen05_decode_bf16(
            _ptr(x), _ptr(weight), _ptr(bias), c_int(self._dt(bias, "bias") if bias is not None else 0), _ptr(residual),
            _ptr(out), c_int(1 if out_dtype == torch.float32 else 0), c_int(M), c_int(N), c_int(K),
            c_int(1 if gated else 0), c_int(splits), c_int(1 if cluster else 0), _ptr(scratch),
            _ptr(self._decode_counters if splits > 1 else None),
            _ptr(status if status is not None else self._status), *self._norm_args(norm, K), self._stream())
        _check("gemm_tcgen05_decode", st)
        return out

    def qkv_rope_cache_write(self, x, weight, bias, positions, cos, sin, slot_mapping, cache_layer,
                             num_heads, num_kv_heads, head_dim, norm=None) -> torch.Tensor:
        """The q/k/v product of the step's rows, then bias, rotation of q and k and the write of k
        and v into the rows' cache slots; returns q [T, num_heads * head_dim].  For few bfloat16
        rows this is one kernel (the decode GEMM's rotary epilogue); otherwise the product and
        `rope_cache_write` run one after the other, with the same result.  Tables narrower than
        head_dim / 2 (a rotation of the leading part of each head only) always take the latter.
        norm = (gamma, eps): x is normalised first (RMSNorm), inside the fused kernel where that runs."""
        M, K = x.shape
        full_rotation = cos is None or cos.shape[1] == head_dim // 2      # the rotary epilogues rotate whole heads
        few = 0 < M <= self.FUSED_QKV_MAX_ROWS or (M > self.DECODE_MAX_ROWS and self._use_decode_gemm(M, weight.shape[0], K, False))
        if (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and few and full_rotation
                and 128 % head_dim == 0 and K % 8 == 0 and weight.shape[0] == (num_heads + 2 * num_kv_heads) * head_dim):
            if norm is not None and not self._can_fuse_norm(x, norm):
                x, norm = self.rmsnorm(x, *norm), None
            return self._qkv_rope_fused(x, weight, bias, positions, cos, sin, slot_mapping, cache_layer,
                                        num_heads, num_kv_heads, head_dim, norm=norm)
        if norm is not None:
            x = self.rmsnorm(x, *norm)
        if (self.FUSED_QKV_PREFILL and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and full_rotation
                and self._tcgen05_fills(M, weight.shape[0]) and head_dim in (64, 128, 256) and K % 8 == 0
                and weight.shape[0] == (num_heads + 2 * num_kv_heads) * head_dim):
            return self._qkv_rope_tcgen05(x, weight, bias, positions, cos, sin, slot_mapping, cache_layer,
                                          num_heads, num_kv_heads, head_dim)
        # the product leaves its kernel in float and is rounded once, after bias and rotation
        qkv = self.linear(x, weight, out_dtype=torch.float32)
        return self.rope_cache_write(qkv, bias, positions, cos, sin, slot_mapping, cache_layer,
                                     num_heads, num_kv_heads, head_dim, out_dtype=x.dtype)

    def _qkv_rope_tcgen05(self, x, weight, bias, positions, cos, sin, slot_mapping, cache_layer,
                          num_heads, num_kv_heads, head_dim, status=None, max_ctas=0, pair=None, splits=None):
        """The prefill tcgen05 GEMM with the rotary epilogue (many rows, head sizes 64 / 128 / 256)."""
        _need(x, "x", torch.bfloat16, 2); _need(weight, "weight", torch.bfloat16, 2)
        _need(positions, "positions", torch.int32, 1); _need(slot_mapping, "slot_mapping", torch.int32, 1)
        _need(cache_layer, "cache_layer", torch.bfloat16, 5)
        M, K = x.shape
        if weight.shape[1] != K or positions.shape[0] < M or slot_mapping.shape[0] < M:
            raise KernelError("qkv_rope_cache_write: shapes of x, weight, positions and slot_mapping do not agree")
        if tuple(cache_layer.shape[1:3]) != (2, num_kv_heads) or cache_layer.shape[4] != head_dim:
            raise KernelError(f"qkv_rope_cache_write: cache layer of shape {tuple(cache_layer.shape)} does not "
                              f"fit {num_kv_heads} kv heads of {head_dim}")
        if cos is not None:
            _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
            if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
                raise KernelError("qkv_rope_cache_write: cos/sin tables must be [rows, head_dim/2]")
        if bias is not None:
            _need(bias, "bias", dims=1)
        q = torch.empty((M, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
        if splits is None:
            splits = self._prefill_splits(M, weight.shape[0], K, False, head_dim) if (max_ctas == 0 and pair is None) else 1
        if splits > 1:
            lib = self._lib("gemm_tcgen05.cu", ())
        else:
            lib = self._prefill_gemm_lib(M, pair, weight.shape[0], head_dim=head_dim)
        st = lib.rv_gemm_tcgen05_qkv_rope(
            _ptr(x), _ptr(weight), _ptr(bias), c_int(self._dt(bias, "bias") if bias is not None else 0),
            _ptr(positions), _ptr(cos), _ptr(sin), _ptr(slot_mapping), _ptr(cache_layer), _ptr(q), c_int(M), c_int(K),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(cache_layer.shape[3]),
            c_int(cos.shape[0] if cos is not None else 1), _ptr(status if status is not None else self._status), c_int(max_ctas),
            c_int(splits), self._stream())
        _check("gemm_tcgen05_qkv_rope", st)
        return q

    def _qkv_rope_fused(self, x, weight, bias, positions, cos, sin, slot_mapping, cache_layer,
                        num_heads, num_kv_heads, head_dim, splits=None, status=None, norm=None, cluster=None):
        _need(x, "x", torch.bfloat16, 2); _need(weight, "weight", torch.bfloat16, 2)
        _need(positions, "positions", torch.int32, 1); _need(slot_mapping, "slot_mapping", torch.int32, 1)
        _need(cache_layer, "cache_layer", torch.bfloat16, 5)
        M, K = x.shape
        N = weight.shape[0]
        if weight.shape[1] != K or positions.shape[0] < M or slot_mapping.shape[0] < M:
            raise KernelError("qkv_rope_cache_write: shapes of x, weight, positions and slot_mapping do not agree")
        if tuple(cache_layer.shape[1:3]) != (2, num_kv_heads) or cache_layer.shape[4] != head_dim:
            raise KernelError(f"qkv_rope_cache_write: cache layer of shape {tuple(cache_layer.shape)} does not "
                              f"fit {num_kv_heads} kv heads of {head_dim}")
        if cos is not None:
            _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
            if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
                raise KernelError("qkv_rope_cache_write: cos/sin tables must be [rows, head_dim/2]")
        if bias is not None:
            _need(bias, "bias", dims=1)
        lib = self._lib("gemm_tcgen05_decode.cu")
        tiles = lib.rv_gemm_decode_tiles(c_int(N), c_int(0))
        chosen = splits is not None
        if splits is None:
            splits = self.gemm_splits(tiles, K)
        splits = max(1, min(splits, (K + 63) // 64))
        splits, cluster = self._cluster_policy(M, False, splits, cluster, tiles, K, chosen)
        scratch = None
        if splits > 1 and not (cluster and M > self.DECODE_MAX_ROWS):
            if self._decode_counters is None or self._decode_counters.numel() < tiles:
                self._decode_counters = torch.zeros((max(tiles, 4096),), dtype=torch.int32, device=x.device)
            mb = lib.rv_gemm_decode_padded_rows(c_int(M))
            scratch = torch.empty((tiles * splits * mb * 128,), dtype=torch.float32, device=x.device)
        q = torch.empty((M, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
        st = lib.rv_gemm_decode_qkv_rope(
            _ptr(x), _ptr(weight), _ptr(bias), c_int(self._dt(bias, "bias") if bias is not None else 0),
            _ptr(positions), _ptr(cos), _ptr(sin), _ptr(slot_mapping), _ptr(cache_layer), _ptr(q), c_int(M), c_int(K),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(cache_layer.shape[3]),
            c_int(cos.shape[0] if cos is not None else 1), c_int(splits), c_int(1 if cluster else 0), _ptr(scratch),
            _ptr(self._decode_counters if splits > 1 else None), _ptr(status if status is not None else self._status), *self._norm_args(norm, K), self._stream())
        _check("gemm_decode_qkv_rope", st)
        return q

    def gate_up_silu(self, x, weight, norm=None) -> torch.Tensor:
        """silu(x Wg^T) * (x Wu^T) for weight rows [Wg | Wu]: one fused kernel for few bfloat16
        rows, else the product followed by the SiLU kernel.  norm = (gamma, eps): x is normalised
        first (RMSNorm), inside the kernel for few rows."""
        M, K = x.shape
        if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.shape[0] % 2 == 0 \
                and self._use_decode_gemm(M, weight.shape[0], K, True):
            if norm is not None and not self._can_fuse_norm(x, norm):
                x, norm = self.rmsnorm(x, *norm), None
            return self.linear_decode(x, weight, gated=True, norm=norm)
        if norm is not None:
            x = self.rmsnorm(x, *norm)
        if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and self._tcgen05_fills(M, weight.shape[0], True) \
                and K % 8 == 0 and weight.shape[0] % 2 == 0:
            return self.linear_tcgen05(x, weight, gated=True)
        return self.silu_mul(self.linear(x, weight))

    # ------------------------------------------------------------------ sampling
    def sample(self, logits, temperature=None, top_k=None, top_p=None, seeds=None, draw_index=None) -> torch.Tensor:
        """One token id per row of float logits.  All parameter tensors are per row; rows with
        temperature 0 (or `temperature` None) are greedy."""
        _need(logits, "logits", torch.float32, 2)
        R, V = logits.shape
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
        if temperature is not None:
            _need(temperature, "temperature", torch.float32, 1)
            _need(seeds, "seeds", torch.int64, 1); _need(draw_index, "draw_index", torch.int64, 1)
        if top_k is not None:
            _need(top_k, "top_k", torch.int32, 1)
        if top_p is not None:
            _need(top_p, "top_p", torch.float32, 1)
        st = self._lib("sampling.cu").rv_sample(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                                _ptr(seeds), _ptr(draw_index), _ptr(out), c_int(R), c_int(V),
                                                self._stream())
        _check("sample", st)
        return out
