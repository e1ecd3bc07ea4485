"""The host-side choices of the kernel library (how a product is cut over CTAs, which build of a
kernel serves a shape): plain arithmetic, checked without a GPU."""
from types import SimpleNamespace

from rvllm_b200.kernels.library import CudaKernels


def _k():
    return CudaKernels.__new__(CudaKernels)        # the policies read class constants only


def test_split_k_of_the_decode_gemm():
    k = _k()
    # many tiles: no split; few tiles: about two CTAs per SM with at least four k blocks each
    assert k.gemm_splits(1002, 4096) == 1 and k.gemm_splits(224, 4096) == 1
    assert k.gemm_splits(32, 4096) == 9 and k.gemm_splits(48, 4096) == 6
    assert k.gemm_splits(32, 14336) == 13                    # three per SM where sixteen k blocks are left for each
    assert k.gemm_splits(4, 64) == 1 and k.gemm_splits(1, 128) == 1


def test_cluster_reduce_is_chosen_for_few_rows_and_caps_the_splits():
    k = _k()
    # left open: about CLUSTER_TARGET_CTAS CTAs in all, at most 8 per tile, at least four k blocks each
    assert k._cluster_policy(8, False, 9, None, 32, 4096, False) == (7, True)
    assert k._cluster_policy(1, False, 6, None, 48, 4096, False) == (4, True)
    assert k._cluster_policy(32, False, 13, None, 32, 14336, False) == (7, True)
    assert k._cluster_policy(4, False, 2, None, 8, 512, False) == (2, True)
    # given by the caller: kept, up to 8
    assert k._cluster_policy(8, False, 3, None, 32, 4096, True) == (3, True)
    assert k._cluster_policy(8, False, 12, None, 32, 4096, True) == (8, True)
    # no cluster: one split, gated products, or when asked not to
    assert k._cluster_policy(8, False, 1, None, 1002, 4096, False) == (1, False)
    assert k._cluster_policy(8, True, 2, None, 224, 4096, False) == (2, False)
    assert k._cluster_policy(8, False, 9, False, 32, 4096, False) == (9, False)
    # beyond DECODE_MAX_ROWS, blocks of 128 rows: tiles x row blocks x splits within the SMs, four k blocks each at least
    assert k._cluster_policy(65, False, 9, None, 32, 4096, False) == (4, True)
    assert k._cluster_policy(128, False, 9, None, 48, 4096, False) == (2, True)
    assert k._cluster_policy(256, False, 9, None, 32, 4096, False) == (2, True)
    assert k._cluster_policy(300, False, 9, None, 48, 14336, False) == (1, False)
    assert k._cluster_policy(100, False, 7, None, 5, 1032, True) == (4, True)        # given: kept up to 8 and to four k blocks each


def test_which_products_take_the_weight_streaming_gemm():
    k = _k()
    assert k._use_decode_gemm(8, 4096, 4096, False) and k._use_decode_gemm(32, 4096, 14336, False)
    assert k._use_decode_gemm(64, 4096, 4096, False)         # K split over a cluster, up to 64 rows
    k.CLUSTER_REDUCE = False
    try:
        assert not k._use_decode_gemm(64, 4096, 4096, False) # without clusters K is split for at most 8 rows: the library there
        assert k._use_decode_gemm(8, 4096, 4096, False)
    finally:
        del k.CLUSTER_REDUCE
    assert k._use_decode_gemm(64, 28672, 4096, True) and k._use_decode_gemm(64, 128256, 4096, False)
    assert not k._use_decode_gemm(65, 28672, 4096, True) and not k._use_decode_gemm(8, 4096, 4100, False)
    # short prompts: q/k/v, o and down in blocks of 128 rows while tiles x row blocks leave SMs idle
    assert k._use_decode_gemm(65, 4096, 4096, False) and k._use_decode_gemm(256, 4096, 14336, False)
    assert k._use_decode_gemm(256, 6144, 4096, False) and not k._use_decode_gemm(256, 10240, 4096, False)
    assert not k._use_decode_gemm(257, 4096, 4096, False) and not k._use_decode_gemm(128, 128256, 4096, False)
    assert not k._use_decode_gemm(0, 4096, 4096, False)


def test_the_prefill_gemm_and_its_build_are_chosen_by_rows():
    k = _k()
    assert not k._tcgen05_fills(127, 4096) and k._tcgen05_fills(128, 4096) and k._tcgen05_fills(2048, 28672, True)
    # with a threshold on how full the rounds of the persistent workers are
    k.TCGEN05_MIN_FILL = 0.8
    try:
        assert k._tcgen05_fills(2048, 4096) and k._tcgen05_fills(2048, 6144) and k._tcgen05_fills(2048, 28672, True)
        assert not k._tcgen05_fills(512, 4096) and not k._tcgen05_fills(1536, 4096) and k._tcgen05_fills(1536, 6144)
    finally:
        del k.TCGEN05_MIN_FILL
    # pairs of CTAs where the last 256-row tile has rows in its second half
    picked = []
    k._lib = lambda source, defines=(): picked.append((source, tuple(defines)))
    for rows in (2048, 300, 129, 256, 128, 640):
        k._prefill_gemm_lib(rows)
    assert [bool(d) for _, d in picked] == [True, False, True, True, False, False]
    assert all(src == "gemm_tcgen05.cu" for src, _ in picked)
    # tiles of 128 columns where the 256-column ones would give at most half of the workers a tile
    picked.clear()
    for rows, n, gated, hd in ((384, 4096, False, 0), (512, 4096, False, 0), (2048, 4096, False, 0), (512, 28672, True, 0),
                               (384, 6144, False, 128), (384, 1536, False, 256)):
        k._prefill_gemm_lib(rows, None, n, gated, hd)
    assert [("-DBN=128" in d) for _, d in picked] == [True, True, False, False, True, False]


def test_k_of_the_prefill_gemm_is_cut_over_a_cluster_where_the_tiles_leave_sms_idle():
    k = _k()
    assert k._prefill_splits(512, 4096, 14336) == 2 and k._prefill_splits(384, 4096, 14336) == 2       # down: 64 / 48 tiles
    assert k._prefill_splits(300, 4096, 14336) == 2 and k._prefill_splits(2048, 4096, 14336) == 1
    assert k._prefill_splits(512, 4096, 4096) == 2 and k._prefill_splits(512, 6144, 4096) == 1         # 64 tiles; 96 tiles
    assert k._prefill_splits(384, 6144, 4096, False, 128) == 2 and k._prefill_splits(384, 1536, 4096, False, 256) == 1
    assert k._prefill_splits(512, 28672, 4096, True) == 1 and k._prefill_splits(100, 4096, 14336) == 1  # gated; too few rows
    assert k._prefill_splits(512, 4096, 2048) == 1                                                   # 32 k blocks a part at least


def test_key_splits_of_decode_attention_follow_the_wave_model():
    meta = lambda seqs, ctx: SimpleNamespace(num_seqs=seqs, max_ctx_len=ctx)
    assert _k().decode_splits(meta(8, 2088), 32, 8) == 6           # 384 CTAs: one wave of 444
    assert _k().decode_splits(meta(1, 2048), 32, 8) == 16          # two tiles per CTA at least
    for seqs in (1, 2, 3, 5, 8, 13, 24, 31):                              # never a split of fewer than two tiles, never more than 64
        for ctx in (1, 64, 65, 300, 1000, 4096, 100000):
            s = _k().decode_splits(meta(seqs, ctx), 32, 8)
            tiles = (ctx + 63) // 64
            assert 1 <= s <= 64 and (s == 1 or -(-tiles // s) >= 2)
    assert _k().decode_splits(meta(1, 32768), 32, 8) >= 40         # a long context alone still fills the GPU
    assert _k().decode_splits(meta(4, 64), 32, 8) == 1             # one tile: nothing to split


def test_the_build_check_compiles_both_builds_of_the_prefill_gemm():
    from rvllm_b200.kernels.variants import all_variants
    jobs = [(src, tuple(defs)) for src, defs in all_variants()]
    assert ("gemm_tcgen05.cu", ()) in jobs and ("gemm_tcgen05.cu", ("-DRV_PAIR=1",)) in jobs
    assert ("sampling.cu", ()) in jobs and ("gemm_tcgen05_decode.cu", ()) in jobs
    assert len(jobs) == len(set(jobs))
