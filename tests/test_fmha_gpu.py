"""GPU parity tests: the CUDA path (through the C ABI, via flashck_b200.ops) against the CPU oracle on the
same seeded inputs."""
import pytest
import torch

from flashck_b200 import _lib, ops
from flashck_b200.utils import MaskEnum, RopeEnum
from flashck_b200.utils.inputs import (make_paged_cache, normal_tensor, rotary_cos_sin, to_seqstarts,
                                       uniform_seqlens)
from helpers import assert_bits_equal, assert_lse_close, assert_o_close
from oracle import cpu as oracle

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("device_ok")]
DEV = "cuda:0"


def _cu(t):
    return None if t is None else t.to(DEV)


# ------------------------------------------------------------------------------------------------
# fmha_fwd, batch mode
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
def test_fmha_fwd_config1(dtype, causal):
    # BASELINE config 1: b=2, h=8, sq=sk=128, hdim=64, scale=1/sqrt(64)
    b, s, h, d = 2, 128, 8, 64
    q, k, v = (normal_tensor((b, s, h, d), dtype, 100 + i) for i in range(3))
    mt = 1 if causal else 0
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, scale=0.125, mask_type=mt, window=(-1, 0) if causal else (-1, -1))
    o, lse = ops.fmha_fwd(_cu(q), _cu(k), _cu(v), scale=0.125, causal=causal, return_lse=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


@pytest.mark.parametrize("sq,sk", [(1, 1), (1, 77), (15, 15), (17, 63), (64, 64), (65, 129), (127, 300), (129, 129),
                                   (200, 40)])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("mask", [(0, -1, -1), (1, -1, 0), (2, -1, 0), (2, 20, 0), (1, 5, 7), (3, 33, 0)])
def test_fmha_fwd_shapes_and_masks(sq, sk, d, mask):
    dtype = torch.bfloat16
    b, hq, hkv = 2, 4, 2
    q = normal_tensor((b, sq, hq, d), dtype, 1)
    k = normal_tensor((b, sk, hkv, d), dtype, 2)
    v = normal_tensor((b, sk, hkv, d), dtype, 3)
    mt, wl, wr = mask
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, mask_type=mt, window=(wl, wr))
    o, lse = ops.fmha_fwd(_cu(q), _cu(k), _cu(v), window_size=(wl, wr), mask_type=mt, return_lse=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("sq,sk,mt", [(384, 384, 1), (1000, 1000, 1), (300, 777, 0), (513, 1024, 2), (700, 300, 2),
                                      (257, 257, 0), (128, 128, 1), (256, 2048, 2), (1, 500, 0)])
def test_fmha_fwd_hdim128_many_tiles(dtype, sq, sk, mt):
    # hdim 128 with no mask / causal goes to the tcgen05 instance: several 128-key tiles, both Q tiles of a CTA,
    # ragged tails, bottom-right alignment with sq != sk
    b, hq, hkv, d = 2, 4, 2, 128
    q = normal_tensor((b, sq, hq, d), dtype, 1)
    k = normal_tensor((b, sk, hkv, d), dtype, 2)
    v = normal_tensor((b, sk, hkv, d), dtype, 3)
    win = (-1, 0) if mt else (-1, -1)
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, mask_type=mt, window=win)
    o, lse = ops.fmha_fwd(_cu(q), _cu(k), _cu(v), window_size=win, mask_type=mt, return_lse=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


@pytest.mark.parametrize("hq,hkv", [(4, 2), (8, 2), (3, 3)])
@pytest.mark.parametrize("sq,sk,mask", [
    (1000, 1000, (1, 256, 0)),    # causal sliding window: tiles left of the window are skipped
    (1000, 1000, (2, 100, 0)),
    (513, 1400, (2, 300, 0)),     # chunked prefill with a window, bottom-right aligned
    (700, 700, (3, 200, 150)),    # two-sided window
    (640, 640, (1, 0, 0)),        # only the diagonal
    (300, 900, (1, 64, -1)),      # left window only, top-left aligned: the last rows see to the end
    (900, 300, (2, 128, 0)),      # more queries than keys: the first rows see nothing
    (257, 257, (1, -1, 100)),     # right window only
])
def test_fmha_fwd_hdim128_window_masks(hq, hkv, sq, sk, mask):
    # window masks at hdim 128 on the tcgen05 instance, with paired heads (even GQA ratio) and with two row blocks of one
    # head per work item (odd ratio: the second block walks its first key tile fully masked under a left window)
    dtype = torch.bfloat16
    b, d = 2, 128
    q = normal_tensor((b, sq, hq, d), dtype, 11)
    k = normal_tensor((b, sk, hkv, d), dtype, 12)
    v = normal_tensor((b, sk, hkv, d), dtype, 13)
    mt, wl, wr = mask
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, mask_type=mt, window=(wl, wr))
    o, lse = ops.fmha_fwd(_cu(q), _cu(k), _cu(v), window_size=(wl, wr), mask_type=mt, return_lse=True)
    assert _lib.device_status() == 0
    assert _lib.get_instance_param(0, "last_instance") == 1
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


def test_fmha_fwd_instances_agree():
    # the tcgen05 instance and the general instance on the same problem
    from flashck_b200 import _lib
    dtype = torch.bfloat16
    lens = [700, 130, 1025]
    cu = to_seqstarts(lens)
    q = normal_tensor((sum(lens), 8, 128), dtype, 5).to(DEV)
    k = normal_tensor((sum(lens), 2, 128), dtype, 6).to(DEV)
    v = normal_tensor((sum(lens), 2, 128), dtype, 7).to(DEV)
    outs = []
    for use in (1, 0):
        _lib.set_instance_param(0, "use_sm100", use)
        try:
            outs.append(ops.fmha_fwd_var_len(q, k, v, cu.to(DEV), cu.to(DEV), max(lens), causal=True, return_lse=True))
        finally:
            _lib.set_instance_param(0, "use_sm100", 1)
    assert_o_close(outs[0][0], outs[1][0])
    assert_lse_close(outs[0][1], outs[1][1])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("exp_mode", [0, 1, 11, 12, 13])
def test_fmha_fwd_exp_modes_match_the_oracle(dtype, exp_mode):
    """Every way the tcgen05 softmax takes its exponentials (instance parameter exp_mode: fp32 on the exp2 unit, packed
    f16x2 on the exp2 unit, fp32 with a share on the FMA-pipe polynomial) against the oracle, causal and unmasked."""
    lens = [900, 130, 1, 385]
    cu = to_seqstarts(lens)
    q = normal_tensor((sum(lens), 8, 128), dtype, 15)
    k = normal_tensor((sum(lens), 2, 128), dtype, 16)
    v = normal_tensor((sum(lens), 2, 128), dtype, 17)
    old = _lib.get_instance_param(0, "exp_mode")
    _lib.set_instance_param(0, "exp_mode", exp_mode)
    try:
        for mt, window in ((1, (-1, 0)), (0, (-1, -1)), (2, (200, 0))):
            o_ref, lse_ref = oracle.fmha_fwd(q, k, v, seqstart_q=cu, seqstart_k=cu, mask_type=mt, window=window)
            o, lse = ops.fmha_fwd_var_len(_cu(q), _cu(k), _cu(v), _cu(cu), _cu(cu), max(lens), mask_type=mt,
                                          window_size=window, return_lse=True)
            assert_o_close(o, o_ref, f"O, exp_mode {exp_mode}, mask {mt}")
            assert_lse_close(lse, lse_ref, f"LSE, exp_mode {exp_mode}, mask {mt}")
    finally:
        _lib.set_instance_param(0, "exp_mode", old)
    assert _lib.get_instance_param(0, "exp_mode") == old


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fmha_fwd_packed_exp2_lse_with_one_dominant_late_key(dtype):
    """The hard case for the packed f16x2 exponentials: a row whose sum is one key, and that key arrives in a later key
    tile with a score a little above the running max, so that its exponential is taken at a positive argument (where f16
    is coarser) and nothing averages its rounding.  Queries and keys lie along one direction u: the ordinary keys score
    far below two others, key 5 (the running max after the first tile) and key 401, which beats it by 0.14 to 1.9 in log2
    units depending on the row -- so l = 1 + 2^delta, the share of the late key is up to 0.79, and its rounding shows in
    the LSE undiluted."""
    d, L, first, star = 128, 640, 5, 401  # the dominant key sits in the fourth 128-key tile
    g = torch.Generator().manual_seed(7)
    u = torch.zeros(d)
    u[:16] = 0.25  # |u| = 1
    a = torch.linspace(0.5, 6.5, L)                        # row r: q = a_r * sqrt(d) * u, so that q.k * scale = a_r * (k.u)
    q = (a[:, None] * d ** 0.5 * u[None, :]).to(dtype)
    ku = torch.full((L,), -40.0)                            # ordinary keys: weight e^(-33 a) against the two below
    ku[first] = -7.0                                        # the running max after the first tile
    ku[star] = -6.8                                         # 0.2 a_r above it: 0.14 .. 1.9 in log2 units over the rows
    k = (ku[:, None] * u[None, :]).to(dtype)
    v = torch.randn(L, d, generator=g).to(dtype)
    q, k, v = q[None, :, None, :].contiguous(), k[None, :, None, :].contiguous(), v[None, :, None, :].contiguous()
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v)
    worst = {}
    for exp_mode in (0, 1):
        old = _lib.get_instance_param(0, "exp_mode")
        _lib.set_instance_param(0, "exp_mode", exp_mode)
        try:
            o, lse = ops.fmha_fwd(_cu(q), _cu(k), _cu(v), return_lse=True)
        finally:
            _lib.set_instance_param(0, "exp_mode", old)
        assert_o_close(o, o_ref, f"O, exp_mode {exp_mode}")
        assert_lse_close(lse, lse_ref, f"LSE, exp_mode {exp_mode}")
        worst[exp_mode] = float((lse.cpu() - lse_ref).abs().max())
    print("max LSE error: fp32 exp2 %.3g, packed f16x2 exp2 %.3g" % (worst[0], worst[1]))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fmha_fwd_hdim64_runs_on_the_tcgen05_instance_and_agrees_with_the_general_one(dtype):
    """BASELINE config 1's geometry (hdim 64) and a longer varlen GQA problem at hdim 64: served by the tcgen05 kernel's
    hdim-64 instances (instance parameter use_sm100_hdim64), equal to the oracle and to the general instance."""
    lens = [128, 700, 1, 333]
    cu = to_seqstarts(lens)
    q, k, v = (normal_tensor((sum(lens), h, 64), dtype, 40 + i) for i, h in enumerate((8, 2, 2)))
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, seqstart_q=cu, seqstart_k=cu, mask_type=1, window=(-1, 0))
    outs = {}
    for use in (1, 0):
        _lib.set_instance_param(0, "use_sm100_hdim64", use)
        try:
            outs[use] = ops.fmha_fwd_var_len(_cu(q), _cu(k), _cu(v), _cu(cu), _cu(cu), max(lens), causal=True, return_lse=True)
            assert _lib.get_instance_param(0, "last_instance") == use
        finally:
            _lib.set_instance_param(0, "use_sm100_hdim64", 1)
    for use in (1, 0):
        assert_o_close(outs[use][0], o_ref, f"use_sm100_hdim64={use}")
        assert_lse_close(outs[use][1], lse_ref, f"use_sm100_hdim64={use}")
    assert _lib.device_status() == 0


def test_fmha_fwd_var_len_gqa():
    dtype = torch.bfloat16
    lens = [1, 64, 65, 200, 0, 333]
    cu = to_seqstarts(lens)
    hq, hkv, d = 8, 2, 128
    total = int(cu[-1])
    q = normal_tensor((total, hq, d), dtype, 11)
    k = normal_tensor((total, hkv, d), dtype, 12)
    v = normal_tensor((total, hkv, d), dtype, 13)
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, seqstart_q=cu, seqstart_k=cu, mask_type=1, window=(-1, 0))
    o, lse = ops.fmha_fwd_var_len(_cu(q), _cu(k), _cu(v), _cu(cu), _cu(cu), max(lens), causal=True, return_lse=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


def test_fmha_fwd_var_len_config2_small():
    # BASELINE config 2 at reduced size: same head geometry (32/8, hdim 128), fewer and shorter sequences
    dtype = torch.bfloat16
    lens = uniform_seqlens(4, 512, 1024, seed=2)
    cu = to_seqstarts(lens)
    hq, hkv, d = 32, 8, 128
    total = int(cu[-1])
    q = normal_tensor((total, hq, d), dtype, 21)
    k = normal_tensor((total, hkv, d), dtype, 22)
    v = normal_tensor((total, hkv, d), dtype, 23)
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, seqstart_q=cu, seqstart_k=cu, mask_type=1, window=(-1, 0))
    o, lse = ops.fmha_fwd_var_len(_cu(q), _cu(k), _cu(v), _cu(cu), _cu(cu), max(lens), causal=True, return_lse=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


def test_paged_prefill_variants():
    dtype = torch.bfloat16
    hq, hkv, d, page = 8, 2, 128, 16
    lens_k = [40, 129, 16, 300]
    lens_q = [40, 100, 3, 64]
    cache = make_paged_cache(lens_k, hkv, d, d, page, dtype, seed=5)
    cu_q = to_seqstarts(lens_q)
    q = normal_tensor((int(cu_q[-1]), hq, d), dtype, 31)
    o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqstart_q=cu_q, seqlen_k=cache.seqlen_k,
                                     block_table=cache.block_table, mask_type=2, window=(-1, 0))
    # block-table form
    o, lse = ops.fmha_fwd_paged_kv_prefill(_cu(q), _cu(cache.k), _cu(cache.v), _cu(cache.block_table),
                                           _cu(cache.seqlen_k), cu_seqlens_q=_cu(cu_q), max_seqlen_q=max(lens_q),
                                           causal=True, return_lse=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)
    # SGLang-style page table form of the same cache
    npages = [-(-l // page) for l in lens_k]
    indptr = torch.tensor([0] + list(torch.tensor(npages).cumsum(0)), dtype=torch.int32)
    indices = torch.cat([cache.block_table[b, :n] for b, n in enumerate(npages)]).to(torch.int32)
    last = torch.tensor([l - (n - 1) * page for l, n in zip(lens_k, npages)], dtype=torch.int32)
    o2, lse2 = ops.batch_prefill(_cu(q), _cu(cache.k), _cu(cache.v), _cu(cu_q), _cu(indptr), _cu(indices), _cu(last),
                                 max(lens_q), causal=True, return_lse=True)
    assert_o_close(o2, o_ref)
    assert_lse_close(lse2, lse_ref)


def _poison_page_tails(cache, lens, page):
    """NaN in every token slot of a sequence's pages past its length (what a cache allocated with torch.empty may
    hold there): no kernel may let those slots reach the output."""
    k, v = cache.k.clone(), cache.v.clone()
    for b, n in enumerate(lens):
        pages = -(-n // page)
        if pages == 0 or n % page == 0:
            continue
        pid = int(cache.block_table[b, pages - 1])
        k[pid, n % page:] = float("nan")
        v[pid, n % page:] = float("nan")
    return k, v


@pytest.mark.parametrize("page", [16, 32, 64, 128, 256])
def test_paged_paths_ignore_garbage_past_the_sequence_end(page):
    dtype = torch.bfloat16
    hq, hkv, d = 8, 2, 128
    lens_k = [40, 129, 17, 300, 1, 700, 256]
    lens_q = [40, 100, 3, 64, 1, 515, 256]
    cache = make_paged_cache(lens_k, hkv, d, d, page, dtype, seed=15)
    k_bad, v_bad = _poison_page_tails(cache, lens_k, page)
    cu_q = to_seqstarts(lens_q)
    q = normal_tensor((int(cu_q[-1]), hq, d), dtype, 32)
    o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqstart_q=cu_q, seqlen_k=cache.seqlen_k,
                                     block_table=cache.block_table, mask_type=2, window=(-1, 0))
    o, lse = ops.fmha_fwd_paged_kv_prefill(_cu(q), _cu(k_bad), _cu(v_bad), _cu(cache.block_table),
                                           _cu(cache.seqlen_k), cu_seqlens_q=_cu(cu_q), max_seqlen_q=max(lens_q),
                                           causal=True, return_lse=True)
    assert_o_close(o, o_ref, "paged prefill O")
    assert_lse_close(lse, lse_ref, "paged prefill LSE")
    # decode over the same poisoned cache
    qd = normal_tensor((len(lens_k), 1, hq, d), dtype, 33)
    od_ref, lsed_ref = oracle.fmha_fwd(qd, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
    for splits in (1, 3):
        od, lsed = ops.fmha_fwd_splitkv(_cu(qd), _cu(k_bad), _cu(v_bad), seqlen_k=_cu(cache.seqlen_k),
                                        block_table=_cu(cache.block_table), num_splits=splits, return_lse=True)
        assert_o_close(od, od_ref, f"decode O splits={splits}")
        assert_lse_close(lsed, lsed_ref, f"decode LSE splits={splits}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("page,hq,hkv", [(16, 8, 2), (64, 6, 2), (128, 4, 4), (512, 8, 1)])
def test_paged_prefill_tcgen05_instance_agrees_with_general_instance_and_oracle(dtype, page, hq, hkv):
    """hdim 128 paged prefill runs on the tcgen05 instance; the general instance and the oracle are the checks.
    Lengths cover: keys ending inside a page, inside a 128-key tile, on a tile edge; queries shorter than keys
    (chunked prefill, bottom-right causal) and equal to them; a sequence with no keys."""
    d = 128
    lens_k = [1, 127, 128, 129, 640, 1000, 0, 333]
    lens_q = [1, 100, 128, 5, 640, 300, 4, 333]
    cache = make_paged_cache(lens_k, hkv, d, d, page, dtype, seed=21)
    k_bad, v_bad = _poison_page_tails(cache, lens_k, page)
    cu_q = to_seqstarts(lens_q)
    q = normal_tensor((int(cu_q[-1]), hq, d), dtype, 34)
    o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqstart_q=cu_q, seqlen_k=cache.seqlen_k,
                                     block_table=cache.block_table, mask_type=2, window=(-1, 0))

    def run():
        return ops.fmha_fwd_paged_kv_prefill(_cu(q), _cu(k_bad), _cu(v_bad), _cu(cache.block_table),
                                             _cu(cache.seqlen_k), cu_seqlens_q=_cu(cu_q), max_seqlen_q=max(lens_q),
                                             causal=True, return_lse=True)
    o, lse = run()
    _lib.set_instance_param(0, "use_sm100", 0)
    try:
        o_gen, lse_gen = run()
    finally:
        _lib.set_instance_param(0, "use_sm100", 1)
    assert _lib.device_status() == 0
    assert_o_close(o, o_ref, "tcgen05 paged O")
    assert_lse_close(lse, lse_ref, "tcgen05 paged LSE")
    assert_o_close(o_gen, o_ref, "general paged O")
    assert_lse_close(lse_gen, lse_ref, "general paged LSE")
    # the SGLang-style page list of the same cache, no mask
    npages = [-(-l // page) for l in lens_k]
    indptr = torch.tensor([0] + list(torch.tensor(npages).cumsum(0)), dtype=torch.int32)
    indices = torch.cat([cache.block_table[b, :n] for b, n in enumerate(npages)]).to(torch.int32)
    last = torch.tensor([l - (n - 1) * page if n else 0 for l, n in zip(lens_k, npages)], dtype=torch.int32)
    o2_ref, lse2_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqstart_q=cu_q, seqlen_k=cache.seqlen_k,
                                       block_table=cache.block_table)
    o2, lse2 = ops.batch_prefill(_cu(q), _cu(k_bad), _cu(v_bad), _cu(cu_q), _cu(indptr), _cu(indices), _cu(last),
                                 max(lens_q), causal=False, return_lse=True)
    assert_o_close(o2, o2_ref, "batch_prefill O")
    assert_lse_close(lse2, lse2_ref, "batch_prefill LSE")


# ------------------------------------------------------------------------------------------------
# split-KV decode + combine
# ------------------------------------------------------------------------------------------------
def test_combine_matches_oracle():
    torch.manual_seed(0)
    bs, hq, S, rows, dv = 3, 5, 7, 4, 128
    lse_acc = torch.randn(bs, hq, S, rows) * 3
    lse_acc[0, 0, 2] = float("-inf")
    lse_acc[1, 1, :, 1] = float("-inf")  # a row no split saw
    o_acc = torch.randn(bs, hq, S, rows, dv)
    o_acc[0, 0, 2] = float("nan")  # the slot of an empty split is never read
    o_ref, lse_ref = oracle.splitkv_combine(lse_acc, torch.nan_to_num(o_acc), torch.bfloat16)
    o, lse = ops.fmha_fwd_splitkv_combine(_cu(lse_acc), _cu(o_acc), torch.bfloat16, return_lse=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("hq,hkv", [(32, 8), (16, 8), (8, 4), (6, 2), (3, 1), (16, 16)])
@pytest.mark.parametrize("num_splits", [1, 2, 5, 0])
def test_splitkv_paged_decode(page, hq, hkv, num_splits):
    dtype = torch.bfloat16
    d = 128
    lens = [1, 15, 16, 17, 127, 129, 1000, 0, 2049, 333]
    cache = make_paged_cache(lens, hkv, d, d, page, dtype, seed=7)
    q = normal_tensor((len(lens), 1, hq, d), dtype, 41)
    o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
    o, lse = ops.fmha_fwd_splitkv(_cu(q), _cu(cache.k), _cu(cache.v), seqlen_k=_cu(cache.seqlen_k),
                                  block_table=_cu(cache.block_table), num_splits=num_splits, return_lse=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


@pytest.mark.parametrize("dtype,d", [(torch.float16, 64), (torch.float16, 128), (torch.bfloat16, 64)])
def test_splitkv_dtypes_hdims(dtype, d):
    hq, hkv, page = 8, 2, 16
    lens = [100, 3, 777]
    cache = make_paged_cache(lens, hkv, d, d, page, dtype, seed=8)
    q = normal_tensor((len(lens), 1, hq, d), dtype, 42)
    o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
    o, lse = ops.fmha_fwd_splitkv(_cu(q), _cu(cache.k), _cu(cache.v), seqlen_k=_cu(cache.seqlen_k),
                                  block_table=_cu(cache.block_table), num_splits=4, return_lse=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


def test_splitkv_contiguous_cache_and_batch_idx():
    dtype = torch.bfloat16
    b, cap, hq, hkv, d = 4, 200, 8, 2, 128
    k = normal_tensor((b + 2, cap, hkv, d), dtype, 51)
    v = normal_tensor((b + 2, cap, hkv, d), dtype, 52)
    q = normal_tensor((b, 1, hq, d), dtype, 53)
    sl = torch.tensor([200, 1, 57, 128], dtype=torch.int32)
    idx = torch.tensor([5, 0, 3, 2], dtype=torch.int64)
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, seqlen_k=sl, cache_batch_idx=idx)
    o, lse = ops.fmha_fwd_splitkv(_cu(q), _cu(k), _cu(v), seqlen_k=_cu(sl), cache_batch_idx=_cu(idx), num_splits=3,
                                  return_lse=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


def test_splitkv_multi_token_queries_causal_and_window():
    # seqlen_q > 1 (the append + decode case): ragged q rows, bottom-right causal, optional sliding window
    dtype = torch.bfloat16
    hq, hkv, d, page = 32, 8, 128, 16
    lens_k = [300, 64, 1025, 17]
    lens_q = [16, 1, 7, 17]
    cache = make_paged_cache(lens_k, hkv, d, d, page, dtype, seed=9)
    cu_q = to_seqstarts(lens_q)
    q = normal_tensor((int(cu_q[-1]), hq, d), dtype, 61)
    for wl in (-1, 100):
        o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqstart_q=cu_q, seqlen_k=cache.seqlen_k,
                                         block_table=cache.block_table, mask_type=2, window=(wl, 0))
        o, lse = ops.fmha_fwd_splitkv(_cu(q), _cu(cache.k), _cu(cache.v), seqlen_k=_cu(cache.seqlen_k),
                                      block_table=_cu(cache.block_table), cu_seqlens_q=_cu(cu_q),
                                      max_seqlen_q=max(lens_q), num_splits=4, causal=True, window_size=(wl, 0),
                                      return_lse=True)
        assert_o_close(o, o_ref)
        assert_lse_close(lse, lse_ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("page,hq,hkv", [(16, 32, 8), (64, 16, 2), (128, 8, 8), (256, 8, 1)])
@pytest.mark.parametrize("num_splits", [1, 3, 16])
def test_splitkv_many_query_rows_tcgen05_instance(dtype, page, hq, hkv, num_splits):
    """More than 16 (token, group head) rows per kv head at hdim 128: the split-KV call runs on the tcgen05 instance
    (packed rows as one Q tile, pieces of the context as splits).  Checked against the oracle and against the
    mma.sync instance; page tails are poisoned with NaN.  Ragged query lengths (one sequence with a single token, one
    with more tokens than keys are not possible here: bottom-right causal needs sq <= sk for every row to see a key,
    so a short context is included instead), a sequence without keys, none and causal masks."""
    d = 128
    lens_k = [2000, 40, 1300, 0, 129, 3100]
    lens_q = [16, 7, 1, 3, 40, 33]
    cache = make_paged_cache(lens_k, hkv, d, d, page, dtype, seed=23)
    k_bad, v_bad = _poison_page_tails(cache, lens_k, page)
    cu_q = to_seqstarts(lens_q)
    q = normal_tensor((int(cu_q[-1]), hq, d), dtype, 35)
    for causal in (True, False):
        o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqstart_q=cu_q, seqlen_k=cache.seqlen_k,
                                         block_table=cache.block_table, mask_type=2 if causal else 0,
                                         window=(-1, 0) if causal else (-1, -1))

        def run():
            return ops.fmha_fwd_splitkv(_cu(q), _cu(k_bad), _cu(v_bad), seqlen_k=_cu(cache.seqlen_k),
                                        block_table=_cu(cache.block_table), cu_seqlens_q=_cu(cu_q),
                                        max_seqlen_q=max(lens_q), num_splits=num_splits, causal=causal, return_lse=True)
        o, lse = run()
        _lib.set_instance_param(0, "use_sm100_splitkv", 0)
        try:
            o_mma, lse_mma = run()
        finally:
            _lib.set_instance_param(0, "use_sm100_splitkv", 1)
        assert _lib.device_status() == 0
        assert_o_close(o, o_ref, f"tcgen05 split-KV O causal={causal}")
        assert_lse_close(lse, lse_ref, f"tcgen05 split-KV LSE causal={causal}")
        assert_o_close(o_mma, o_ref, f"mma.sync split-KV O causal={causal}")
        assert_lse_close(lse_mma, lse_ref, f"mma.sync split-KV LSE causal={causal}")


def test_splitkv_many_query_rows_contiguous_cache_batch_mode():
    # batch-mode q [b, sq, hq, d] against a contiguous cache [b, cap, hkv, d] with garbage behind each length
    dtype = torch.bfloat16
    b, sq, hq, hkv, d, cap = 3, 12, 16, 4, 128, 700
    lens = [700, 129, 333]
    k = normal_tensor((b, cap, hkv, d), dtype, 81)
    v = normal_tensor((b, cap, hkv, d), dtype, 82)
    k_bad, v_bad = k.clone(), v.clone()
    for i, n in enumerate(lens):
        k_bad[i, n:] = float("nan")
        v_bad[i, n:] = float("nan")
    q = normal_tensor((b, sq, hq, d), dtype, 83)
    sl = torch.tensor(lens, dtype=torch.int32)
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, seqlen_k=sl, mask_type=2, window=(-1, 0))
    o, lse = ops.fmha_fwd_splitkv(_cu(q), _cu(k_bad), _cu(v_bad), seqlen_k=_cu(sl), num_splits=4, causal=True,
                                  return_lse=True)
    assert _lib.device_status() == 0
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


def test_splitkv_many_query_rows_batch_mode_paged_cache_batch_idx_and_top_left_mask():
    """The remaining forms of the multi-token split-KV call on the tcgen05 instance: batch-mode q against a paged
    cache; a contiguous cache addressed through cache_batch_idx; a top-left aligned causal mask with far more keys
    than queries (most pieces of the context are then invisible and must come out as empty splits)."""
    dtype = torch.bfloat16
    hq, hkv, d, sq = 16, 4, 128, 9
    # batch mode + pages
    lens = [1500, 260, 17]
    cache = make_paged_cache(lens, hkv, d, d, 32, dtype, seed=27)
    q = normal_tensor((len(lens), sq, hq, d), dtype, 91)
    for mt in (2, 1):
        o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table,
                                         mask_type=mt, window=(-1, 0))
        o, lse = ops.fmha_fwd_splitkv(_cu(q), _cu(cache.k), _cu(cache.v), seqlen_k=_cu(cache.seqlen_k),
                                      block_table=_cu(cache.block_table), num_splits=6, mask_type=mt, window_size=(-1, 0),
                                      return_lse=True)
        assert _lib.device_status() == 0
        assert_o_close(o, o_ref, f"paged batch mode, mask {mt}")
        assert_lse_close(lse, lse_ref, f"paged batch mode, mask {mt}")
    # contiguous cache rows picked by cache_batch_idx
    rows, cap = 5, 600
    k = normal_tensor((rows, cap, hkv, d), dtype, 92)
    v = normal_tensor((rows, cap, hkv, d), dtype, 93)
    idx = torch.tensor([3, 0, 4], dtype=torch.int64)
    sl = torch.tensor([600, 77, 300], dtype=torch.int32)
    o_ref, lse_ref = oracle.fmha_fwd(q, k[idx], v[idx], seqlen_k=sl, mask_type=2, window=(-1, 0))
    o, lse = ops.fmha_fwd_splitkv(_cu(q), _cu(k), _cu(v), seqlen_k=_cu(sl), cache_batch_idx=_cu(idx), num_splits=4,
                                  causal=True, return_lse=True)
    assert _lib.device_status() == 0
    assert_o_close(o, o_ref, "contiguous cache with cache_batch_idx")
    assert_lse_close(lse, lse_ref, "contiguous cache with cache_batch_idx")


@pytest.mark.parametrize("num_splits", [1, 2, 3, 4, 16])
@pytest.mark.parametrize("sq", [8, 40])
def test_splitkv_many_query_rows_long_stream_and_few_splits(num_splits, sq):
    """One context far longer than a CTA's share of the work: its key tiles are cut over many CTAs, and the number of
    cuts is bounded by the splits the workspace has (a single split: the whole stream stays in one CTA; two pieces: one
    cut; 16 splits: as many as fit).  sq = 8 gives 32 packed rows (the form with duplicated rows, two splits per piece),
    sq = 40 gives 160 (two row blocks, one split per piece)."""
    dtype = torch.bfloat16
    hq, hkv, d, page = 8, 2, 128, 64
    lens_k = [40000, 5000, 300]
    cache = make_paged_cache(lens_k, hkv, d, d, page, dtype, seed=29)
    q = normal_tensor((len(lens_k), sq, hq, d), dtype, 97)
    o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table,
                                     mask_type=2, window=(-1, 0))
    o, lse = ops.fmha_fwd_splitkv(_cu(q), _cu(cache.k), _cu(cache.v), seqlen_k=_cu(cache.seqlen_k),
                                  block_table=_cu(cache.block_table), num_splits=num_splits, causal=True, return_lse=True)
    assert _lib.device_status() == 0
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("kind", ["bias0", "bias1", "bias2", "alibi0", "alibi1", "softcap", "softcap+bias2"])
def test_fmha_fwd_bias_alibi_and_soft_cap(dtype, d, kind):
    """The score additions of the reference's instance schema (bias_enum, bias_rank_info, has_logits_soft_cap) in batch
    mode, with a bottom-right causal mask, GQA, ragged sizes that end inside a tile."""
    b, sq, sk, hq, hkv = 2, 100, 171, 8, 2
    q, k, v = (normal_tensor(sh, dtype, sd) for sh, sd in (((b, sq, hq, d), 1), ((b, sk, hkv, d), 2), ((b, sk, hkv, d), 3)))
    bias = slopes = None
    cap = 0.0
    if "bias" in kind:
        bias = normal_tensor(((1, 1), (1, hq), (b, hq))[int(kind[-1])] + (sq, sk), dtype, 4)
    if "alibi" in kind:
        slopes = torch.rand((b if kind.endswith("1") else 1, hq), generator=torch.Generator().manual_seed(5)) * 0.5
    if "softcap" in kind:
        cap = 2.0
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, mask_type=2, window=(-1, 0), bias=bias, alibi_slopes=slopes,
                                     logits_soft_cap=cap)
    o, lse = ops.fmha_fwd(_cu(q), _cu(k), _cu(v), causal=True, return_lse=True, bias=_cu(bias) if bias is not None else None,
                          alibi_slopes=_cu(slopes) if slopes is not None else None, logits_soft_cap=cap)
    assert_o_close(o, o_ref, kind)
    assert_lse_close(lse, lse_ref, kind)
    # ALiBi and the soft cap are flags of the tcgen05 softmax; a bias tensor has tcgen05 instances at hdim 128
    assert _lib.get_instance_param(0, "last_instance") == (0 if "bias" in kind and d == 64 else 1)
    # the additions change the result (the test would pass vacuously if they were dropped on both sides)
    o_plain, _ = oracle.fmha_fwd(q, k, v, mask_type=2, window=(-1, 0))
    assert (o_plain.float() - o_ref.float()).abs().max() > 0.05


@pytest.mark.parametrize("window", [(-1, 0), (40, 0), (-1, -1)])
def test_fmha_fwd_alibi_and_soft_cap_together_on_the_tcgen05_instance(window):
    """ALiBi (per-batch slopes) and a soft cap in one call, group mode over several key tiles, with causal, sliding-window
    and no mask: the score-addition instances of the tcgen05 kernel."""
    dtype, hq, hkv, d = torch.bfloat16, 8, 2, 128
    lens = [300, 129, 1, 640]
    cu = to_seqstarts(lens)
    q, k, v = (normal_tensor((sum(lens), h, d), dtype, 30 + i) for i, h in enumerate((hq, hkv, hkv)))
    slopes = torch.rand((len(lens), hq), generator=torch.Generator().manual_seed(9)) * 0.3
    mt = 0 if window == (-1, -1) else 2
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, seqstart_q=cu, seqstart_k=cu, mask_type=mt, window=window, alibi_slopes=slopes,
                                     logits_soft_cap=15.0)
    o, lse = ops.fmha_fwd_var_len(_cu(q), _cu(k), _cu(v), _cu(cu), _cu(cu), max(lens), mask_type=mt, window_size=window,
                                  return_lse=True, alibi_slopes=_cu(slopes), logits_soft_cap=15.0)
    assert _lib.get_instance_param(0, "last_instance") == 1
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


def test_fallback_to_the_general_instance_is_reported_when_logging_is_on(capfd):
    import flashck_b200 as fck
    q = normal_tensor((1, 40, 4, 64), torch.bfloat16, 1)
    bias = _cu(normal_tensor((1, 1, 40, 40), torch.bfloat16, 2))  # a bias tensor is served by the general instance
    old = fck.get_flag_value("FC_TUNING_LOG")
    try:
        fck.set_flag_value("FC_TUNING_LOG", True)
        ops.fmha_fwd(_cu(q), _cu(q), _cu(q), bias=bias)
        torch.cuda.synchronize()
        assert "general (mma.sync) instance" in capfd.readouterr().err
        fck.set_flag_value("FC_TUNING_LOG", False)
        ops.fmha_fwd(_cu(q), _cu(q), _cu(q), bias=bias)
        torch.cuda.synchronize()
        assert "general" not in capfd.readouterr().err
    finally:
        fck.set_flag_value("FC_TUNING_LOG", old)
    assert _lib.get_instance_param(0, "last_instance") == 0


def test_fmha_fwd_var_len_bias_plane_and_alibi():
    """Group mode: the bias is one [1, hq, total_q, total_k] plane of which every sequence uses its own block; ALiBi
    slopes per (sequence, head)."""
    dtype = torch.bfloat16
    hq, hkv, d = 8, 4, 128
    lens_q, lens_k = [5, 130, 64], [77, 130, 300]
    cu_q, cu_k = to_seqstarts(lens_q), to_seqstarts(lens_k)
    tq, tk = int(cu_q[-1]), int(cu_k[-1])
    q, k, v = normal_tensor((tq, hq, d), dtype, 11), normal_tensor((tk, hkv, d), dtype, 12), normal_tensor((tk, hkv, d), dtype, 13)
    bias = normal_tensor((1, hq, tq, tk), dtype, 14)
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, seqstart_q=cu_q, seqstart_k=cu_k, mask_type=2, window=(-1, 0), bias=bias)
    o, lse = ops.fmha_fwd_var_len(_cu(q), _cu(k), _cu(v), _cu(cu_q), _cu(cu_k), max(lens_q), causal=True, return_lse=True,
                                  bias=_cu(bias))
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)
    slopes = torch.rand((len(lens_q), hq), generator=torch.Generator().manual_seed(6)) * 0.3
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, seqstart_q=cu_q, seqstart_k=cu_k, mask_type=2, window=(-1, 0),
                                     alibi_slopes=slopes)
    o, lse = ops.fmha_fwd_var_len(_cu(q), _cu(k), _cu(v), _cu(cu_q), _cu(cu_k), max(lens_q), causal=True, return_lse=True,
                                  alibi_slopes=_cu(slopes))
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rank,sq,sk,mask,window,cap", [
    (1, 300, 512, 2, (-1, 0), 0.0),     # rows of 512 keys: 16-byte loads; the last row block is ragged
    (2, 256, 640, 0, (-1, -1), 0.0),    # per-batch planes, no mask, whole tiles only
    (0, 200, 392, 2, (-1, 0), 3.0),     # shared plane, soft cap, sk a multiple of 8 but not of 128 (tail tile by elements)
    (1, 384, 384, 1, (100, 0), 0.0),    # sliding window: the instance with the second mask bound
    (1, 130, 259, 2, (-1, 0), 0.0),     # odd key count: every row starts unaligned
])
def test_fmha_fwd_elementwise_bias_on_the_tcgen05_instance(dtype, rank, sq, sk, mask, window, cap):
    """An elementwise bias tensor at hdim 128 runs on the tcgen05 kernel's BIAS instances (each softmax thread reads its
    row's 128 bias values per key tile): equal to the oracle, and to the general instance on the same call."""
    b, hq, hkv, d = 2, 4, 2, 128
    q, k, v = (normal_tensor(sh, dtype, sd) for sh, sd in (((b, sq, hq, d), 31), ((b, sk, hkv, d), 32), ((b, sk, hkv, d), 33)))
    bias = normal_tensor(((1, 1), (1, hq), (b, hq))[rank] + (sq, sk), dtype, 34)
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, mask_type=mask, window=window, bias=bias, logits_soft_cap=cap)
    kw = dict(return_lse=True, bias=_cu(bias), logits_soft_cap=cap)
    if mask:
        kw.update(window_size=window, mask_type=mask)

    def run():
        return ops.fmha_fwd(_cu(q), _cu(k), _cu(v), **kw)
    o, lse = run()
    assert _lib.get_instance_param(0, "last_instance") == 1
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)
    _lib.set_instance_param(0, "use_sm100_bias", 0)
    try:
        o_gen, lse_gen = run()
        assert _lib.get_instance_param(0, "last_instance") == 0
    finally:
        _lib.set_instance_param(0, "use_sm100_bias", 1)
    assert_o_close(o, o_gen, "tcgen05 against the general instance")
    assert_lse_close(lse, lse_gen)
    assert _lib.device_status() == 0


def test_fmha_fwd_bias_pointer_read_as_the_instance_parameters_say():
    """The reference's FmhaFwd symbol has a bias pointer and fixes its meaning per compiled instance; here the instance
    parameters bias_enum / bias_rank_info of the family do, and an inconsistent request is refused."""
    dtype = torch.float16
    b, s, h, d = 1, 48, 4, 64
    q, k, v = (normal_tensor((b, s, h, d), dtype, sd) for sd in (1, 2, 3))
    slopes = torch.tensor([[0.5, 0.25, 0.125, 0.0625]], dtype=torch.float32)
    o_ref, _ = oracle.fmha_fwd(q, k, v, alibi_slopes=slopes)
    qc, kc, vc, sc = _cu(q), _cu(k), _cu(v), _cu(slopes)
    o = torch.empty_like(qc)
    _lib.set_instance_param(0, "bias_enum", 2)
    try:
        assert _lib.get_instance_param(0, "bias_enum") == 2
        rc = _lib.lib().FmhaFwd(qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), sc.data_ptr(), o.data_ptr(), None, None, None,
                                b, s, s, h, h, d, d, s, 0.0, -1, -1, 0, torch.cuda.current_stream().cuda_stream, None, 3)
        _lib.check(rc, "FmhaFwd")
    finally:
        _lib.set_instance_param(0, "bias_enum", 1)
    assert_o_close(o, o_ref)
    with pytest.raises(RuntimeError):  # bias_enum without a buffer
        _lib.check(_lib.lib().FmhaFwdBias(qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), None, o.data_ptr(), None, None, None,
                                          b, s, s, h, h, d, d, s, 0.0, -1, -1, 0, None, None, 3, 1, 0, 0.0), "FmhaFwdBias")


def test_splitkv_many_query_rows_many_short_streams():
    """Many more streams than SMs, most of them one or two key tiles long, some empty, one long: every CTA's piece of the
    work then holds a list of whole streams between two cut ones."""
    dtype = torch.bfloat16
    hq, hkv, d, page, sq = 16, 4, 128, 16, 6
    lens_k = [(37 * i) % 290 for i in range(150)]
    lens_k[7] = 9000
    lens_k[60] = 0
    cache = make_paged_cache(lens_k, hkv, d, d, page, dtype, seed=31)
    q = normal_tensor((len(lens_k), sq, hq, d), dtype, 99)
    o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
    o, lse = ops.fmha_fwd_splitkv(_cu(q), _cu(cache.k), _cu(cache.v), seqlen_k=_cu(cache.seqlen_k),
                                  block_table=_cu(cache.block_table), num_splits=8, return_lse=True)
    assert _lib.device_status() == 0
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


@pytest.mark.parametrize("rank", [0, 1])
@pytest.mark.parametrize("sq", [1, 5, 24])
def test_splitkv_and_paged_prefill_with_alibi(rank, sq):
    """ALiBi slopes through the bias pointer of the paged entry points (decode with one and several query tokens, the
    latter beyond one 16-row tile too; paged prefill through a block table and through an SGLang-style page list)."""
    dtype = torch.bfloat16
    hq, hkv, d, page = 8, 2, 128, 16
    lens_k = [700, 45, 1290]
    b = len(lens_k)
    cache = make_paged_cache(lens_k, hkv, d, d, page, dtype, seed=41)
    q = normal_tensor((b, sq, hq, d), dtype, 42)
    slopes = torch.rand((b if rank else 1, hq), generator=torch.Generator().manual_seed(7)) * 0.2
    o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table,
                                     mask_type=2, window=(-1, 0), alibi_slopes=slopes)
    o_plain, _ = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table,
                                 mask_type=2, window=(-1, 0))
    assert (o_plain.float() - o_ref.float()).abs().max() > 0.05
    o, lse = ops.fmha_fwd_splitkv(_cu(q), _cu(cache.k), _cu(cache.v), seqlen_k=_cu(cache.seqlen_k),
                                  block_table=_cu(cache.block_table), num_splits=4, causal=True, return_lse=True,
                                  alibi_slopes=_cu(slopes))
    assert _lib.device_status() == 0
    assert_o_close(o, o_ref, "split-KV with ALiBi")
    assert_lse_close(lse, lse_ref, "split-KV with ALiBi")
    o, lse = ops.fmha_fwd_paged_kv_prefill(_cu(q), _cu(cache.k), _cu(cache.v), _cu(cache.block_table), _cu(cache.seqlen_k),
                                           causal=True, return_lse=True, alibi_slopes=_cu(slopes))
    assert_o_close(o, o_ref, "paged prefill with ALiBi")
    assert_lse_close(lse, lse_ref, "paged prefill with ALiBi")
    # the instance parameters are back at their defaults, and a bias pointer without them is refused
    assert _lib.get_instance_param(0, "bias_enum") == 1
    with pytest.raises(RuntimeError):
        qc = _cu(q)
        _lib.check(_lib.lib().FmhaFwdSplitKV(qc.data_ptr(), qc.data_ptr(), qc.data_ptr(), qc.data_ptr(), None, qc.data_ptr(),
                                             None, None, None, None, None, b, sq, 16, hq, hkv, d, d, sq, 1, 0, 0, 0.0, -1, -1,
                                             0, None, 4), "FmhaFwdSplitKV")


def test_splitkv_config3_small():
    # BASELINE config 3 geometry (32/8 heads, hdim 128, page 16, shuffled block table) at reduced batch/context
    dtype = torch.bfloat16
    lens = uniform_seqlens(8, 1024, 4096, seed=3)
    cache = make_paged_cache(lens, 8, 128, 128, 16, dtype, seed=10)
    q = normal_tensor((8, 1, 32, 128), dtype, 71)
    o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
    o, lse = ops.fmha_fwd_splitkv(_cu(q), _cu(cache.k), _cu(cache.v), seqlen_k=_cu(cache.seqlen_k),
                                  block_table=_cu(cache.block_table), return_lse=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


def test_combine_fp32_output_and_strided_form():
    torch.manual_seed(1)
    bs, hq, S, rows, dv = 2, 4, 3, 2, 128
    lse_acc = torch.randn(bs, hq, S, rows) * 2
    lse_acc[1, 2, 1] = float("-inf")
    o_acc = torch.randn(bs, hq, S, rows, dv)
    o_ref, lse_ref = oracle.splitkv_combine(lse_acc, o_acc, torch.bfloat16)
    o32, lse = ops.fmha_fwd_splitkv_combine(_cu(lse_acc), _cu(o_acc), torch.float32, return_lse=True)
    assert o32.dtype == torch.float32
    assert_o_close(o32, o_ref)
    assert_lse_close(lse, lse_ref)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_sequence_sharded_decode_ranks_emulated_on_one_gpu(world):
    # BASELINE config 5 geometry (64/8 heads, page 64) at reduced context; the ranks run one after the other on this
    # GPU and their fp32 partials are stacked where the all-gather would put them
    from flashck_b200 import dist as fdist
    dtype = torch.bfloat16
    lens = [5000, 130, 64, 0]
    hq, hkv, d, page = 64, 8, 128, 64
    cache = make_paged_cache(lens, hkv, d, d, page, dtype, seed=14)
    q = normal_tensor((len(lens), 1, hq, d), dtype, 111)
    o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
    qd, kd, vd = _cu(q), _cu(cache.k), _cu(cache.v)
    slots = []

    def capture(slot, group):
        slots.append(slot.clone())
        return slot.view(1, -1)

    for rank in range(world):
        table, local = fdist.shard_pages(lens, cache.block_table, page, rank, world)
        fdist.sequence_sharded_decode(qd, kd, vd, _cu(table), _cu(local), gather=capture)
    stacked = torch.stack(slots)

    def replay(slot, group):
        return stacked

    table, local = fdist.shard_pages(lens, cache.block_table, page, 0, world)
    o, lse = fdist.sequence_sharded_decode(qd, kd, vd, _cu(table), _cu(local), gather=replay, return_lse=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_sharded_combine_kernel_ranks_played_in_one_cooperative_launch(world):
    """FmhaFwdSplitKVShardedCombine (merge of the local splits + exchange of the partials + merge over the ranks in one
    kernel) with all ranks of the group played on this GPU in one cooperative launch, every exchange buffer local.
    Each rank's split partials come from the split-KV kernel on that rank's page shard; every rank's result must be the
    oracle's attention over the whole cache.  Three calls in a row on the same buffers: the second uses the other half
    of the buffers, the third finds the first call's flags in its half."""
    import ctypes
    from flashck_b200 import dist as fdist
    dtype = torch.bfloat16
    hq, hkv, d, page, S = 16, 2, 128, 64, 5
    lens = [8192 + 17, 130, 0, 64 * 9]
    b = len(lens)
    cache = make_paged_cache(lens, hkv, d, d, page, dtype, seed=61)
    k, v = _cu(cache.k), _cu(cache.v)
    shards = [fdist.shard_pages(lens, cache.block_table, page, r, world) for r in range(world)]
    lib = _lib.lib()
    nbytes = lib.FlashckShardExchangeBytes(b, 1, hq, d, world)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(world)]
    outs = [torch.empty(b, 1, hq, d, dtype=dtype, device=DEV) for _ in range(world)]
    lses = [torch.empty(b, hq, 1, dtype=torch.float32, device=DEV) for _ in range(world)]
    arr = lambda ts: (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(3):
        q = normal_tensor((b, 1, hq, d), dtype, 62 + call)
        o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
        qd = _cu(q)
        parts = [ops.fmha_fwd_splitkv(qd, k, v, seqlen_k=_cu(sl), block_table=_cu(bt), num_splits=S, combine=False)
                 for bt, sl in shards]
        for o_, l_ in zip(outs, lses):
            o_.fill_(float("nan"))
            l_.fill_(float("nan"))
        _lib.check(lib.FmhaFwdSplitKVShardedCombine(arr([p[0] for p in parts]), arr([p[1] for p in parts]), arr(outs),
                                                    arr(lses), arr(bufs), 0, world, world, b, 1, hq, d, S, _lib.BFLOAT16,
                                                    stream), "FmhaFwdSplitKVShardedCombine")
        assert _lib.device_status() == 0
        for r in range(world):
            assert_o_close(outs[r], o_ref, f"call {call}, rank {r} of {world}")
            assert_lse_close(lses[r], lse_ref, f"LSE, call {call}, rank {r} of {world}")
        header = bufs[0][:8].view(torch.int32).tolist()
        assert header == [call + 1, 0]  # calls completed, CTAs still running


def test_sharded_decoder_single_rank_matches_the_oracle_with_and_without_a_graph():
    """ShardedDecoder with one rank (no process group): two launches per step, nothing allocated per step, and the same
    step replayed from a CUDA graph after the inputs were updated in place."""
    from flashck_b200 import dist as fdist
    dtype = torch.bfloat16
    hq, hkv, d, page = 64, 8, 128, 64
    lens = [4096 + 5, 640]
    b = len(lens)
    cache = make_paged_cache(lens, hkv, d, d, page, dtype, seed=71)
    k, v, bt, sl = _cu(cache.k), _cu(cache.v), _cu(cache.block_table), _cu(cache.seqlen_k)
    q = normal_tensor((b, 1, hq, d), dtype, 72)
    qd = _cu(q)
    dec = fdist.ShardedDecoder(qd.shape, d, dtype, DEV)
    try:
        o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
        o, lse = dec(qd, k, v, bt, sl)
        assert_o_close(o, o_ref)
        assert_lse_close(lse, lse_ref)
        dec.capture(qd, k, v, bt, sl)
        q2 = normal_tensor((b, 1, hq, d), dtype, 73)
        qd.copy_(_cu(q2))
        o_ref, lse_ref = oracle.fmha_fwd(q2, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
        for _ in range(3):
            o, lse = dec.replay()
        torch.cuda.synchronize()
        assert_o_close(o, o_ref, "graph replay")
        assert_lse_close(lse, lse_ref, "graph replay")
        assert _lib.device_status() == 0
    finally:
        dec.close()


# ------------------------------------------------------------------------------------------------
# append-KV
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rope,rotary_dim", [(RopeEnum.INTERLEAVED, 128), (RopeEnum.HALF_ROTATED, 128),
                                             (RopeEnum.INTERLEAVED, 64), (RopeEnum.NONE, 0)])
def test_appendkv_paged_bit_exact(dtype, rope, rotary_dim):
    hq, hkv, d, page = 8, 2, 128, 16
    lens = [0, 5, 16, 31, 100]
    new = [3, 16, 1, 2, 9]
    cap = [l + n for l, n in zip(lens, new)]
    cache = make_paged_cache(lens, hkv, d, d, page, dtype, seed=12, capacity=cap)
    cu_n = to_seqstarts(new)
    total = int(cu_n[-1])
    q = normal_tensor((total, hq, d), dtype, 81)
    knew = normal_tensor((total, hkv, d), dtype, 82)
    vnew = normal_tensor((total, hkv, d), dtype, 83)
    cos, sin = rotary_cos_sin(max(cap) + 1, max(rotary_dim, 2), dtype)
    # oracle (in place on CPU copies)
    q_ref, k_ref, v_ref = q.clone(), cache.k.clone(), cache.v.clone()
    oracle.fmha_fwd_appendkv(q_ref, k_ref, knew, v_ref, vnew, cache.seqlen_k, cos, sin, rope_type=int(rope),
                             rotary_dim=rotary_dim, block_table=cache.block_table, seqstart_q=cu_n,
                             seqstart_knew=cu_n)
    qd, kd, vd = _cu(q), _cu(cache.k), _cu(cache.v)
    ops.fmha_fwd_append_kv(qd, kd, vd, _cu(knew), _cu(vnew), _cu(cache.seqlen_k), _cu(cos), _cu(sin), rope=rope,
                           rotary_dim=rotary_dim, block_table=_cu(cache.block_table), cu_seqlens_q=_cu(cu_n),
                           cu_seqlens_knew=_cu(cu_n))
    assert_bits_equal(kd, k_ref, "k cache")
    assert_bits_equal(vd, v_ref, "v cache")
    assert_bits_equal(qd, q_ref, "rotated q")


def test_appendkv_contiguous_batch_mode():
    dtype = torch.bfloat16
    b, cap, hq, hkv, d, n = 3, 64, 4, 4, 64, 4
    k = normal_tensor((b, cap, hkv, d), dtype, 91)
    v = normal_tensor((b, cap, hkv, d), dtype, 92)
    q = normal_tensor((b, n, hq, d), dtype, 93)
    knew = normal_tensor((b, n, hkv, d), dtype, 94)
    vnew = normal_tensor((b, n, hkv, d), dtype, 95)
    sl = torch.tensor([0, 10, 60], dtype=torch.int32)
    cos, sin = rotary_cos_sin(cap, d, dtype)
    q_ref, k_ref, v_ref = q.clone(), k.clone(), v.clone()
    oracle.fmha_fwd_appendkv(q_ref, k_ref, knew, v_ref, vnew, sl, cos, sin, rope_type=2)
    qd, kd, vd = _cu(q), _cu(k), _cu(v)
    ops.fmha_fwd_append_kv(qd, kd, vd, _cu(knew), _cu(vnew), _cu(sl), _cu(cos), _cu(sin), rope=RopeEnum.HALF_ROTATED)
    assert_bits_equal(kd, k_ref, "k cache")
    assert_bits_equal(vd, v_ref, "v cache")
    assert_bits_equal(qd, q_ref, "rotated q")


def test_appendkv_full_cache_skips_the_tokens_and_reports_it():
    """A token that does not fit its sequence's cache is not written and the status word says so.  Sequence 0 fills its
    two pages (32 tokens) and is asked to take 3 more: the block-table entry such a token would index is the first entry
    of sequence 1's row (a valid page of the pool, so that even a missing guard would stay inside the pool), and that
    page must come out unchanged.  Sequence 1 has room and takes its token."""
    dtype, hq, hkv, d, page = torch.bfloat16, 4, 2, 128, 16
    lens, new = [32, 10], [3, 1]
    cache = make_paged_cache(lens, hkv, d, d, page, dtype, seed=14, capacity=[32, 32])
    assert cache.block_table.shape[1] == 2
    cu_n = to_seqstarts(new)
    total = int(cu_n[-1])
    q = normal_tensor((total, hq, d), dtype, 111)
    knew = normal_tensor((total, hkv, d), dtype, 112)
    vnew = normal_tensor((total, hkv, d), dtype, 113)
    cos, sin = rotary_cos_sin(64, d, dtype)
    # expected: only sequence 1's token lands (oracle run on that sequence alone)
    q1, k_ref, v_ref = q[3:].clone(), cache.k.clone(), cache.v.clone()
    oracle.fmha_fwd_appendkv(q1, k_ref, knew[3:].contiguous(), v_ref, vnew[3:].contiguous(), cache.seqlen_k[1:], cos, sin,
                             rope_type=1, block_table=cache.block_table[1:].contiguous(), seqstart_q=to_seqstarts([1]),
                             seqstart_knew=to_seqstarts([1]))
    assert _lib.device_status() == 0
    kd, vd = _cu(cache.k), _cu(cache.v)
    ops.fmha_fwd_append_kv(_cu(q), kd, vd, _cu(knew), _cu(vnew), _cu(cache.seqlen_k), _cu(cos), _cu(sin),
                           block_table=_cu(cache.block_table), cu_seqlens_q=_cu(cu_n), cu_seqlens_knew=_cu(cu_n))
    assert_bits_equal(kd, k_ref, "k cache")
    assert_bits_equal(vd, v_ref, "v cache")
    assert _lib.device_status() == 0x40000000  # FLASHCK_STATUS_APPEND_OVERFLOW; reading clears it
    assert _lib.device_status() == 0


def test_append_then_decode_config4_small():
    # BASELINE config 4 flow at reduced size: append 1..16 tokens with interleaved RoPE, then split-KV decode
    dtype = torch.bfloat16
    b, hq, hkv, d, page = 6, 32, 8, 128, 16
    lens = uniform_seqlens(b, 200, 1500, seed=4)
    new = uniform_seqlens(b, 1, 16, seed=5)
    cap = [l + n for l, n in zip(lens, new)]
    cache = make_paged_cache(lens, hkv, d, d, page, dtype, seed=13, capacity=cap)
    cu_n = to_seqstarts(new)
    total = int(cu_n[-1])
    q = normal_tensor((total, hq, d), dtype, 101)
    knew = normal_tensor((total, hkv, d), dtype, 102)
    vnew = normal_tensor((total, hkv, d), dtype, 103)
    cos, sin = rotary_cos_sin(max(cap) + 1, d, dtype)
    q_ref, k_ref, v_ref = q.clone(), cache.k.clone(), cache.v.clone()
    oracle.fmha_fwd_appendkv(q_ref, k_ref, knew, v_ref, vnew, cache.seqlen_k, cos, sin, rope_type=1,
                             block_table=cache.block_table, seqstart_q=cu_n, seqstart_knew=cu_n)
    new_len = torch.tensor(cap, dtype=torch.int32)
    o_ref, lse_ref = oracle.fmha_fwd(q_ref, k_ref, v_ref, seqstart_q=cu_n, seqlen_k=new_len,
                                     block_table=cache.block_table, mask_type=2, window=(-1, 0))
    qd, kd, vd = _cu(q), _cu(cache.k), _cu(cache.v)
    ops.fmha_fwd_append_kv(qd, kd, vd, _cu(knew), _cu(vnew), _cu(cache.seqlen_k), _cu(cos), _cu(sin),
                           block_table=_cu(cache.block_table), cu_seqlens_q=_cu(cu_n), cu_seqlens_knew=_cu(cu_n))
    assert_bits_equal(kd, k_ref, "k cache")
    assert_bits_equal(vd, v_ref, "v cache")
    o, lse = ops.fmha_fwd_splitkv(qd, kd, vd, seqlen_k=_cu(new_len), block_table=_cu(cache.block_table),
                                  cu_seqlens_q=_cu(cu_n), max_seqlen_q=max(new), causal=True, return_lse=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


def test_dependent_launches_do_not_change_a_serving_loop():
    """Four append -> split-KV -> merge steps enqueued back to back without a synchronisation, once with programmatic
    dependent launches (instance parameter use_pdl = 1, the default: each kernel sets itself up under the tail of the one
    before it) and once with ordinary launches: every step's O and LSE and the final caches are bit for bit the same,
    and the last step matches the oracle."""
    dtype = torch.bfloat16
    b, hq, hkv, d, page, steps = 5, 32, 8, 128, 16, 4
    lens = uniform_seqlens(b, 300, 2500, seed=24)
    news = [uniform_seqlens(b, 1, 8, seed=30 + i) for i in range(steps)]
    cap = [l + sum(n[j] for n in news) for j, l in enumerate(lens)]
    cache = make_paged_cache(lens, hkv, d, d, page, dtype, seed=17, capacity=cap)
    cos, sin = rotary_cos_sin(max(cap) + 1, d, dtype)
    toks = [(normal_tensor((sum(n), hq, d), dtype, 200 + i), normal_tensor((sum(n), hkv, d), dtype, 300 + i),
             normal_tensor((sum(n), hkv, d), dtype, 400 + i)) for i, n in enumerate(news)]
    assert _lib.get_instance_param(0, "use_pdl") == 1

    def loop(pdl):
        _lib.set_instance_param(0, "use_pdl", pdl)
        try:
            kd, vd, cur = _cu(cache.k.clone()), _cu(cache.v.clone()), list(lens)
            outs = []
            for n, (q, kn, vn) in zip(news, toks):
                cu_n = _cu(to_seqstarts(n))
                qd = _cu(q.clone())
                ops.fmha_fwd_append_kv(qd, kd, vd, _cu(kn), _cu(vn), _cu(torch.tensor(cur, dtype=torch.int32)), _cu(cos), _cu(sin),
                                       block_table=_cu(cache.block_table), cu_seqlens_q=cu_n, cu_seqlens_knew=cu_n)
                cur = [c + x for c, x in zip(cur, n)]
                outs.append(ops.fmha_fwd_splitkv(qd, kd, vd, seqlen_k=_cu(torch.tensor(cur, dtype=torch.int32)),
                                                 block_table=_cu(cache.block_table), cu_seqlens_q=cu_n, max_seqlen_q=max(n),
                                                 causal=True, return_lse=True) + (qd,))
            torch.cuda.synchronize()
            return outs, kd, vd
        finally:
            _lib.set_instance_param(0, "use_pdl", 1)

    outs1, k1, v1 = loop(1)
    outs0, k0, v0 = loop(0)
    assert _lib.device_status() == 0
    assert torch.equal(k1, k0) and torch.equal(v1, v0)
    for (o1, l1, _), (o0, l0, _) in zip(outs1, outs0):
        assert torch.equal(o1, o0) and torch.equal(l1, l0)
    # the last step against the oracle, on the caches the loop left behind
    n, (o, lse, q_rot) = news[-1], outs1[-1]
    o_ref, lse_ref = oracle.fmha_fwd(q_rot.cpu(), k1.cpu(), v1.cpu(), seqstart_q=to_seqstarts(n),
                                     seqlen_k=torch.tensor(cap, dtype=torch.int32), block_table=cache.block_table,
                                     mask_type=2, window=(-1, 0))
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


def test_errors_are_loud():
    q = torch.zeros(1, 1, 3, 128, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(1, 16, 2, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="multiple"):
        ops.fmha_fwd(q, k, k)  # 3 q heads over 2 kv heads
    q = torch.zeros(1, 1, 2, 96, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(1, 16, 2, 96, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="hdim"):
        ops.fmha_fwd(q, k, k)
