"""GPU tests at the full sizes of the BASELINE configurations, through properties that do not need the oracle on
the whole problem: two independent kernel instances agree, the number of splits does not change the merged
result, the oracle confirms the shortest sequences (which it finishes in a second or two) and, on the longest
sequences -- where the lazy rescale of the running max, the 31-bit row arithmetic and the bounds of the work lists
matter -- sampled query rows (prefill: one row costs L*d multiply-adds per head) or whole sequences (decode: a few
rows each)."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from flashck_b200 import _lib, ops  # noqa: E402
from helpers import assert_lse_close, assert_o_close  # noqa: E402
from oracle import cpu as oracle  # noqa: E402

pytestmark = pytest.mark.gpu


def _bench():
    import bench  # the workload generators of the benchmark: the same seeded shapes and value distributions
    return bench


def _shortest(lens, n):
    return sorted(range(len(lens)), key=lambda i: lens[i])[:n]


def _longest(lens, n):
    return sorted(range(len(lens)), key=lambda i: -lens[i])[:n]


def _sample_rows(L, n, seed):
    """Row indices of a sequence of L rows: both ends, the rows either side of every 128-row tile edge near the ends
    and the middle, and seeded random ones."""
    g = torch.Generator().manual_seed(seed)
    fixed = [0, 1, 126, 127, 128, 129, L // 2 // 128 * 128 - 1, L // 2 // 128 * 128, L - 130, L - 129, L - 128, L - 2, L - 1]
    rnd = torch.randint(0, L, (n,), generator=g).tolist()
    return sorted({r for r in fixed + rnd if 0 <= r < L})


def _gather_pages(w, b):
    """The K/V rows of sequence b of a paged workload, in token order, on the CPU."""
    n, page = w["lens"][b], w["page"]
    ids = w["table"][b, :-(-n // page)].long()
    k = w["k"][ids].reshape(-1, w["hkv"], w["k"].shape[-1])[:n].cpu()
    v = w["v"][ids].reshape(-1, w["hkv"], w["v"].shape[-1])[:n].cpu()
    return k, v


def test_config2_full_size_instances_agree_and_shortest_sequences_match_the_oracle():
    bench = _bench()
    dev = torch.device("cuda:0")
    w = bench.make_prefill(1234, dev)

    def run():
        return ops.fmha_fwd_var_len(w["q"], w["k"], w["v"], w["cu"], w["cu"], w["max_len"], causal=True, return_lse=True)
    o, lse = run()
    _lib.set_instance_param(0, "use_sm100", 0)
    try:
        o_gen, lse_gen = run()
    finally:
        _lib.set_instance_param(0, "use_sm100", 1)
    assert _lib.device_status() == 0
    assert_o_close(o, o_gen, "tcgen05 instance against the general instance, config 2")
    assert_lse_close(lse, lse_gen, "LSE, tcgen05 against general, config 2")
    cu = w["cu"].cpu()
    for b in _shortest(w["lens"], 3):
        sl = slice(int(cu[b]), int(cu[b + 1]))
        o_ref, lse_ref = oracle.fmha_fwd(w["q"][sl].cpu()[None], w["k"][sl].cpu()[None], w["v"][sl].cpu()[None],
                                         mask_type=2, window=(-1, 0))
        assert_o_close(o[sl], o_ref[0], f"sequence {b} against the oracle")
        assert_lse_close(lse[:, sl], lse_ref[0], f"LSE of sequence {b} against the oracle")


def test_config2_full_size_sampled_rows_of_the_longest_sequences_match_the_oracle():
    """Causal row i of a sequence sees keys 0..i, so its O and LSE for all heads are an unmasked attention of one query
    row over the first i + 1 keys: the oracle computes exactly that, for about 40 rows of each of the three longest
    sequences of BASELINE config 2 (lengths close to 4096)."""
    bench = _bench()
    dev = torch.device("cuda:0")
    w = bench.make_prefill(1234, dev)
    o, lse = ops.fmha_fwd_var_len(w["q"], w["k"], w["v"], w["cu"], w["cu"], w["max_len"], causal=True, return_lse=True)
    assert _lib.device_status() == 0
    cu = w["cu"].cpu()
    o, lse = o.cpu(), lse.cpu()
    checked = 0
    for b in _longest(w["lens"], 3):
        s0, L = int(cu[b]), w["lens"][b]
        qb, kb, vb = (w[n][s0:s0 + L].cpu() for n in ("q", "k", "v"))
        for i in _sample_rows(L, 28, seed=100 + b):
            o_ref, lse_ref = oracle.fmha_fwd(qb[i:i + 1][None], kb[None, :i + 1].contiguous(), vb[None, :i + 1].contiguous())
            assert_o_close(o[s0 + i], o_ref[0, 0], f"sequence {b} (L={L}) row {i} against the oracle")
            assert_lse_close(lse[:, s0 + i], lse_ref[0, :, 0], f"LSE of sequence {b} row {i} against the oracle")
            checked += 1
    assert checked >= 100


def test_config3_full_size_split_count_does_not_change_the_result_and_oracle_on_shortest():
    bench = _bench()
    dev = torch.device("cuda:0")
    w = bench.make_decode(4321, dev)

    def run(splits):
        return ops.fmha_fwd_splitkv(w["q"], w["k"], w["v"], seqlen_k=w["seqlen"], block_table=w["table"],
                                    num_splits=splits, return_lse=True)
    o, lse = run(0)      # the default depth
    o1, lse1 = run(1)    # one split per sequence: no merge arithmetic at all
    o9, lse9 = run(9)
    assert _lib.device_status() == 0
    assert_o_close(o, o1, "default splits against one split, config 3")
    assert_lse_close(lse, lse1, "LSE, default splits against one split")
    assert_o_close(o9, o1, "nine splits against one split, config 3")
    assert_lse_close(lse9, lse1, "LSE, nine splits against one split")
    for b in _shortest(w["lens"], 3) + _longest(w["lens"], 6):  # (a decode row is cheap: the longest ones in full)
        k, v = _gather_pages(w, b)
        o_ref, lse_ref = oracle.fmha_fwd(w["q"][b:b + 1].cpu(), k[None], v[None])
        assert_o_close(o[b:b + 1], o_ref, f"sequence {b} against the oracle")
        assert_lse_close(lse[b:b + 1], lse_ref, f"LSE of sequence {b} against the oracle")


def test_config4_full_size_append_then_decode_both_instances_and_oracle_on_shortest():
    bench = _bench()
    dev = torch.device("cuda:0")
    w = bench.make_append_decode(777, dev)
    cu_n, max_new = w["cu_new"], max(w["new"])
    k_before = w["k"].clone()
    q_rot = w["qn"].clone()
    ops.fmha_fwd_append_kv(q_rot, w["k"], w["v"], w["kn"], w["vn"], w["ctx_len"], w["cos"], w["sin"],
                           block_table=w["table"], cu_seqlens_q=cu_n, cu_seqlens_knew=cu_n)
    # the append touched exactly the new tokens' slots: every other row of the K pool is bit for bit what it was
    changed = (w["k"] != k_before).flatten(2).any(dim=2)  # [pages, page]
    assert int(changed.sum()) <= sum(w["new"])
    del k_before, changed

    def run():
        return ops.fmha_fwd_splitkv(q_rot, w["k"], w["v"], seqlen_k=w["seqlen"], block_table=w["table"], cu_seqlens_q=cu_n,
                                    max_seqlen_q=max_new, causal=True, return_lse=True)
    o, lse = run()
    _lib.set_instance_param(0, "use_sm100_splitkv", 0)
    try:
        o_mma, lse_mma = run()
    finally:
        _lib.set_instance_param(0, "use_sm100_splitkv", 1)
    assert _lib.device_status() == 0
    assert_o_close(o, o_mma, "tcgen05 split modes against the mma.sync decode kernel, config 4")
    assert_lse_close(lse, lse_mma, "LSE, tcgen05 against mma.sync, config 4")
    cu = cu_n.cpu()
    for b in _shortest(w["lens"], 3) + _longest(w["lens"], 4):  # (at most 16 query rows each: the longest ones in full)
        k, v = _gather_pages(w, b)
        sl = slice(int(cu[b]), int(cu[b + 1]))
        o_ref, lse_ref = oracle.fmha_fwd(q_rot[sl].cpu()[None], k[None], v[None], mask_type=2, window=(-1, 0))
        assert_o_close(o[sl], o_ref[0], f"sequence {b} against the oracle")
        assert_lse_close(lse[:, sl], lse_ref[0], f"LSE of sequence {b} against the oracle")


def test_config2_full_size_on_8bit_operands_instances_agree_and_sampled_rows_match_the_oracle():
    """BASELINE config 2 quantised to E4M3 (the bench's 8-bit leg): the kind::f8f6f4 tcgen05 instance against the general
    instance on the whole problem, and against the oracle on sampled rows of the longest sequence (a causal row is an
    unmasked attention of one query over the keys before it).  Bound: one 8-bit unit of P per key, i.e. the attention of
    the same weights over |V| (see tests/test_fp8_gpu.py)."""
    bench = _bench()
    dev = torch.device("cuda:0")
    w = bench.make_prefill(1234, dev)
    dtype = torch.float8_e4m3fn
    (q8, dq), (k8, dk), (v8, dv8) = (ops.quantize_fp8(w[n], dtype) for n in ("q", "k", "v"))
    scale_s, scale_p = dq * dk / 128 ** 0.5, 256.0
    scale_o = dv8 / scale_p

    def run():
        return ops.fmha_fwd_fp8(q8, k8, v8, scale_s=scale_s, scale_p=scale_p, scale_o=scale_o, cu_seqlens_q=w["cu"],
                                cu_seqlens_k=w["cu"], max_seqlen_q=w["max_len"], causal=True, out_dtype=torch.bfloat16,
                                return_lse=True)
    o, lse = run()
    assert _lib.get_instance_param(0, "last_instance") == 1
    _lib.set_instance_param(0, "use_sm100_fp8", 0)
    try:
        o_gen, lse_gen = run()
        assert _lib.get_instance_param(0, "last_instance") == 0
    finally:
        _lib.set_instance_param(0, "use_sm100_fp8", 1)
    assert _lib.device_status() == 0
    assert torch.isfinite(o.float()).all()
    assert_lse_close(lse, lse_gen, "LSE, tcgen05 8-bit instance against the general one")
    # both round P to 8 bits relative to their own running maximum: two units of P apart at most, measured against |O|
    # of the weights over |V| -- bounded here by the mean magnitude of V's rows times two units (a loose global bound)
    diff = (o.float() - o_gen.float()).abs()
    assert float(diff.max()) < 0.25 and float(diff.mean()) < 0.01
    cu = w["cu"].cpu()
    b = _longest(w["lens"], 1)[0]
    s0, L = int(cu[b]), w["lens"][b]
    qb, kb, vb = (t[s0:s0 + L].cpu() for t in (q8, k8, v8))
    o_c, lse_c = o.cpu(), lse.cpu()
    kw = dict(scale_s=scale_s, scale_p=scale_p, scale_o=scale_o, mask_type=0, window=(-1, -1), out_dtype=torch.bfloat16)
    for i in _sample_rows(L, 10, seed=5):
        kk, vv = kb[None, :i + 1].contiguous(), vb[None, :i + 1].contiguous()
        o_ref, lse_ref = oracle.fmha_fwd_fp8(qb[i:i + 1][None], kk, vv, **kw)
        o_abs, _ = oracle.fmha_fwd_fp8(qb[i:i + 1][None], kk, vv.float().abs().to(dtype), **kw)
        err = (o_c[s0 + i].float() - o_ref[0, 0].float()).abs()
        assert bool((err <= 2.0 ** -3 * o_abs[0, 0].float() + 1e-2).all()), f"row {i}: max err {float(err.max()):.4g}"
        assert_lse_close(lse_c[:, s0 + i], lse_ref[0, :, 0], f"LSE of row {i}")
