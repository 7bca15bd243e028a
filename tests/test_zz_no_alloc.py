"""FmhaFwdSplitKVStatic -- the entry point for callers that cannot allocate device memory (a serving loop with a
fixed memory plan, code confined to a framework allocator).  It keeps the split-KV workspaces in an array
inside the library, so its result must equal what the regular pair FmhaFwdSplitKV + FmhaFwdSplitKVCombine gives
with caller-owned workspaces.  Checked through the C ABI on two calls in a row (the second call finds the
array full of the first call's data), and once more with a problem that does not fit the array.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

from flashck_b200 import _lib
from flashck_b200.utils.inputs import make_paged_cache, normal_tensor
from helpers import assert_lse_close, assert_o_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _run_both(lens, hq, hkv, num_splits, seed):
    d, page, dtype = 128, 16, torch.bfloat16
    cache = make_paged_cache(lens, hkv, d, d, page, dtype, seed=seed)
    b = len(lens)
    q = normal_tensor((b, 1, hq, d), dtype, seed + 5).to(DEV)
    k, v = cache.k.to(DEV), cache.v.to(DEV)
    bt, sl = cache.block_table.to(DEV), cache.seqlen_k.to(DEV)
    max_pages = b * bt.shape[1]
    lib = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    # regular pair with caller-owned workspaces
    lse_acc = torch.empty(b, hq, num_splits, 1, dtype=torch.float32, device=DEV)
    o_acc = torch.empty(b, hq, num_splits, 1, d, dtype=torch.float32, device=DEV)
    o_ref = torch.empty(b, 1, hq, d, dtype=dtype, device=DEV)
    lse_ref = torch.empty(b, hq, 1, dtype=torch.float32, device=DEV)
    _lib.check(lib.FmhaFwdSplitKV(_p(q), _p(k), _p(v), None, _p(lse_acc), _p(o_acc), None, None, _p(sl), _p(bt), None,
                                  b, 1, 0, hq, hkv, d, d, 1, num_splits, max_pages, page, 0.0, -1, -1, 0, stream,
                                  _lib.BFLOAT16), "FmhaFwdSplitKV")
    _lib.check(lib.FmhaFwdSplitKVCombine(_p(lse_acc), _p(o_acc), _p(o_ref), None, b, 1, hq, d, 1, num_splits, stream,
                                         _p(lse_ref), _lib.BFLOAT16), "FmhaFwdSplitKVCombine")
    # the entry point under test: no workspace arguments at all
    o = torch.empty_like(o_ref)
    lse = torch.empty_like(lse_ref)
    _lib.check(lib.FmhaFwdSplitKVStatic(_p(q), _p(k), _p(v), _p(o), _p(lse), None, None, _p(sl), _p(bt), None, b, 1, 0,
                                        hq, hkv, d, d, 1, num_splits, max_pages, page, 0.0, -1, -1, 0, stream,
                                        _lib.BFLOAT16), "FmhaFwdSplitKVStatic")
    torch.cuda.synchronize()
    return o, lse, o_ref, lse_ref


def test_static_scratch_matches_regular_entry_points_twice_in_a_row():
    # first call: larger problem, fills much of the array
    o, lse, o_ref, lse_ref = _run_both([1500, 17, 4096, 0, 333, 2049], 32, 8, num_splits=6, seed=21)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)
    # second call: different, smaller problem reusing the array as the first call left it
    o, lse, o_ref, lse_ref = _run_both([64, 900, 5], 16, 8, num_splits=3, seed=22)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)
    assert _lib.device_status() == 0


def test_static_scratch_rejects_oversized_problems():
    lib = _lib.lib()
    dummy = torch.zeros(16, dtype=torch.bfloat16, device=DEV)
    # 512 sequences x 64 heads x 128 splits x (128 + 1) floats is far beyond 16 MiB
    rc = lib.FmhaFwdSplitKVStatic(_p(dummy), _p(dummy), _p(dummy), _p(dummy), None, None, None, _p(dummy), _p(dummy),
                                  None, 512, 1, 0, 64, 8, 128, 128, 1, 128, 512, 16, 0.0, -1, -1, 0, None,
                                  _lib.BFLOAT16)
    assert rc == 2
    msg = lib.FlashckGetLastError().decode()
    assert "built-in scratch" in msg and "bytes" in msg
    # sizes whose product wraps around 64 bits must not slip under the capacity check (they are refused before any
    # CUDA call, so the dummy pointers are never touched)
    rc = lib.FmhaFwdSplitKVStatic(_p(dummy), _p(dummy), _p(dummy), _p(dummy), None, None, None, _p(dummy), _p(dummy),
                                  None, 1 << 30, 1 << 30, 0, 1 << 30, 8, 128, 128, 1, 1024, 1 << 30, 16, 0.0, -1, -1, 0,
                                  None, _lib.BFLOAT16)
    assert rc in (1, 2)
    rc = lib.FmhaFwdSplitKVStatic(_p(dummy), _p(dummy), _p(dummy), _p(dummy), None, None, None, _p(dummy), _p(dummy),
                                  None, 1 << 40, 1, 0, 64, 8, 128, 128, 1, 4, 1 << 40, 16, 0.0, -1, -1, 0, None,
                                  _lib.BFLOAT16)
    assert rc == 1


def test_static_scratch_group_mode_and_contiguous_cache():
    """The same comparison for the two other forms the entry point takes: packed multi-token queries (q_seq_start,
    causal, served by the tcgen05 split instance) over a paged cache, and a contiguous cache in batch mode."""
    from flashck_b200.utils.inputs import to_seqstarts
    lib = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    d, page, dtype, hq, hkv, S = 128, 16, torch.bfloat16, 16, 4, 4
    # ---- group mode over a paged cache
    lens_k, lens_q = [700, 33, 1290], [9, 1, 16]
    cache = make_paged_cache(lens_k, hkv, d, d, page, dtype, seed=31)
    cu = to_seqstarts(lens_q).to(DEV)
    total = sum(lens_q)
    q = normal_tensor((total, hq, d), dtype, 32).to(DEV)
    k, v = cache.k.to(DEV), cache.v.to(DEV)
    bt, sl = cache.block_table.to(DEV), cache.seqlen_k.to(DEV)
    b, max_pages = len(lens_k), len(lens_k) * bt.shape[1]
    lse_acc = torch.empty(1, hq, S, total, dtype=torch.float32, device=DEV)
    o_acc = torch.empty(1, hq, S, total, d, dtype=torch.float32, device=DEV)
    o_ref = torch.empty(total, hq, d, dtype=dtype, device=DEV)
    lse_ref = torch.empty(hq, total, dtype=torch.float32, device=DEV)
    _lib.check(lib.FmhaFwdSplitKV(_p(q), _p(k), _p(v), None, _p(lse_acc), _p(o_acc), _p(cu), None, _p(sl), _p(bt), None,
                                  b, total, 0, hq, hkv, d, d, max(lens_q), S, max_pages, page, 0.0, -1, 0, 2, stream,
                                  _lib.BFLOAT16), "FmhaFwdSplitKV")
    _lib.check(lib.FmhaFwdSplitKVCombine(_p(lse_acc), _p(o_acc), _p(o_ref), _p(cu), b, total, hq, d, max(lens_q), S,
                                         stream, _p(lse_ref), _lib.BFLOAT16), "FmhaFwdSplitKVCombine")
    o, lse = torch.empty_like(o_ref), torch.empty_like(lse_ref)
    _lib.check(lib.FmhaFwdSplitKVStatic(_p(q), _p(k), _p(v), _p(o), _p(lse), _p(cu), None, _p(sl), _p(bt), None, b, total,
                                        0, hq, hkv, d, d, max(lens_q), S, max_pages, page, 0.0, -1, 0, 2, stream,
                                        _lib.BFLOAT16), "FmhaFwdSplitKVStatic")
    torch.cuda.synchronize()
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)
    # ---- batch mode over a contiguous cache [b, capacity, hkv, d] with per-sequence lengths
    b, cap = 3, 640
    kc = normal_tensor((b, cap, hkv, d), dtype, 41).to(DEV)
    vc = normal_tensor((b, cap, hkv, d), dtype, 42).to(DEV)
    sl = torch.tensor([640, 1, 377], dtype=torch.int32, device=DEV)
    q = normal_tensor((b, 1, hq, d), dtype, 43).to(DEV)
    lse_acc = torch.empty(b, hq, S, 1, dtype=torch.float32, device=DEV)
    o_acc = torch.empty(b, hq, S, 1, d, dtype=torch.float32, device=DEV)
    o_ref = torch.empty(b, 1, hq, d, dtype=dtype, device=DEV)
    lse_ref = torch.empty(b, hq, 1, dtype=torch.float32, device=DEV)
    _lib.check(lib.FmhaFwdSplitKV(_p(q), _p(kc), _p(vc), None, _p(lse_acc), _p(o_acc), None, None, _p(sl), None, None,
                                  b, 1, cap, hq, hkv, d, d, 1, S, 0, 0, 0.0, -1, -1, 0, stream, _lib.BFLOAT16),
               "FmhaFwdSplitKV")
    _lib.check(lib.FmhaFwdSplitKVCombine(_p(lse_acc), _p(o_acc), _p(o_ref), None, b, 1, hq, d, 1, S, stream,
                                         _p(lse_ref), _lib.BFLOAT16), "FmhaFwdSplitKVCombine")
    o, lse = torch.empty_like(o_ref), torch.empty_like(lse_ref)
    _lib.check(lib.FmhaFwdSplitKVStatic(_p(q), _p(kc), _p(vc), _p(o), _p(lse), None, None, _p(sl), None, None, b, 1, cap,
                                        hq, hkv, d, d, 1, S, 0, 0, 0.0, -1, -1, 0, stream, _lib.BFLOAT16),
               "FmhaFwdSplitKVStatic")
    torch.cuda.synchronize()
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)
    assert _lib.device_status() == 0
