"""The attention module and the `flash_ck` alias: host-side behaviour on CPU, module == functional API on the GPU."""
import sys

import pytest
import torch

import flashck_b200
from flashck_b200.nn import FlashAttention
from flashck_b200.utils.inputs import make_paged_cache, normal_tensor, to_seqstarts


def test_module_validates_its_configuration():
    with pytest.raises(ValueError):
        FlashAttention(30, 128, num_kv_heads=8)      # not a multiple
    with pytest.raises(ValueError):
        FlashAttention(8, 0)
    with pytest.raises(ValueError):
        FlashAttention(8, 64, window_size=(1,))
    with pytest.raises(ValueError):
        FlashAttention(8, 64, scale=-1.0)
    m = FlashAttention(32, 128, num_kv_heads=8, causal=True)
    assert "num_kv_heads=8" in repr(m) and not list(m.parameters())


def test_module_rejects_wrong_head_layout_before_any_launch():
    m = FlashAttention(8, 64, num_kv_heads=2)
    q = torch.zeros(1, 4, 8, 32)
    with pytest.raises(ValueError):
        m(q, torch.zeros(1, 4, 2, 32), torch.zeros(1, 4, 2, 32))
    with pytest.raises(ValueError):
        m(torch.zeros(1, 4, 8, 64), torch.zeros(1, 4, 4, 64), torch.zeros(1, 4, 4, 64))
    with pytest.raises(ValueError):   # packed inputs without cu_seqlens
        m(torch.zeros(4, 8, 64), torch.zeros(4, 2, 64), torch.zeros(4, 2, 64))


def test_cpu_tensors_fail_loudly_there_is_no_fallback():
    m = FlashAttention(8, 64, num_kv_heads=2)
    with pytest.raises((RuntimeError, ValueError, TypeError)):
        m(torch.zeros(1, 4, 8, 64, dtype=torch.float16), torch.zeros(1, 4, 2, 64, dtype=torch.float16),
          torch.zeros(1, 4, 2, 64, dtype=torch.float16))


def test_flash_ck_alias_resolves_to_this_package():
    saved = {k: v for k, v in sys.modules.items() if k == "flash_ck" or k.startswith("flash_ck.")}
    try:
        for k in saved:
            del sys.modules[k]
        flashck_b200.install_as_flash_ck()
        import flash_ck
        from flash_ck.nn import FlashAttention as Aliased
        from flash_ck.ops import fmha_fwd, fmha_fwd_var_len  # noqa: F401
        from flash_ck.ops.fmha import batch_prefill  # noqa: F401
        assert flash_ck is flashck_b200 and Aliased is FlashAttention
        assert flash_ck.utils.is_available("fmha") and flash_ck.is_available("fmha")
        # a foreign module of that name is not shadowed silently
        sys.modules["flash_ck"] = sys
        with pytest.raises(RuntimeError):
            flashck_b200.install_as_flash_ck()
        flashck_b200.install_as_flash_ck(force=True)
        assert sys.modules["flash_ck"] is flashck_b200
    finally:
        for k in [k for k in sys.modules if k == "flash_ck" or k.startswith("flash_ck.")]:
            del sys.modules[k]
        sys.modules.update(saved)


@pytest.mark.gpu
def test_module_matches_functional_api_on_gpu():
    from flashck_b200 import ops
    from helpers import assert_bits_equal
    dev = torch.device("cuda:0")
    dtype = torch.bfloat16
    m = FlashAttention(8, 128, num_kv_heads=2, causal=True)
    # dense
    q = normal_tensor((2, 96, 8, 128), dtype, 1).to(dev)
    k = normal_tensor((2, 96, 2, 128), dtype, 2).to(dev)
    v = normal_tensor((2, 96, 2, 128), dtype, 3).to(dev)
    assert_bits_equal(m(q, k, v), ops.fmha_fwd(q, k, v, causal=True))
    # packed
    lens = [33, 200, 7]
    cu = to_seqstarts(lens).to(dev)
    qp = normal_tensor((sum(lens), 8, 128), dtype, 4).to(dev)
    kp = normal_tensor((sum(lens), 2, 128), dtype, 5).to(dev)
    vp = normal_tensor((sum(lens), 2, 128), dtype, 6).to(dev)
    o, lse = m(qp, kp, vp, cu, cu, max(lens), max(lens), return_lse=True)
    o2, lse2 = ops.fmha_fwd_var_len(qp, kp, vp, cu, cu, max(lens), max(lens), causal=True, return_lse=True)
    assert_bits_equal(o, o2)
    assert torch.equal(lse, lse2)
    # paged: one query token per sequence goes to split-KV, long queries to the paged prefill
    cache = make_paged_cache(lens, 2, 128, 128, 16, dtype, seed=9)
    kc, vc, bt, sl = cache.k.to(dev), cache.v.to(dev), cache.block_table.to(dev), cache.seqlen_k.to(dev)
    qd = normal_tensor((len(lens), 1, 8, 128), dtype, 7).to(dev)
    assert_bits_equal(m.forward_paged(qd, kc, vc, bt, sl),
                      ops.fmha_fwd_splitkv(qd, kc, vc, seqlen_k=sl, block_table=bt, causal=True))
    assert_bits_equal(m.forward_paged(qp, kc, vc, bt, sl, cu_seqlens_q=cu, max_seqlen_q=max(lens)),
                      ops.fmha_fwd_paged_kv_prefill(qp, kc, vc, bt, sl, cu_seqlens_q=cu, max_seqlen_q=max(lens), causal=True))
