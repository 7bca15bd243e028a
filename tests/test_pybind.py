"""The compiled PyTorch binding `flash_ck` (pybind11 over the C++ operator API over the C ABI): import, surface and
argument errors on CPU; every function against the CPU oracle on the GPU."""
import pytest
import torch

from flashck_b200.utils.inputs import make_paged_cache, normal_tensor, rotary_cos_sin, to_seqstarts
from helpers import assert_bits_equal, assert_lse_close, assert_o_close

DEV = "cuda:0"


def _ext():
    from flashck_b200 import build
    build.build_pybind()
    from flashck_b200 import flash_ck
    return flash_ck


def test_extension_surface_and_errors_without_a_gpu():
    ext = _ext()
    for name in ("fmha_fwd", "fmha_fwd_varlen", "fmha_batch_prefill", "fmha_fwd_paged_kv_prefill", "fmha_fwd_splitkv",
                 "fmha_fwd_appendkv", "get_flag_value", "set_flag_value", "print_all_flags", "print_flag_info"):
        assert callable(getattr(ext, name))
    assert int(ext.MaskEnum.MASK_FROM_BOTTOM_RIGHT) == 2 and int(ext.BiasEnum.ALIBI) == 2 and int(ext.RopeEnum.HALF_ROTATED) == 2
    assert "sm_100a" in ext.version()
    x = torch.zeros(1, 4, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):   # TORCH_CHECK -> RuntimeError, as in the reference
        ext.fmha_fwd(x, x, x)
    with pytest.raises(RuntimeError, match="float16 and bfloat16"):
        ext.fmha_fwd(x.float(), x.float(), x.float())
    # the flag API reaches the package's registry
    old = ext.get_flag_value("FC_TUNING_NUM_REPEATS")
    ext.set_flag_value("FC_TUNING_NUM_REPEATS", "7")
    import flashck_b200 as fck
    assert fck.get_flag_value("FC_TUNING_NUM_REPEATS") == "7"
    ext.set_flag_value("FC_TUNING_NUM_REPEATS", old)
    with pytest.raises(Exception):
        ext.get_flag_value("FC_NO_SUCH_FLAG")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_extension_fmha_fwd_and_varlen_match_the_oracle(dtype):
    from oracle import cpu as oracle
    ext = _ext()
    q = normal_tensor((2, 300, 8, 128), dtype, 1)
    k = normal_tensor((2, 300, 2, 128), dtype, 2)
    v = normal_tensor((2, 300, 2, 128), dtype, 3)
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, mask_type=2, window=(-1, 0))
    o, lse = ext.fmha_fwd(q.to(DEV), k.to(DEV), v.to(DEV), causal=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)
    # score additions through the layer's bias path: ALiBi slopes and a soft cap (hdim 64: the general instance)
    q6, k6, v6 = (normal_tensor((2, 90, 4, 64), dtype, 4 + i) for i in range(3))
    slopes = torch.rand(1, 4, generator=torch.Generator().manual_seed(1)) * 0.3
    o_ref, lse_ref = oracle.fmha_fwd(q6, k6, v6, alibi_slopes=slopes, logits_soft_cap=20.0)
    o, lse = ext.fmha_fwd(q6.to(DEV), k6.to(DEV), v6.to(DEV), alibi_slopes=slopes.to(DEV), logits_soft_cap=20.0)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)
    # varlen
    lens = [200, 1, 513]
    cu = to_seqstarts(lens)
    qp = normal_tensor((sum(lens), 8, 128), dtype, 7)
    kp = normal_tensor((sum(lens), 2, 128), dtype, 8)
    vp = normal_tensor((sum(lens), 2, 128), dtype, 9)
    o_ref, lse_ref = oracle.fmha_fwd(qp, kp, vp, seqstart_q=cu, seqstart_k=cu, mask_type=1, window=(-1, 0))
    o, lse = ext.fmha_fwd_varlen(qp.to(DEV), kp.to(DEV), vp.to(DEV), cu.to(DEV), cu.to(DEV), max(lens), causal=True)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)


@pytest.mark.gpu
def test_extension_paged_prefill_splitkv_and_appendkv_match_the_oracle():
    from oracle import cpu as oracle
    ext = _ext()
    dtype, hq, hkv, d, page = torch.bfloat16, 8, 2, 128, 16
    lens_k, lens_q = [700, 45, 1290], [300, 45, 130]
    cache = make_paged_cache(lens_k, hkv, d, d, page, dtype, seed=5)
    cu = to_seqstarts(lens_q)
    q = normal_tensor((sum(lens_q), hq, d), dtype, 6)
    o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqstart_q=cu, seqlen_k=cache.seqlen_k, block_table=cache.block_table,
                                     mask_type=2, window=(-1, 0))
    k, v, bt, sl = cache.k.to(DEV), cache.v.to(DEV), cache.block_table.to(DEV), cache.seqlen_k.to(DEV)
    o, lse = ext.fmha_fwd_paged_kv_prefill(q.to(DEV), k, v, bt, sl, cu_seqlens_q=cu.to(DEV), max_seqlen_q=max(lens_q))
    assert_o_close(o, o_ref, "paged prefill")
    assert_lse_close(lse, lse_ref, "paged prefill")
    # the same cache as an SGLang-style page list
    npages = [-(-n // page) for n in lens_k]
    indptr = torch.tensor([0] + list(torch.tensor(npages).cumsum(0)), dtype=torch.int32)
    indices = torch.cat([cache.block_table[b, :n] for b, n in enumerate(npages)]).to(torch.int32)
    last = torch.tensor([n - (p - 1) * page for n, p in zip(lens_k, npages)], dtype=torch.int32)
    o, lse = ext.fmha_batch_prefill(q.to(DEV), k, v, cu.to(DEV), indptr.to(DEV), indices.to(DEV), last.to(DEV), max(lens_q))
    assert_o_close(o, o_ref, "batch prefill")
    assert_lse_close(lse, lse_ref, "batch prefill")
    # decode: one token per sequence
    qd = normal_tensor((3, 1, hq, d), dtype, 7)
    o_ref, lse_ref = oracle.fmha_fwd(qd, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
    o, lse = ext.fmha_fwd_splitkv(qd.to(DEV), k, v, seqlen_k=sl, block_table=bt, num_splits=4)
    assert_o_close(o, o_ref, "split-KV")
    assert_lse_close(lse, lse_ref, "split-KV")
    # append two tokens per sequence (interleaved RoPE) into a cache with room, bit-exact against the oracle
    cap = [n + 2 for n in lens_k]
    cache2 = make_paged_cache(lens_k, hkv, d, d, page, dtype, seed=8, capacity=cap)
    qn, kn, vn = (normal_tensor((3, 2, h, d), dtype, 9 + i) for i, h in enumerate((hq, hkv, hkv)))
    cos, sin = rotary_cos_sin(max(cap) + 1, d, dtype)
    q_ref, k_ref, v_ref = qn.clone(), cache2.k.clone(), cache2.v.clone()
    oracle.fmha_fwd_appendkv(q_ref, k_ref, kn, v_ref, vn, cache2.seqlen_k, cos, sin, rope_type=1, block_table=cache2.block_table)
    qd2, kd2, vd2 = qn.to(DEV), cache2.k.to(DEV), cache2.v.to(DEV)
    out = ext.fmha_fwd_appendkv(qd2, kd2, vd2, kn.to(DEV), vn.to(DEV), cache2.seqlen_k.to(DEV), cos.to(DEV), sin.to(DEV), 1,
                                cache2.block_table.to(DEV))
    assert out.data_ptr() == qd2.data_ptr()
    assert_bits_equal(kd2, k_ref, "k cache")
    assert_bits_equal(vd2, v_ref, "v cache")
    assert_bits_equal(qd2, q_ref, "rotated q")
    from flashck_b200 import _lib
    assert _lib.device_status() == 0
