"""Host-side logic that needs no GPU: registry, enums, input generators, argument validation in the Python API."""
import pytest
import torch

import flashck_b200
from flashck_b200 import ops
from flashck_b200.ops.fmha import _mask, default_num_splits
from flashck_b200.utils import FlashCKOperationType, MaskEnum, RopeEnum, get_operation_function, is_available
from flashck_b200.utils.inputs import iota_shuffle, make_paged_cache, rotary_cos_sin, to_seqstarts, uniform_seqlens


def test_registry_fills_the_fmha_slot():
    assert FlashCKOperationType.FMHA.value == "fmha"
    assert is_available("fmha") and is_available()
    assert not is_available("gemm")
    assert get_operation_function("fmha", "forward") is flashck_b200.fmha_fwd
    assert get_operation_function("fmha", "append_kv") is flashck_b200.fmha_fwd_append_kv
    assert get_operation_function("fmha", "nope") is None


def test_enum_values_follow_the_reference():
    assert [int(m) for m in MaskEnum] == [0, 1, 2, 3]
    assert int(RopeEnum.INTERLEAVED) == 1 and int(RopeEnum.HALF_ROTATED) == 2
    assert int(flashck_b200.utils.DataType.FLOAT16) == 3 and int(flashck_b200.utils.DataType.BFLOAT16) == 4


def test_mask_resolution():
    assert _mask(False, (-1, -1), None) == (0, -1, -1)
    assert _mask(True, (-1, -1), None) == (2, -1, 0)
    assert _mask(True, (128, -1), None) == (2, 128, 0)
    assert _mask(False, (4, 4), None) == (2, 4, 4)
    assert _mask(False, (-1, 0), 1) == (1, -1, 0)


def test_default_num_splits():
    assert default_num_splits(64) == 6
    assert default_num_splits(4) == 75
    assert default_num_splits(100000) == 2
    assert default_num_splits(1) == 128
    assert default_num_splits(32, rows_per_kv_head=64) == 16   # many query rows: tcgen05 instance, pieces as splits
    assert default_num_splits(32, rows_per_kv_head=16) == default_num_splits(32)


def test_input_generators():
    assert to_seqstarts([3, 0, 5]).tolist() == [0, 3, 3, 8] and to_seqstarts([1]).dtype == torch.int64
    a, b = uniform_seqlens(16, 512, 4096, 1), uniform_seqlens(16, 512, 4096, 1)
    assert a == b and min(a) >= 512 and max(a) <= 4096
    p = iota_shuffle(100, 3)
    assert sorted(p.tolist()) == list(range(100)) and p.dtype == torch.int32 and p.tolist() != list(range(100))
    cache = make_paged_cache([5, 33, 0], 2, 64, 64, 16, torch.bfloat16, seed=1, capacity=[20, 33, 1])
    assert cache.k.shape == (2 + 3 + 1, 16, 2, 64) and cache.block_table.shape == (3, 3)
    used = cache.block_table[cache.block_table >= 0]
    assert sorted(used.tolist()) == list(range(6))
    cos, sin = rotary_cos_sin(10, 8, torch.float32)
    assert cos.shape == (10, 4) and torch.allclose(cos[0], torch.ones(4)) and torch.allclose(sin[0], torch.zeros(4))
    assert torch.allclose(cos[3, 1], torch.cos(torch.tensor(3.0 * 10000 ** (-2 / 8))))


def test_python_api_rejects_bad_tensors_before_launch():
    q = torch.zeros(1, 4, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        ops.fmha_fwd(q, q, q)
    with pytest.raises(TypeError):
        ops.fmha_fwd("q", q, q)
    with pytest.raises(ValueError, match="rotary"):
        ops.fmha_fwd_append_kv(q, q, q, q, q, torch.zeros(1, dtype=torch.int32))


def test_comparison_helpers_reject_nan_and_inf():
    """The parity helpers must fail on NaN / Inf output (a NaN error compares False against any bound)."""
    from helpers import assert_lse_close, assert_o_close
    ref = torch.ones(4, 8)
    assert_o_close(ref.clone(), ref)
    for bad in (float("nan"), float("inf"), -float("inf")):
        got = ref.clone()
        got[1, 3] = bad
        with pytest.raises(AssertionError):
            assert_o_close(got, ref)
    with pytest.raises(AssertionError):
        assert_o_close(torch.full_like(ref, float("nan")), ref)
    with pytest.raises(AssertionError):
        assert_o_close(ref + 0.5, ref)
    lse = torch.tensor([0.5, -float("inf"), 2.0])
    assert_lse_close(lse.clone(), lse)
    with pytest.raises(AssertionError):
        assert_lse_close(torch.tensor([0.5, -float("inf"), float("nan")]), lse)
    with pytest.raises(AssertionError):
        assert_lse_close(torch.tensor([0.5, 1.0, 2.0]), lse)
    with pytest.raises(AssertionError):
        assert_lse_close(torch.tensor([0.5, -float("inf"), 2.002]), lse)
