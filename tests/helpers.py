"""Shared comparison helpers.  Tolerances are the ones the task states for this path: O within 2e-2 abs/rel of
the fp32-accumulated reference (it equals the reference's fp16 trait, tests/pytorch/common/test_framework.py:12),
LSE within 1e-3, cache writes bit-exact."""
import torch

O_ATOL = O_RTOL = 2e-2
LSE_ATOL = 1e-3


def assert_o_close(got, ref, what="O"):
    got, ref = got.float().cpu(), ref.float().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    if torch.isfinite(ref).all():
        assert torch.isfinite(got).all(), f"{what}: {int((~torch.isfinite(got)).sum())} of {got.numel()} values are NaN or Inf"
    err = (got - ref).abs()
    bound = O_ATOL + O_RTOL * ref.abs()
    bad = ~(err <= bound)  # written as a negation so that a NaN error counts as a failure
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} outside 2e-2 abs/rel, max err {float(err[~torch.isnan(err)].max()) if (~torch.isnan(err)).any() else float('nan'):.4g}"


def assert_lse_close(got, ref, what="LSE"):
    got, ref = got.float().cpu(), ref.float().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    inf_g, inf_r = torch.isinf(got), torch.isinf(ref)
    assert torch.equal(inf_g, inf_r), f"{what}: -inf pattern differs"
    assert not torch.isnan(got).any(), f"{what}: {int(torch.isnan(got).sum())} NaN values"
    if (~inf_r).any():
        err = (got[~inf_r] - ref[~inf_r]).abs().max()
        assert bool(err <= LSE_ATOL), f"{what}: max err {float(err):.4g} > 1e-3"


def assert_bits_equal(got, ref, what="cache"):
    g = got.cpu().contiguous().view(torch.int16)
    r = ref.cpu().contiguous().view(torch.int16)
    assert g.shape == r.shape
    diff = g != r
    assert not diff.any(), f"{what}: {int(diff.sum())} of {diff.numel()} 16-bit words differ"
