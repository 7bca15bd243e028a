"""8-bit (static quantisation) forward attention on the GPU against the CPU oracle.

Tolerance.  LSE is an fp32 quantity in both (the 8-bit rounding of P does not enter the row sum): 1e-3 as everywhere.
O: the kernel rounds P to 8 bits relative to a running row maximum, the oracle relative to the final one; each rounding
is off by at most half a unit in the last place (relative 2^-4 for E4M3, 2^-3 for E5M2), so the two P8 differ by at most
one unit, and |O - O_ref| <= ulp8 * (scale_o * sum_j P8_j |v_j| / l) elementwise -- the attention of the same weights
over |V|, which the oracle computes too.  An 8-bit O adds half a unit of its own rounding."""
import ctypes

import pytest
import torch

from flashck_b200 import _lib, ops
from flashck_b200.utils.inputs import to_seqstarts
from helpers import assert_lse_close
from oracle import cpu as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ULP = {torch.float8_e4m3fn: 2.0 ** -3, torch.float8_e5m2: 2.0 ** -2}


def _rand8(shape, dtype, seed, std):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype)


def _check(o, o_ref, o_abs, dtype, what):
    o, o_ref, o_abs = o.float().cpu(), o_ref.float(), o_abs.float()
    assert torch.isfinite(o).all(), what
    bound = ULP[dtype] * o_abs + 1e-2
    bad = ~((o - o_ref).abs() <= bound)
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} beyond one 8-bit unit of P, max err {float((o - o_ref).abs().max()):.4g}"


@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("sq,sk,causal", [(1, 77, False), (130, 130, True), (65, 300, True), (257, 64, False)])
def test_fmha_fwd_fp8_batch_mode(dtype, d, sq, sk, causal):
    b, hq, hkv = 2, 4, 2
    q, k, v = _rand8((b, sq, hq, d), dtype, 1, 1.5), _rand8((b, sk, hkv, d), dtype, 2, 1.5), _rand8((b, sk, hkv, d), dtype, 3, 2.0)
    scale_s, scale_p, scale_o = 0.7 / d ** 0.5, 32.0, 1.0 / 32.0
    kw = dict(scale_s=scale_s, scale_p=scale_p, scale_o=scale_o, mask_type=2 if causal else 0,
              window=(-1, 0) if causal else (-1, -1), out_dtype=torch.bfloat16)
    o_ref, lse_ref = oracle.fmha_fwd_fp8(q, k, v, **kw)
    o_abs, _ = oracle.fmha_fwd_fp8(q, k, v.float().abs().to(dtype), **kw)
    o, lse = ops.fmha_fwd_fp8(q.to(DEV), k.to(DEV), v.to(DEV), scale_s=scale_s, scale_p=scale_p, scale_o=scale_o,
                              causal=causal, out_dtype=torch.bfloat16, return_lse=True)
    _check(o, o_ref, o_abs, dtype, "bf16 output")
    assert_lse_close(lse, lse_ref)
    # 8-bit output: one more rounding, to the type of O
    o8 = ops.fmha_fwd_fp8(q.to(DEV), k.to(DEV), v.to(DEV), scale_s=scale_s, scale_p=scale_p, scale_o=scale_o, causal=causal)
    assert o8.dtype == dtype
    o8f, rf = o8.float().cpu(), o_ref.float()
    assert torch.isfinite(o8f).all()
    assert bool(((o8f - rf).abs() <= ULP[dtype] * o_abs.float() + 0.5 * ULP[dtype] * rf.abs() + 2e-2).all())
    assert _lib.device_status() == 0


def test_fmha_fwd_fp8_group_mode_quantised_from_bf16_and_through_fmha_fwd():
    """Packed sequences, GQA 4:1, hdim 128, tensors quantised from bf16 with quantize_fp8; the result de-quantises to the
    16-bit attention of the same inputs within 8-bit accuracy; and FmhaFwd with the 8-bit dtype code is the same kernel
    with scale_p = scale_o = 1."""
    dtype, hq, hkv, d = torch.float8_e4m3fn, 8, 2, 128
    lens = [200, 1, 333, 64]
    cu = to_seqstarts(lens)
    g = torch.Generator().manual_seed(5)
    q16, k16, v16 = (torch.randn(sum(lens), h, d, generator=g).to(torch.bfloat16) for h in (hq, hkv, hkv))
    (q8, dq), (k8, dk), (v8, dv_) = (ops.quantize_fp8(t, dtype) for t in (q16, k16, v16))
    scale_s, scale_p = dq * dk / d ** 0.5, 256.0
    scale_o = dv_ / scale_p
    kw = dict(scale_s=scale_s, scale_p=scale_p, scale_o=scale_o, seqstart_q=cu, seqstart_k=cu, mask_type=1, window=(-1, 0),
              out_dtype=torch.bfloat16)
    o_ref, lse_ref = oracle.fmha_fwd_fp8(q8, k8, v8, **kw)
    o_abs, _ = oracle.fmha_fwd_fp8(q8, k8, v8.float().abs().to(dtype), **kw)
    o, lse = ops.fmha_fwd_fp8(q8.to(DEV), k8.to(DEV), v8.to(DEV), scale_s=scale_s, scale_p=scale_p, scale_o=scale_o,
                              cu_seqlens_q=cu.to(DEV), cu_seqlens_k=cu.to(DEV), max_seqlen_q=max(lens), causal=True,
                              out_dtype=torch.bfloat16, return_lse=True)
    _check(o, o_ref, o_abs, dtype, "group mode")
    assert_lse_close(lse, lse_ref)
    # against the 16-bit attention of the unquantised tensors: 8-bit accuracy (a loose, end-to-end sanity bound)
    o16, _ = oracle.fmha_fwd(q16, k16, v16, seqstart_q=cu, seqstart_k=cu, mask_type=1, window=(-1, 0))
    assert float((o.float().cpu() - o16.float()).abs().mean()) < 0.05
    # the reference-shaped symbol with the 8-bit dtype code
    qd, kd, vd, cud = q8.to(DEV), k8.to(DEV), v8.to(DEV), cu.to(DEV)
    o_a = torch.empty(sum(lens), hq, d, dtype=dtype, device=DEV)
    o_b = torch.empty_like(o_a)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    lib = _lib.lib()
    _lib.check(lib.FmhaFwd(P(qd), P(kd), P(vd), None, P(o_a), P(cud), P(cud), None, len(lens), sum(lens), sum(lens), hq, hkv, d,
                           d, max(lens), float(scale_s), -1, 0, 1, stream, None, _lib.FLOAT8), "FmhaFwd")
    _lib.check(lib.FmhaFwdFp8(P(qd), P(kd), P(vd), P(o_b), P(cud), P(cud), len(lens), sum(lens), sum(lens), hq, hkv, d, d,
                              max(lens), float(scale_s), 1.0, 1.0, -1, 0, 1, stream, None, _lib.FLOAT8, _lib.FLOAT8),
               "FmhaFwdFp8")
    torch.cuda.synchronize()
    assert torch.equal(o_a.view(torch.uint8), o_b.view(torch.uint8))
    with pytest.raises(TypeError):
        ops.fmha_fwd_fp8(q16.to(DEV), k16.to(DEV), v16.to(DEV))


def _last_instance():
    return _lib.get_instance_param(0, "last_instance")


@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("b,sq,sk,hq,hkv,mask,window", [
    (2, 300, 300, 4, 2, 0, (-1, -1)),      # several key tiles, paired heads
    (1, 515, 515, 3, 3, 1, (-1, 0)),       # causal, unpaired heads (two row blocks per item)
    (2, 129, 700, 4, 1, 2, (-1, 0)),       # bottom-right causal, sk > sq
    (1, 640, 640, 4, 2, 1, (200, 0)),      # sliding window: the WINDOW instance
])
def test_fmha_fwd_fp8_hdim128_runs_on_the_tcgen05_instance_and_matches_oracle_and_general_instance(dtype, b, sq, sk, hq, hkv, mask, window):
    """hdim 128 with contiguous K/V goes to the kind::f8f6f4 instance (the instance query says so); it agrees with the
    oracle within one 8-bit unit of P and with the general instance, which rounds the same way from half precision."""
    d = 128
    q, k, v = _rand8((b, sq, hq, d), dtype, 11, 1.5), _rand8((b, sk, hkv, d), dtype, 12, 1.5), _rand8((b, sk, hkv, d), dtype, 13, 2.0)
    scale_s, scale_p, scale_o = 0.9 / d ** 0.5, 64.0, 1.0 / 64.0
    kw = dict(scale_s=scale_s, scale_p=scale_p, scale_o=scale_o, mask_type=mask, window=window, out_dtype=torch.bfloat16)
    o_ref, lse_ref = oracle.fmha_fwd_fp8(q, k, v, **kw)
    o_abs, _ = oracle.fmha_fwd_fp8(q, k, v.float().abs().to(dtype), **kw)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    lib = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    code = _lib.FLOAT8 if dtype == torch.float8_e4m3fn else _lib.BFLOAT8

    def run(o_code, o_dtype):
        o = torch.empty(b, sq, hq, d, dtype=o_dtype, device=DEV)
        lse = torch.empty(b, hq, sq, dtype=torch.float32, device=DEV)
        _lib.check(lib.FmhaFwdFp8(P(qd), P(kd), P(vd), P(o), None, None, b, sq, sk, hq, hkv, d, d, sq, float(scale_s),
                                  float(scale_p), float(scale_o), window[0], window[1], mask, stream, P(lse), code, o_code),
                   "FmhaFwdFp8")
        torch.cuda.synchronize()
        return o, lse

    o, lse = run(_lib.BFLOAT16, torch.bfloat16)
    assert _last_instance() == 1
    _check(o, o_ref, o_abs, dtype, "tcgen05 8-bit instance, bf16 output")
    assert_lse_close(lse, lse_ref)
    o8, _ = run(code, dtype)
    o8f, rf = o8.float().cpu(), o_ref.float()
    assert torch.isfinite(o8f).all()
    assert bool(((o8f - rf).abs() <= ULP[dtype] * o_abs.float() + 0.5 * ULP[dtype] * rf.abs() + 2e-2).all())
    oh, _ = run(_lib.FLOAT16, torch.float16)
    _check(oh, o_ref, o_abs, dtype, "tcgen05 8-bit instance, fp16 output")
    _lib.set_instance_param(0, "use_sm100_fp8", 0)
    try:
        o_gen, lse_gen = run(_lib.BFLOAT16, torch.bfloat16)
        assert _last_instance() == 0
    finally:
        _lib.set_instance_param(0, "use_sm100_fp8", 1)
    _check(o, o_gen.float().cpu(), 2 * o_abs, dtype, "tcgen05 against the general instance")
    assert_lse_close(lse, lse_gen)
    assert _lib.device_status() == 0


def test_fmha_fwd_fp8_large_scores_do_not_saturate_p():
    """A key that arrives late and dominates: the running max must follow it at once, or P stretched by scale_p would
    leave the range of the 8-bit format and saturate."""
    dtype, d, sq, sk = torch.float8_e4m3fn, 128, 128, 512
    q, k, v = _rand8((1, sq, 2, d), dtype, 21, 1.0), _rand8((1, sk, 2, d), dtype, 22, 0.5), _rand8((1, sk, 2, d), dtype, 23, 2.0)
    k[0, 300] = (q[0, 5].float() * 3).to(dtype)  # a large dot product with most rows, in the third key tile
    scale_s, scale_p, scale_o = 1.0 / d ** 0.5, 256.0, 1.0 / 256.0
    kw = dict(scale_s=scale_s, scale_p=scale_p, scale_o=scale_o, mask_type=0, window=(-1, -1), out_dtype=torch.bfloat16)
    o_ref, lse_ref = oracle.fmha_fwd_fp8(q, k, v, **kw)
    o_abs, _ = oracle.fmha_fwd_fp8(q, k, v.float().abs().to(dtype), **kw)
    o, lse = ops.fmha_fwd_fp8(q.to(DEV), k.to(DEV), v.to(DEV), scale_s=scale_s, scale_p=scale_p, scale_o=scale_o,
                              out_dtype=torch.bfloat16, return_lse=True)
    assert _last_instance() == 1
    _check(o, o_ref, o_abs, dtype, "dominant late key")
    assert_lse_close(lse, lse_ref)
    assert _lib.device_status() == 0
