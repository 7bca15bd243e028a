"""CPU tests of the oracle: against an independent PyTorch fp32 statement of the same math, against numpy's
16-bit conversions, and against the committed golden fixtures."""
import importlib.util
import os

import numpy as np
import pytest
import torch

from flashck_b200.utils.inputs import make_paged_cache, normal_tensor, rotary_cos_sin, to_seqstarts
from oracle import cpu as oracle
from oracle import torch_twin as twin
from helpers import assert_lse_close, assert_o_close

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load_gen():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("mask", [(0, -1, -1), (1, -1, 0), (2, -1, 0), (1, 16, 0), (2, 7, 3), (3, 5, 5)])
@pytest.mark.parametrize("sq,sk", [(128, 128), (3, 77), (40, 9)])
def test_oracle_matches_torch_twin(dtype, mask, sq, sk):
    b, hq, hkv, d = 2, 4, 2, 64
    q = normal_tensor((b, sq, hq, d), dtype, 1)
    k = normal_tensor((b, sk, hkv, d), dtype, 2)
    v = normal_tensor((b, sk, hkv, d), dtype, 3)
    mt, wl, wr = mask
    o, lse = oracle.fmha_fwd(q, k, v, mask_type=mt, window=(wl, wr))
    for bi in range(b):
        o2, l2 = twin.attend(q[bi], k[bi], v[bi], mask_type=mt, window=(wl, wr))
        assert torch.allclose(o[bi].float(), o2.float(), atol=1e-2, rtol=1e-2)
        fin = ~torch.isinf(l2)
        assert torch.equal(torch.isinf(lse[bi]), torch.isinf(l2))
        assert torch.allclose(lse[bi][fin], l2[fin], atol=1e-4, rtol=1e-5)


@pytest.mark.parametrize("kind", ["bias0", "bias1", "bias2", "alibi0", "alibi1", "softcap", "softcap+alibi"])
def test_oracle_bias_alibi_softcap_match_twin(kind):
    """The score additions of the reference's instance schema (bias_enum / bias_rank_info / has_logits_soft_cap):
    both statements of the math agree, in batch mode for every rank of the bias."""
    dtype = torch.bfloat16
    b, sq, sk, hq, hkv, d = 2, 37, 70, 4, 2, 64
    q, k, v = (normal_tensor(sh, dtype, sd) for sh, sd in (((b, sq, hq, d), 1), ((b, sk, hkv, d), 2), ((b, sk, hkv, d), 3)))
    bias = slopes = None
    cap = 0.0
    if kind.startswith("bias"):
        rank = int(kind[-1])
        bias = normal_tensor(((1, 1), (1, hq), (b, hq))[rank] + (sq, sk), dtype, 4)
    if "alibi" in kind:
        slopes = torch.rand((b if kind.endswith("1") else 1, hq), generator=torch.Generator().manual_seed(5)) * 0.5
    if "softcap" in kind:
        cap = 1.5
    o, lse = oracle.fmha_fwd(q, k, v, mask_type=2, window=(-1, 0), bias=bias, alibi_slopes=slopes, logits_soft_cap=cap)
    for bi in range(b):
        bb = None if bias is None else bias[bi if bias.shape[0] > 1 else 0]
        ss = None if slopes is None else slopes[bi if slopes.shape[0] > 1 else 0]
        o2, l2 = twin.attend(q[bi], k[bi], v[bi], mask_type=2, window=(-1, 0), bias=bb, alibi_slopes=ss,
                             logits_soft_cap=cap)
        assert_o_close(o[bi], o2, kind)
        assert_lse_close(lse[bi], l2, kind)


def test_oracle_group_mode_bias_uses_the_block_of_each_sequence():
    """Group mode: one [1, hq, total_q, total_k] plane; sequence b reads rows seqstart_q[b].. and keys seqstart_k[b].."""
    dtype = torch.float16
    hq, hkv, d = 4, 4, 64
    lens_q, lens_k = [5, 33, 17], [40, 33, 90]
    cu_q, cu_k = to_seqstarts(lens_q), to_seqstarts(lens_k)
    tq, tk = int(cu_q[-1]), int(cu_k[-1])
    q, k, v = normal_tensor((tq, hq, d), dtype, 11), normal_tensor((tk, hkv, d), dtype, 12), normal_tensor((tk, hkv, d), dtype, 13)
    bias = normal_tensor((1, hq, tq, tk), dtype, 14)
    o, lse = oracle.fmha_fwd(q, k, v, seqstart_q=cu_q, seqstart_k=cu_k, bias=bias)
    for bi in range(len(lens_q)):
        qs, ks = slice(int(cu_q[bi]), int(cu_q[bi + 1])), slice(int(cu_k[bi]), int(cu_k[bi + 1]))
        o2, l2 = twin.attend(q[qs], k[ks], v[ks], bias=bias[0, :, qs, ks])
        assert_o_close(o[qs], o2)
        assert_lse_close(lse[:, qs], l2)


def test_oracle_paged_group_mode_matches_twin():
    lens, qs = [5, 130, 17, 64, 0], [3, 1, 2, 4, 2]
    hq, hkv, d = 8, 2, 128
    cache = make_paged_cache(lens, hkv, d, d, 16, torch.bfloat16, 7)
    cu = to_seqstarts(qs)
    q = normal_tensor((sum(qs), hq, d), torch.bfloat16, 9)
    o, lse = oracle.fmha_fwd(q, cache.k, cache.v, seqstart_q=cu, seqlen_k=cache.seqlen_k,
                             block_table=cache.block_table, mask_type=2, window=(-1, 0))
    for bi, n in enumerate(lens):
        sl = slice(int(cu[bi]), int(cu[bi + 1]))
        if n == 0:
            assert torch.all(o[sl] == 0) and torch.all(torch.isinf(lse[:, sl]))
            continue
        kk = twin.gather_paged(cache.k, cache.block_table[bi], n)
        vv = twin.gather_paged(cache.v, cache.block_table[bi], n)
        o2, l2 = twin.attend(q[sl], kk, vv, mask_type=2, window=(-1, 0))
        assert torch.allclose(o[sl].float(), o2.float(), atol=1e-2, rtol=1e-2)
        assert torch.allclose(lse[:, sl], l2, atol=1e-4)


def test_oracle_combine_matches_twin_and_split_identity():
    torch.manual_seed(0)
    la = torch.randn(2, 4, 5, 3)
    la[0, 0, 2, :] = float("-inf")
    la[1, 1, :, 1] = float("-inf")
    oa = torch.randn(2, 4, 5, 3, 64)
    o, lse = oracle.splitkv_combine(la, oa, torch.bfloat16)
    o2, l2 = twin.combine(la, oa, torch.bfloat16)
    assert torch.allclose(o.float(), o2.float(), atol=1e-2, rtol=1e-2)
    assert torch.equal(torch.isinf(lse), torch.isinf(l2))
    assert torch.allclose(lse[~torch.isinf(lse)], l2[~torch.isinf(l2)], atol=1e-5)
    # attention over a key range == combine of attention over its two halves
    q = normal_tensor((1, 1, 2, 64), torch.bfloat16, 5)
    k = normal_tensor((1, 96, 2, 64), torch.bfloat16, 6)
    v = normal_tensor((1, 96, 2, 64), torch.bfloat16, 7)
    o_full, lse_full = oracle.fmha_fwd(q, k, v)
    parts = [oracle.fmha_fwd(q, k[:, a:b].contiguous(), v[:, a:b].contiguous()) for a, b in ((0, 40), (40, 96))]
    la = torch.stack([p[1] for p in parts], dim=2)                               # [b,hq,S,sq]
    oa = torch.stack([p[0].float().permute(0, 2, 1, 3) for p in parts], dim=2)   # [b,hq,S,sq,dv]
    o_c, lse_c = oracle.splitkv_combine(la.contiguous(), oa.contiguous(), torch.bfloat16)
    assert torch.allclose(o_c.float(), o_full.float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(lse_c, lse_full, atol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rope", [1, 2])
def test_oracle_appendkv_matches_twin(dtype, rope):
    lens, new = [0, 5, 16, 31], [3, 16, 1, 2]
    cap = [a + b for a, b in zip(lens, new)]
    hq, hkv, d = 4, 2, 64
    cache = make_paged_cache(lens, hkv, d, d, 16, dtype, seed=12, capacity=cap)
    cu = to_seqstarts(new)
    total = int(cu[-1])
    q = normal_tensor((total, hq, d), dtype, 81)
    knew = normal_tensor((total, hkv, d), dtype, 82)
    vnew = normal_tensor((total, hkv, d), dtype, 83)
    cos, sin = rotary_cos_sin(max(cap) + 1, d, dtype)
    q2, k2, v2 = q.clone(), cache.k.clone(), cache.v.clone()
    oracle.fmha_fwd_appendkv(q2, k2, knew, v2, vnew, cache.seqlen_k, cos, sin, rope_type=rope,
                             block_table=cache.block_table, seqstart_q=cu, seqstart_knew=cu)
    untouched = torch.ones(k2.shape[:2], dtype=torch.bool)
    for b, (L, n) in enumerate(zip(lens, new)):
        for j in range(n):
            pos = L + j
            pg, off = int(cache.block_table[b, pos // 16]), pos % 16
            t = int(cu[b]) + j
            want_k = twin.rope(knew[t], cos[pos], sin[pos], rope)
            assert torch.allclose(k2[pg, off].float(), want_k.float(), atol=2e-2, rtol=2e-2)
            assert torch.equal(v2[pg, off], vnew[t])
            want_q = twin.rope(q[t], cos[pos], sin[pos], rope)  # sq == n, so q pos == k pos
            assert torch.allclose(q2[t].float(), want_q.float(), atol=2e-2, rtol=2e-2)
            untouched[pg, off] = False
    assert torch.equal(k2[untouched], cache.k[untouched]) and torch.equal(v2[untouched], cache.v[untouched])


def test_oracle_16bit_conversions_match_torch():
    # bf16 / fp16 round trips inside the oracle use hand-written RNE; compare with torch's casts through a
    # problem whose output is just a cast: one key, so P == 1 and O == V exactly, LSE == scaled dot product.
    for dtype in (torch.float16, torch.bfloat16):
        v = normal_tensor((1, 1, 1, 64), dtype, 3) * 37.0
        q = normal_tensor((1, 5, 1, 64), dtype, 4)
        k = normal_tensor((1, 1, 1, 64), dtype, 5)
        o, lse = oracle.fmha_fwd(q, k, v.to(dtype), scale=1.0)
        assert torch.equal(o, v.to(dtype).expand(1, 5, 1, 64))
        want = (q.float() * k.float()).sum(-1).permute(0, 2, 1)
        assert torch.allclose(lse, want, atol=1e-4, rtol=1e-5)


def test_golden_fixtures():
    gen = _load_gen()
    g = np.load(os.path.join(GOLDEN, "config1_fp16_causal.npz"))
    q, k, v = gen.case_config1()
    o, lse = oracle.fmha_fwd(q, k, v, scale=0.125, mask_type=1, window=(-1, 0))
    assert np.array_equal(gen.words(o), g["o"]) and np.allclose(lse.numpy(), g["lse"], atol=1e-6)

    g = np.load(os.path.join(GOLDEN, "paged_decode_bf16.npz"))
    q, cache = gen.case_paged_decode()
    o, lse = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
    assert np.array_equal(gen.words(o), g["o"]) and np.allclose(lse.numpy(), g["lse"], atol=1e-6)

    g = np.load(os.path.join(GOLDEN, "appendkv_bf16_interleaved.npz"))
    q, knew, vnew, cache, cu, cos, sin = gen.case_append()
    oracle.fmha_fwd_appendkv(q, cache.k, knew, cache.v, vnew, cache.seqlen_k, cos, sin, rope_type=1,
                             block_table=cache.block_table, seqstart_q=cu, seqstart_knew=cu)
    assert np.array_equal(gen.words(q), g["q"])
    assert np.array_equal(gen.words(cache.k), g["k"]) and np.array_equal(gen.words(cache.v), g["v"])


# ------------------------------------------------------------------------------------------------
# 8-bit (static quantisation) forward attention
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_fp8_conversions_match_torch(dtype):
    """The oracle's own E4M3 / E5M2 decode and encode (round to nearest even, saturating) against PyTorch's float8 types:
    all 256 codes, and a sweep of magnitudes from the subnormal range to the largest finite value."""
    codes = torch.arange(256, dtype=torch.uint8)
    ref = codes.view(dtype).float()
    mine = torch.tensor([oracle.f8_to_f32(int(c), dtype) for c in codes])
    assert torch.equal(torch.nan_to_num(ref, nan=7e7), torch.nan_to_num(mine, nan=7e7))
    fmax = 448.0 if dtype == torch.float8_e4m3fn else 57344.0
    g = torch.Generator().manual_seed(3)
    xs = torch.cat([torch.randn(500, generator=g) * s for s in (1e-3, 0.05, 1.0, 30.0, fmax / 3)]).clamp(-fmax, fmax)
    want = xs.to(dtype).view(torch.uint8)
    got = torch.tensor([oracle.f32_to_f8(float(x), dtype) for x in xs], dtype=torch.uint8)
    assert torch.equal(got, want)
    assert oracle.f8_to_f32(oracle.f32_to_f8(1e9, dtype), dtype) == fmax  # saturation, not infinity


@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("causal", [False, True])
def test_fp8_oracle_matches_a_torch_statement(dtype, causal):
    """oracle_fmha_fwd_fp8 against the same algorithm written with torch ops (float8 casts for the roundings)."""
    g = torch.Generator().manual_seed(11)
    b, sq, sk, hq, hkv, d = 2, 33, 50, 4, 2, 64
    q = (torch.randn(b, sq, hq, d, generator=g) * 1.5).to(dtype)
    k = (torch.randn(b, sk, hkv, d, generator=g) * 1.5).to(dtype)
    v = (torch.randn(b, sk, hkv, d, generator=g) * 2.0).to(dtype)
    scale_s, scale_p, scale_o = 0.11, 16.0, 1.0 / 16.0
    o, lse = oracle.fmha_fwd_fp8(q, k, v, scale_s=scale_s, scale_p=scale_p, scale_o=scale_o, mask_type=2 if causal else 0,
                                 window=(-1, 0) if causal else (-1, -1), out_dtype=torch.bfloat16)
    qf, kf, vf = q.float(), k.float().repeat_interleave(hq // hkv, dim=2), v.float().repeat_interleave(hq // hkv, dim=2)
    s = torch.einsum("bihd,bjhd->bhij", qf, kf) * scale_s
    if causal:
        i, j = torch.arange(sq)[:, None], torch.arange(sk)[None, :]
        s = s.masked_fill(j > i + sk - sq, float("-inf"))
    m = s.max(dim=-1, keepdim=True).values
    p = torch.exp(s - m)
    l = p.sum(dim=-1)
    p8 = (p * scale_p).to(dtype).float()
    want = scale_o * torch.einsum("bhij,bjhd->bihd", p8, vf) / l.permute(0, 2, 1)[..., None]
    assert torch.allclose(lse, m[..., 0] + torch.log(l), atol=1e-5)
    assert torch.allclose(o.float(), want.to(torch.bfloat16).float(), atol=1e-2, rtol=1e-2)
    # 8-bit output: the same values rounded to the 8-bit type
    o8, _ = oracle.fmha_fwd_fp8(q, k, v, scale_s=scale_s, scale_p=scale_p, scale_o=scale_o, mask_type=2 if causal else 0,
                                window=(-1, 0) if causal else (-1, -1))
    assert o8.dtype == dtype
    diff = (o8.float() - want).abs()
    ulp = want.abs() * (2.0 ** -3 if dtype == torch.float8_e4m3fn else 2.0 ** -2) + 2.0 ** -9
    assert bool((diff <= ulp).all())
