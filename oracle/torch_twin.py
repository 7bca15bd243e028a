"""TEST INFRASTRUCTURE ONLY -- an independent PyTorch fp32 statement of the same attention math.

It exists to cross-check the C++ oracle (two implementations that share no code).  It follows
the same conventions (see ``fmha_oracle.cpp``) except that the probabilities are *not* rounded
to the input dtype before the second GEMM, so it agrees with the oracle to rounding noise of
the 16-bit P (a few 1e-3), not bit for bit.
"""
from __future__ import annotations

import math

import torch


def visible_mask(sq: int, sk: int, mask_type: int, window=(-1, -1)) -> torch.Tensor:
    """Boolean [sq, sk]: True where query i may see key j (fmha_library.h:81-87 window rules)."""
    if mask_type == 0:
        return torch.ones(sq, sk, dtype=torch.bool)
    shift = sk - sq if mask_type == 2 else 0
    i = torch.arange(sq)[:, None] + shift
    j = torch.arange(sk)[None, :]
    ok = torch.ones(sq, sk, dtype=torch.bool)
    if window[0] >= 0:
        ok &= j >= i - window[0]
    if window[1] >= 0:
        ok &= j <= i + window[1]
    return ok


def attend(q, k, v, scale=0.0, mask_type=0, window=(-1, -1), bias=None, alibi_slopes=None, logits_soft_cap=0.0):
    """q [sq,hq,d], k [sk,hkv,d], v [sk,hkv,dv] -> (o [sq,hq,dv] in q.dtype, lse [hq,sq] fp32).
    bias [1|hq, sq, sk] is added to the scaled scores, alibi_slopes [hq] add -slope * |i + sk - sq - j|, a soft cap
    bounds the scaled scores with cap * tanh(score / cap) before either."""
    sq, hq, d = q.shape
    sk, hkv, _ = k.shape
    if scale == 0.0:
        scale = 1.0 / math.sqrt(d)
    ratio = hq // hkv
    qf = q.float().permute(1, 0, 2)                                  # [hq,sq,d]
    kf = k.float().permute(1, 0, 2).repeat_interleave(ratio, dim=0)  # [hq,sk,d]
    vf = v.float().permute(1, 0, 2).repeat_interleave(ratio, dim=0)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    if logits_soft_cap > 0:
        s = logits_soft_cap * torch.tanh(s / logits_soft_cap)
    if bias is not None:
        s = s + bias.float()
    if alibi_slopes is not None:
        dist = (torch.arange(sq)[:, None] + (sk - sq) - torch.arange(sk)[None, :]).abs().float()
        s = s - alibi_slopes.float()[:, None, None] * dist[None]
    s = s.masked_fill(~visible_mask(sq, sk, mask_type, window)[None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    p = torch.nan_to_num(p, nan=0.0)  # fully masked rows: exp(-inf - -inf)
    o = torch.matmul(p, vf).permute(1, 0, 2).to(q.dtype)
    return o, lse


def gather_paged(pool, block_table_row, length):
    """pool [pages,page,h,d], one block-table row -> [length,h,d]."""
    page = pool.shape[1]
    npages = -(-length // page)
    idx = block_table_row[:npages].long()
    return pool[idx].reshape(npages * page, *pool.shape[2:])[:length]


def combine(lse_acc, o_acc, dtype):
    """lse_acc [bs,hq,S,rows], o_acc [bs,hq,S,rows,dv] -> (O [bs,rows,hq,dv], LSE [bs,hq,rows])."""
    lse = torch.logsumexp(lse_acc, dim=2)
    w = torch.exp(lse_acc - lse[:, :, None, :])
    w = torch.nan_to_num(w, nan=0.0)
    o = (w[..., None] * torch.nan_to_num(o_acc, nan=0.0, posinf=0.0, neginf=0.0)).sum(dim=2)
    return o.permute(0, 2, 1, 3).contiguous().to(dtype), lse


def rope(x, cos, sin, rope_type):
    """x [..., d] with per-row cos/sin [..., rotary_dim/2] broadcastable; fp32 math without FMA
    contraction is not guaranteed here, so this twin is compared to tolerance, not bits."""
    if rope_type == 0:
        return x.clone()
    half = cos.shape[-1]
    r = 2 * half
    xf = x.float()
    c, s = cos.float(), sin.float()
    out = xf.clone()
    if rope_type == 1:
        x0, x1 = xf[..., 0:r:2], xf[..., 1:r:2]
        out[..., 0:r:2] = x0 * c - x1 * s
        out[..., 1:r:2] = x0 * s + x1 * c
    else:
        x0, x1 = xf[..., :half], xf[..., half:r]
        out[..., :half] = x0 * c - x1 * s
        out[..., half:r] = x0 * s + x1 * c
    return out.to(x.dtype)
