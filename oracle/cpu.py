"""TEST INFRASTRUCTURE ONLY -- ctypes front end of the CPU oracle (``liboracle.so``).

PARITY UNPINNED: the reference holds no golden vectors for its attention path (see the
header of ``fmha_oracle.cpp``).  Only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import this module.
All tensors are CPU torch tensors; fp16/bf16 payloads cross the boundary as raw 16-bit words.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB: Optional[ctypes.CDLL] = None

FLOAT8, BFLOAT8, FLOAT16, BFLOAT16 = 1, 2, 3, 4  # core/utils/dtype.h:16-28


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file (make rebuilds what is older than its source); returns
    the library path."""
    path = os.path.join(_HERE, "liboracle.so")
    sources = [os.path.join(_HERE, n) for n in os.listdir(_HERE) if n.endswith(".cpp") or n == "Makefile"]
    stale = not os.path.exists(path) or os.path.getmtime(path) < max(os.path.getmtime(s) for s in sources)
    if force or stale:
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return path


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
    return _LIB


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return FLOAT16
    if t.dtype == torch.bfloat16:
        return BFLOAT16
    raise TypeError(f"oracle supports float16/bfloat16, got {t.dtype}")


def _p(t: Optional[torch.Tensor]):
    if t is None:
        return ctypes.c_void_p(0)
    assert t.device.type == "cpu" and t.is_contiguous()
    return ctypes.c_void_p(t.data_ptr())


def _i64(x):
    return ctypes.c_int64(int(x))


def fmha_fwd(q, k, v, *, seqstart_q=None, seqstart_k=None, seqlen_k=None, block_table=None,
             cache_batch_idx=None, seqlen_q_shape=None, scale=0.0, window=(-1, -1), mask_type=0,
             nthreads=0, bias=None, alibi_slopes=None, logits_soft_cap=0.0):
    """Returns (O, LSE).  Batch mode: q [b,sq,hq,d]; group mode (seqstart_q given): q [total_q,hq,d].
    LSE is [b,hq,sq] (batch) or [hq,total_q] (group).  bias: [1|b, 1|hq, sq, sk] in q's dtype (group mode: the packed
    totals); alibi_slopes: fp32 [1|b, hq]."""
    dt = _dt(q)
    group = seqstart_q is not None
    paged = block_table is not None
    if group:
        batch = seqstart_q.numel() - 1
        total_q, hq, d = q.shape
        sq = 0
    else:
        batch, sq, hq, d = q.shape
        total_q = batch * sq
    hkv, dv = k.shape[-2], v.shape[-1]
    if paged:
        page = k.shape[1]
        bt_stride = block_table.shape[1]
        sk = 0
    else:
        page, bt_stride = 0, 0
        sk = k.shape[1] if k.dim() == 4 else k.shape[0]  # (group mode: the packed total, the row length of a bias)
    o = torch.empty(q.shape[:-1] + (dv,), dtype=q.dtype)
    lse = torch.empty((hq, total_q) if group else (batch, hq, sq), dtype=torch.float32)
    if seqlen_k is not None:
        seqlen_k = seqlen_k.to(torch.int32).contiguous()
    bias_enum, rank, bias_buf = 0, 0, None
    if bias is not None:
        assert alibi_slopes is None and bias.dim() == 4 and bias.dtype == q.dtype
        bias_enum, bias_buf = 1, bias
        rank = 0 if bias.shape[0] == 1 and bias.shape[1] == 1 else (1 if bias.shape[0] == 1 else 2)
    elif alibi_slopes is not None:
        assert alibi_slopes.dim() == 2 and alibi_slopes.dtype == torch.float32
        bias_enum, bias_buf, rank = 2, alibi_slopes, (0 if alibi_slopes.shape[0] == 1 else 1)
    rc = lib().oracle_fmha_fwd_bias(
        _p(q), _p(k), _p(v), _p(o), _p(lse), _p(seqstart_q), _p(seqstart_k), _p(seqlen_k), _p(block_table),
        _p(cache_batch_idx), _i64(batch), _i64(sq), _i64(sk), _i64(hq), _i64(hkv), _i64(d), _i64(dv),
        _i64(bt_stride), _i64(page), ctypes.c_float(scale), _i64(window[0]), _i64(window[1]),
        ctypes.c_uint32(mask_type), ctypes.c_int(dt), ctypes.c_int(nthreads), _p(bias_buf), ctypes.c_int(bias_enum),
        ctypes.c_int(rank), ctypes.c_float(logits_soft_cap))
    if rc != 0:
        raise RuntimeError(f"oracle_fmha_fwd failed with status {rc}")
    return o, lse


def splitkv_combine(lse_acc, o_acc, dtype):
    """lse_acc [bs,hq,S,rows], o_acc [bs,hq,S,rows,dv] fp32 -> (O [bs,rows,hq,dv] dtype, LSE [bs,hq,rows])."""
    bs, hq, S, rows, dv = o_acc.shape
    o = torch.empty((bs, rows, hq, dv), dtype=dtype)
    lse = torch.empty((bs, hq, rows), dtype=torch.float32)
    rc = lib().oracle_splitkv_combine(_p(lse_acc), _p(o_acc), _p(o), _p(lse), _i64(bs), _i64(rows), _i64(hq),
                                      _i64(dv), _i64(S), ctypes.c_int(_dt(o)))
    if rc != 0:
        raise RuntimeError(f"oracle_splitkv_combine failed with status {rc}")
    return o, lse


def fmha_fwd_appendkv(q, k_cache, knew, v_cache, vnew, seqlen_k, rotary_cos, rotary_sin, *, rope_type=1,
                      rotary_dim=None, block_table=None, cache_batch_idx=None, seqstart_q=None,
                      seqstart_knew=None):
    """In place: rotates ``q`` and writes rotated ``knew`` / ``vnew`` into the caches."""
    dt = _dt(q)
    group = seqstart_q is not None
    if group:
        batch = seqstart_q.numel() - 1
        sq = n = 0
    else:
        batch, sq = q.shape[0], q.shape[1]
        n = knew.shape[1]
    hq, d = q.shape[-2], q.shape[-1]
    hkv, dv = knew.shape[-2], vnew.shape[-1]
    if rotary_dim is None:
        rotary_dim = 2 * rotary_cos.shape[-1] if rope_type != 0 else 0
    if block_table is not None:
        page, bt_stride, cap = k_cache.shape[1], block_table.shape[1], 0
    else:
        page, bt_stride, cap = 0, 0, k_cache.shape[1]
    rc = lib().oracle_fmha_fwd_appendkv(
        _p(q), _p(k_cache), _p(knew), _p(v_cache), _p(vnew), _p(seqlen_k.to(torch.int32).contiguous()),
        _p(seqstart_q), _p(seqstart_knew), _p(rotary_cos), _p(rotary_sin), _p(block_table), _p(cache_batch_idx),
        _i64(batch), _i64(sq), _i64(cap), _i64(n), _i64(hq), _i64(hkv), _i64(d), _i64(dv), _i64(rotary_dim),
        ctypes.c_int(rope_type), _i64(bt_stride), _i64(page), ctypes.c_int(dt))
    if rc != 0:
        raise RuntimeError(f"oracle_fmha_fwd_appendkv failed with status {rc}")


def num_threads() -> int:
    return int(lib().oracle_num_threads())


_F8 = {torch.float8_e4m3fn: FLOAT8, torch.float8_e5m2: BFLOAT8}
_OUT = {torch.float8_e4m3fn: FLOAT8, torch.float8_e5m2: BFLOAT8, torch.float16: FLOAT16, torch.bfloat16: BFLOAT16}


def f8_to_f32(bits: int, dtype=torch.float8_e4m3fn) -> float:
    fn = lib().oracle_f8_to_f32
    fn.restype = ctypes.c_float
    return float(fn(ctypes.c_uint8(bits), ctypes.c_int(_F8[dtype])))


def f32_to_f8(x: float, dtype=torch.float8_e4m3fn) -> int:
    fn = lib().oracle_f32_to_f8
    fn.restype = ctypes.c_uint8
    return int(fn(ctypes.c_float(x), ctypes.c_int(_F8[dtype])))


def fmha_fwd_fp8(q, k, v, *, scale_s, scale_p=1.0, scale_o=1.0, seqstart_q=None, seqstart_k=None, window=(-1, -1),
                 mask_type=0, out_dtype=None, nthreads=0):
    """8-bit (static-quantisation) forward attention; q/k/v are torch.float8_e4m3fn or float8_e5m2 tensors in BSHD
    (or packed with seqstart arrays).  Returns (O in ``out_dtype`` (default: the input type), LSE fp32)."""
    dt = _F8[q.dtype]
    out_dtype = out_dtype or q.dtype
    group = seqstart_q is not None
    if group:
        batch, sq, sk = seqstart_q.numel() - 1, 0, 0
        total_q, hq, d = q.shape
    else:
        batch, sq, hq, d = q.shape
        sk = k.shape[1]
        total_q = batch * sq
    hkv, dv = k.shape[-2], v.shape[-1]
    o = torch.empty(q.shape[:-1] + (dv,), dtype=out_dtype)
    lse = torch.empty((hq, total_q) if group else (batch, hq, sq), dtype=torch.float32)
    rc = lib().oracle_fmha_fwd_fp8(
        _p(q), _p(k), _p(v), _p(o), _p(lse), _p(seqstart_q), _p(seqstart_k), _i64(batch), _i64(sq), _i64(sk), _i64(hq),
        _i64(hkv), _i64(d), _i64(dv), ctypes.c_float(scale_s), ctypes.c_float(scale_p), ctypes.c_float(scale_o),
        _i64(window[0]), _i64(window[1]), ctypes.c_uint32(mask_type), ctypes.c_int(dt), ctypes.c_int(_OUT[out_dtype]),
        ctypes.c_int(nthreads))
    if rc != 0:
        raise RuntimeError(f"oracle_fmha_fwd_fp8 failed with status {rc}")
    return o, lse
