"""Functional attention API -- the ``flash_ck.ops`` surface for the FMHA family.

The reference reserves this slot (``flash_ck/utils/utils.py:50-59`` keeps a commented ``fmha`` registration and
``tests/pytorch/fmha/test_{fmha_fwd,fmha_fwd_var_len,batch_prefill,fmha_fwd_append_kv}.py`` name the intended
functions) but ships no implementation.  The functions here follow the pattern of its one finished operator
(``flash_ck/ops/norm/layer_norm.py:21-134``): validate the tensors, then call the registered backend --
except that there is **no PyTorch fallback**: a missing library or an unsupported problem raises.

Tensors are BSHD like the reference's ``AttentionLayer`` (``core/module/layers/attention_layers/
attention_layer.h:25-33``): q ``[b, sq, hq, d]``, k ``[b, sk, hkv, d]``, v ``[b, sk, hkv, dv]``; varlen
functions take packed ``[total, h, d]`` tensors plus ``cu_seqlens`` (int64 ``[b+1]``, the reference's
``seqstart``).  LSE is fp32 ``[b, hq, sq]`` (batch) or ``[hq, total_q]`` (varlen).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import torch

from .. import _lib
from ..utils.enums import MaskEnum, RopeEnum

__all__ = [
    "fmha_fwd",
    "fmha_fwd_var_len",
    "fmha_fwd_fp8",
    "quantize_fp8",
    "batch_prefill",
    "fmha_fwd_paged_kv_prefill",
    "fmha_fwd_splitkv",
    "fmha_fwd_splitkv_combine",
    "fmha_fwd_splitkv_combine_strided",
    "fmha_fwd_append_kv",
    "splitkv_workspace",
    "default_num_splits",
]


# --------------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------------
def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return _lib.FLOAT16
    if t.dtype == torch.bfloat16:
        return _lib.BFLOAT16
    raise TypeError(f"attention supports torch.float16 and torch.bfloat16, got {t.dtype}")


def _check_cuda(name: str, t: Optional[torch.Tensor], dtype=None) -> None:
    if t is None:
        return
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor, got {type(t)}")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must have dtype {dtype}, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _mask(causal: bool, window_size: Sequence[int], mask_type: Optional[int]) -> Tuple[int, int, int]:
    """(mask_type, left, right).  ``causal`` means bottom-right aligned window (-1, 0): for sq == sk it equals
    top-left, for decode / append (sq < sk) query i sees keys <= sk - sq + i."""
    left, right = int(window_size[0]), int(window_size[1])
    if mask_type is None:
        if causal:
            return int(MaskEnum.MASK_FROM_BOTTOM_RIGHT), left, 0
        if left >= 0 or right >= 0:
            return int(MaskEnum.MASK_FROM_BOTTOM_RIGHT), left, right
        return int(MaskEnum.NO_MASK), -1, -1
    mt = int(mask_type)
    if causal:
        right = 0
    return mt, left, right


def _as_i64(name: str, t: torch.Tensor) -> torch.Tensor:
    _check_cuda(name, t)
    if t.dtype != torch.int64:
        t = t.to(torch.int64)
    return t


def _as_i32(name: str, t: torch.Tensor) -> torch.Tensor:
    _check_cuda(name, t)
    if t.dtype != torch.int32:
        t = t.to(torch.int32)
    return t


# --------------------------------------------------------------------------------------------
# dense / varlen forward
# --------------------------------------------------------------------------------------------
def _alibi_args(alibi_slopes: Optional[torch.Tensor], batch: int, hq: int):
    """(pointer, bias_enum, bias_rank_info) for the ``...Ex`` symbols of the paged and split-KV families, which take the
    kind of bias per call (ALiBi slopes fp32 ``[1|batch, hq]`` or nothing), so that no process-wide instance parameter
    is touched on the launch path."""
    if alibi_slopes is None:
        return ctypes.c_void_p(0), 0, 0
    _check_cuda("alibi_slopes", alibi_slopes, torch.float32)
    if alibi_slopes.dim() != 2 or alibi_slopes.shape[1] != hq or alibi_slopes.shape[0] not in (1, batch):
        raise ValueError(f"alibi_slopes must be fp32 [1|{batch}, {hq}], got {tuple(alibi_slopes.shape)}")
    return _ptr(alibi_slopes), 2, (0 if alibi_slopes.shape[0] == 1 else 1)


def _dtype_name(t: torch.Tensor) -> str:
    return "fp16" if t.dtype == torch.float16 else "bf16"


def _mask_name(mt: int, wl: int, wr: int) -> str:
    if mt == 0:
        return "none"
    return "causal" if (wl < 0 and wr == 0) else "window"


def _launch_tuned(family: str, problem_args: dict, call):
    """Runs ``call`` (one C-ABI launch that returns a status).  With ``FC_TUNING_MODE`` 1 or 2 the instance parameters
    of the family are first set to the tuning cache's winner for this problem; on a cache miss the candidates are timed
    on this very call's tensors and the winner is cached (the reference tunes at graph-compile time and serves later
    runs from ``flash_ck.db``, core/profiling/graph_codegen.cc:54-126)."""
    from .. import tuner
    if not tuner.tuning_enabled():
        return call()
    from ..instances import FmhaProblem
    def run():  # a candidate that refuses the problem must not look fast: its status is an error
        _lib.check(call(), family)
    tuner.select_instance(family, FmhaProblem(family=family, **problem_args), run)
    return call()


def _bias_args(q: torch.Tensor, bias, alibi_slopes, batch: int, hq: int, sq: int, sk: int):
    """(buffer, bias_enum, bias_rank_info) for the C call; the enum and rank values are those of the reference's
    BiasEnum / BiasEnumInfo (core/profiling/attention/fmha_library.h:121-164)."""
    if bias is not None and alibi_slopes is not None:
        raise ValueError("bias and alibi_slopes are mutually exclusive (one bias_enum per call)")
    if bias is not None:
        _check_cuda("bias", bias, q.dtype)
        if bias.dim() != 4 or bias.shape[2] != sq or bias.shape[3] != sk or bias.shape[0] not in (1, batch) \
                or bias.shape[1] not in (1, hq) or (bias.shape[0] != 1 and bias.shape[1] != hq):
            raise ValueError(f"bias must be [1|{batch}, 1|{hq}, {sq}, {sk}] with a full head axis under a batch axis, "
                             f"got {tuple(bias.shape)}")
        rank = 0 if bias.shape[0] == 1 and bias.shape[1] == 1 else (1 if bias.shape[0] == 1 else 2)
        return bias, 1, rank
    if alibi_slopes is not None:
        _check_cuda("alibi_slopes", alibi_slopes, torch.float32)
        if alibi_slopes.dim() != 2 or alibi_slopes.shape[1] != hq or alibi_slopes.shape[0] not in (1, batch):
            raise ValueError(f"alibi_slopes must be fp32 [1|{batch}, {hq}], got {tuple(alibi_slopes.shape)}")
        return alibi_slopes, 2, (0 if alibi_slopes.shape[0] == 1 else 1)
    return None, 0, 0


def fmha_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: Optional[float] = None,
             causal: bool = False, window_size: Sequence[int] = (-1, -1), mask_type: Optional[int] = None,
             return_lse: bool = False, bias: Optional[torch.Tensor] = None,
             alibi_slopes: Optional[torch.Tensor] = None, logits_soft_cap: float = 0.0):
    """Dense forward attention (the reference's batch mode, C symbol ``FmhaFwd``).

    q ``[b, sq, hq, d]``, k ``[b, sk, hkv, d]``, v ``[b, sk, hkv, dv]`` -> o ``[b, sq, hq, dv]``
    (and LSE ``[b, hq, sq]`` when ``return_lse``).  ``bias`` ``[1|b, 1|hq, sq, sk]`` (q's dtype) is added to the scaled
    scores; ``alibi_slopes`` fp32 ``[1|b, hq]`` adds ``-slope * |i + sk - sq - j|``; ``logits_soft_cap`` > 0 caps the
    scaled scores with ``cap * tanh(score / cap)`` first."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _check_cuda(n, t, getattr(q, "dtype", None))
        if t.dim() != 4:
            raise ValueError(f"{n} must be [batch, seqlen, heads, hdim], got shape {tuple(t.shape)}")
    b, sq, hq, d = q.shape
    bk, sk, hkv, dk = k.shape
    if bk != b or v.shape[0] != b or v.shape[1] != sk or v.shape[2] != hkv or dk != d:
        raise ValueError(f"inconsistent shapes q{tuple(q.shape)} k{tuple(k.shape)} v{tuple(v.shape)}")
    dv = v.shape[3]
    mt, wl, wr = _mask(causal, window_size, mask_type)
    o = torch.empty((b, sq, hq, dv), dtype=q.dtype, device=q.device)
    lse = torch.empty((b, hq, sq), dtype=torch.float32, device=q.device) if return_lse else None
    bias_buf, bias_enum, bias_rank = _bias_args(q, bias, alibi_slopes, b, hq, sq, sk)
    with torch.cuda.device(q.device):
        rc = _launch_tuned(
            "fmha_fwd", dict(dtype=_dtype_name(q), mode="batch", batch=b, hq=hq, hkv=hkv, d=d, dv=dv, max_seqlen_q=sq,
                             max_seqlen_k=sk, mask=_mask_name(mt, wl, wr), bias=("none", "elementwise", "alibi")[bias_enum],
                             soft_cap=logits_soft_cap > 0),
            lambda: _lib.lib().FmhaFwdBias(_ptr(q), _ptr(k), _ptr(v), _ptr(bias_buf), _ptr(o), None, None, None, b, sq, sk,
                                           hq, hkv, d, dv, sq, float(scale or 0.0), wl, wr, mt, _stream(), _ptr(lse),
                                           _dtype_code(q), bias_enum, bias_rank, float(logits_soft_cap)))
    _lib.check(rc, "FmhaFwd")
    return (o, lse) if return_lse else o


_F8_CODES = {torch.float8_e4m3fn: _lib.FLOAT8, torch.float8_e5m2: _lib.BFLOAT8}
_F8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}


def quantize_fp8(x: torch.Tensor, dtype: torch.dtype = torch.float8_e4m3fn, amax: Optional[float] = None):
    """Static per-tensor quantisation: ``(x8, descale)`` with ``x ~= x8.float() * descale``.  ``amax`` is the calibrated
    range of the tensor (the reference's ``range_q`` / ``range_k`` / ``range_v``, fmha_fwd_jinja.h:27); by default the
    tensor's own maximum magnitude.  Values are scaled to the type's largest finite number and rounded to nearest."""
    fmax = _F8_MAX[dtype]
    amax = float(amax) if amax is not None else float(x.abs().max())
    amax = amax if amax > 0 else 1.0
    scaled = (x.float() * (fmax / amax)).clamp(-fmax, fmax)
    return scaled.to(dtype), amax / fmax


def fmha_fwd_fp8(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale_s: float = 0.0, scale_p: float = 1.0,
                 scale_o: float = 1.0, cu_seqlens_q: Optional[torch.Tensor] = None,
                 cu_seqlens_k: Optional[torch.Tensor] = None, max_seqlen_q: int = 0, causal: bool = False,
                 window_size: Sequence[int] = (-1, -1), mask_type: Optional[int] = None,
                 out_dtype: Optional[torch.dtype] = None, return_lse: bool = False):
    """Forward attention on 8-bit operands with static quantisation scales (C symbol ``FmhaFwdFp8``; the reference's
    ``FmhaFwdTypeConfig<fp8_t / bf8_t>``).  q/k/v are ``torch.float8_e4m3fn`` or ``torch.float8_e5m2`` tensors, BSHD or
    packed with ``cu_seqlens``.  ``S = scale_s * Q K^T`` (0: 1/sqrt(d)), ``P8 = round8(scale_p * p)``,
    ``O = scale_o * (P8 V) / l`` stored as ``out_dtype`` (default: the input type; fp16 / bf16 also allowed).  With
    tensors from :func:`quantize_fp8`: ``scale_s = softmax_scale * dq * dk``, ``scale_o = dv / (scale_p * do)``."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _check_cuda(n, t, getattr(q, "dtype", None))
    code = _F8_CODES.get(q.dtype)
    if code is None:
        raise TypeError(f"fmha_fwd_fp8 takes float8_e4m3fn or float8_e5m2 tensors, got {q.dtype}")
    out_dtype = out_dtype or q.dtype
    out_code = {**_F8_CODES, torch.float16: _lib.FLOAT16, torch.bfloat16: _lib.BFLOAT16}.get(out_dtype)
    if out_code is None:
        raise TypeError(f"out_dtype must be an 8-bit float type, float16 or bfloat16, got {out_dtype}")
    group = cu_seqlens_q is not None
    if group:
        if q.dim() != 3 or cu_seqlens_k is None:
            raise ValueError("packed q/k/v [total, heads, hdim] need cu_seqlens_q and cu_seqlens_k")
        cu_q, cu_k = _as_i64("cu_seqlens_q", cu_seqlens_q), _as_i64("cu_seqlens_k", cu_seqlens_k)
        batch, (total_q, hq, d), (total_k, hkv, _) = cu_q.numel() - 1, q.shape, k.shape
        sq, sk, max_sq = total_q, total_k, int(max_seqlen_q) or total_q
        o_shape, lse_shape = (total_q, hq), (hq, total_q)
    else:
        if q.dim() != 4:
            raise ValueError("q, k, v must be [batch, seqlen, heads, hdim]")
        cu_q = cu_k = None
        batch, sq, hq, d = q.shape
        sk, hkv, max_sq = k.shape[1], k.shape[2], sq
        o_shape, lse_shape = (batch, sq, hq), (batch, hq, sq)
    dv = v.shape[-1]
    mt, wl, wr = _mask(causal, window_size, mask_type)
    o = torch.empty(o_shape + (dv,), dtype=out_dtype, device=q.device)
    lse = torch.empty(lse_shape, dtype=torch.float32, device=q.device) if return_lse else None
    with torch.cuda.device(q.device):
        rc = _lib.lib().FmhaFwdFp8(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(cu_q), _ptr(cu_k), batch, sq, sk, hq, hkv, d, dv,
                                   max_sq, float(scale_s), float(scale_p), float(scale_o), wl, wr, mt, _stream(), _ptr(lse),
                                   code, out_code)
    _lib.check(rc, "FmhaFwdFp8")
    return (o, lse) if return_lse else o


def fmha_fwd_var_len(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor,
                     cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int = 0, *,
                     scale: Optional[float] = None, causal: bool = False, window_size: Sequence[int] = (-1, -1),
                     mask_type: Optional[int] = None, return_lse: bool = False, bias: Optional[torch.Tensor] = None,
                     alibi_slopes: Optional[torch.Tensor] = None, logits_soft_cap: float = 0.0):
    """Variable-length forward attention (the reference's group mode: packed tokens + ``seqstart`` arrays).

    q ``[total_q, hq, d]``, k ``[total_k, hkv, d]``, v ``[total_k, hkv, dv]``; ``cu_seqlens_*`` int64 ``[b+1]``.
    Returns o ``[total_q, hq, dv]`` (and LSE ``[hq, total_q]``).  ``bias`` is ``[1, 1|hq, total_q, total_k]`` here (the
    reference's group-mode shape: one plane over the packed rows and keys, of which every sequence uses its own block);
    ``alibi_slopes`` and ``logits_soft_cap`` as in :func:`fmha_fwd`."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _check_cuda(n, t, getattr(q, "dtype", None))
        if t.dim() != 3:
            raise ValueError(f"{n} must be packed [total_tokens, heads, hdim], got shape {tuple(t.shape)}")
    cu_q = _as_i64("cu_seqlens_q", cu_seqlens_q)
    cu_k = _as_i64("cu_seqlens_k", cu_seqlens_k)
    if cu_q.numel() != cu_k.numel() or cu_q.numel() < 2:
        raise ValueError("cu_seqlens_q and cu_seqlens_k must both have batch + 1 entries")
    batch = cu_q.numel() - 1
    total_q, hq, d = q.shape
    total_k, hkv, dk = k.shape
    if dk != d or v.shape[0] != total_k or v.shape[1] != hkv:
        raise ValueError(f"inconsistent shapes q{tuple(q.shape)} k{tuple(k.shape)} v{tuple(v.shape)}")
    dv = v.shape[2]
    mt, wl, wr = _mask(causal, window_size, mask_type)
    o = torch.empty((total_q, hq, dv), dtype=q.dtype, device=q.device)
    lse = torch.empty((hq, total_q), dtype=torch.float32, device=q.device) if return_lse else None
    bias_buf, bias_enum, bias_rank = _bias_args(q, bias, alibi_slopes, 1 if bias is not None else batch, hq, total_q,
                                                total_k)
    with torch.cuda.device(q.device):
        rc = _launch_tuned(
            "fmha_fwd", dict(dtype=_dtype_name(q), mode="group", batch=batch, hq=hq, hkv=hkv, d=d, dv=dv,
                             max_seqlen_q=int(max_seqlen_q), max_seqlen_k=int(max_seqlen_k) or int(max_seqlen_q),
                             mask=_mask_name(mt, wl, wr), bias=("none", "elementwise", "alibi")[bias_enum],
                             soft_cap=logits_soft_cap > 0),
            lambda: _lib.lib().FmhaFwdBias(_ptr(q), _ptr(k), _ptr(v), _ptr(bias_buf), _ptr(o), _ptr(cu_q), _ptr(cu_k), None,
                                           batch, total_q, total_k, hq, hkv, d, dv, int(max_seqlen_q), float(scale or 0.0),
                                           wl, wr, mt, _stream(), _ptr(lse), _dtype_code(q), bias_enum, bias_rank,
                                           float(logits_soft_cap)))
    _lib.check(rc, "FmhaFwd")
    return (o, lse) if return_lse else o


def batch_prefill(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, cu_seqlens_q: torch.Tensor,
                  kv_indptr: torch.Tensor, kv_page_indices: torch.Tensor, kv_last_page_len: torch.Tensor,
                  max_seqlen_q: int, *, scale: Optional[float] = None, causal: bool = True,
                  window_size: Sequence[int] = (-1, -1), mask_type: Optional[int] = None, return_lse: bool = False,
                  alibi_slopes: Optional[torch.Tensor] = None):
    """Varlen prefill over an SGLang-style page table (``fmha_fwd_batch_prefill``).

    q ``[total_q, hq, d]``; pools ``[num_total_pages, page, hkv, d|dv]``; ``kv_indptr`` int32 ``[b+1]``,
    ``kv_page_indices`` int32, ``kv_last_page_len`` int32 ``[b]``."""
    _check_cuda("q", q)
    _check_cuda("k_pool", k_pool, q.dtype)
    _check_cuda("v_pool", v_pool, q.dtype)
    if q.dim() != 3 or k_pool.dim() != 4 or v_pool.dim() != 4:
        raise ValueError("q must be [total_q, hq, d]; pools must be [pages, page, hkv, hdim]")
    cu_q = _as_i64("cu_seqlens_q", cu_seqlens_q)
    indptr = _as_i32("kv_indptr", kv_indptr)
    indices = _as_i32("kv_page_indices", kv_page_indices)
    last = _as_i32("kv_last_page_len", kv_last_page_len)
    batch = cu_q.numel() - 1
    if indptr.numel() != batch + 1 or last.numel() != batch:
        raise ValueError("kv_indptr must have batch + 1 entries and kv_last_page_len batch entries")
    total_q, hq, d = q.shape
    pages, page, hkv, dk = k_pool.shape
    dv = v_pool.shape[3]
    if dk != d or v_pool.shape[:3] != k_pool.shape[:3]:
        raise ValueError(f"inconsistent shapes q{tuple(q.shape)} k{tuple(k_pool.shape)} v{tuple(v_pool.shape)}")
    mt, wl, wr = _mask(causal, window_size, mask_type)
    o = torch.empty((total_q, hq, dv), dtype=q.dtype, device=q.device)
    lse = torch.empty((hq, total_q), dtype=torch.float32, device=q.device) if return_lse else None
    bias_ptr, bias_enum, bias_rank = _alibi_args(alibi_slopes, batch, hq)
    with torch.cuda.device(q.device):
        rc = _lib.lib().FmhaFwdBatchPrefillEx(_ptr(q), _ptr(k_pool), _ptr(v_pool), bias_ptr, _ptr(o), _ptr(cu_q),
                                              _ptr(indptr), _ptr(indices), _ptr(last), batch, total_q, hq, hkv, d, dv,
                                              int(max_seqlen_q), pages, page, float(scale or 0.0), wl, wr, mt,
                                              _stream(), _ptr(lse), _dtype_code(q), bias_enum, bias_rank)
    _lib.check(rc, "FmhaFwdBatchPrefill")
    return (o, lse) if return_lse else o


def fmha_fwd_paged_kv_prefill(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                              block_table: torch.Tensor, seqlen_k: torch.Tensor, *,
                              cu_seqlens_q: Optional[torch.Tensor] = None, max_seqlen_q: int = 0,
                              cache_batch_idx: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                              causal: bool = True, window_size: Sequence[int] = (-1, -1),
                              mask_type: Optional[int] = None, return_lse: bool = False,
                              alibi_slopes: Optional[torch.Tensor] = None):
    """Prefill reading K/V through a block table (``fmha_fwd_paged_kv_prefill``).

    q ``[b, sq, hq, d]`` or packed ``[total_q, hq, d]`` with ``cu_seqlens_q``; pools ``[pages, page, hkv, *]``;
    ``block_table`` int32 ``[b, pages_per_seq]``; ``seqlen_k`` int32 ``[b]``."""
    _check_cuda("q", q)
    _check_cuda("k_pool", k_pool, q.dtype)
    _check_cuda("v_pool", v_pool, q.dtype)
    bt = _as_i32("block_table", block_table)
    sl = _as_i32("seqlen_k", seqlen_k)
    batch = bt.shape[0]
    group = cu_seqlens_q is not None
    cu_q = _as_i64("cu_seqlens_q", cu_seqlens_q) if group else None
    cbi = _as_i64("cache_batch_idx", cache_batch_idx) if cache_batch_idx is not None else None
    if group:
        total_q, hq, d = q.shape
        shape_sq, max_sq = total_q, int(max_seqlen_q) or total_q
        o_shape, lse_shape = (total_q, hq), (hq, total_q)
    else:
        b, sq, hq, d = q.shape
        if b != batch:
            raise ValueError("q batch and block_table rows differ")
        shape_sq, max_sq = sq, sq
        o_shape, lse_shape = (b, sq, hq), (b, hq, sq)
    pages, page, hkv, dk = k_pool.shape
    dv = v_pool.shape[3]
    mt, wl, wr = _mask(causal, window_size, mask_type)
    o = torch.empty(o_shape + (dv,), dtype=q.dtype, device=q.device)
    lse = torch.empty(lse_shape, dtype=torch.float32, device=q.device) if return_lse else None
    bias_ptr, bias_enum, bias_rank = _alibi_args(alibi_slopes, batch, hq)
    with torch.cuda.device(q.device):
        rc = _lib.lib().FmhaFwdPagedKVPrefillEx(_ptr(q), _ptr(k_pool), _ptr(v_pool), bias_ptr, _ptr(o), _ptr(cu_q),
                                                _ptr(sl), _ptr(bt), _ptr(cbi), batch, shape_sq, hq, hkv, d, dv, max_sq,
                                                batch * bt.shape[1], page, float(scale or 0.0), wl, wr, mt, _stream(),
                                                _ptr(lse), _dtype_code(q), bias_enum, bias_rank, pages)
    _lib.check(rc, "FmhaFwdPagedKVPrefill")
    return (o, lse) if return_lse else o


# --------------------------------------------------------------------------------------------
# split-KV decode
# --------------------------------------------------------------------------------------------
def default_num_splits(batch: int, sm_count: int = 148, max_splits: int = 128, rows_per_kv_head: int = 1) -> int:
    """Workspace depth for ``fmha_fwd_splitkv`` when the caller passes ``num_splits=0``.

    With more than 16 query rows per kv head (``seqlen_q * hq / hkv``) the call runs on the tcgen05 instance, which
    cuts the key tiles of all (sequence, kv head) streams into one equal piece per SM; a stream cut k times uses k + 1
    splits (twice that with at most 64 rows), and the piece is lengthened when the workspace has fewer.  16 splits
    leave room for seven cuts of the longest stream, which measured the same as 8 and 32 on 32 sequences of 2k-16k
    keys.  Otherwise:

    The kernel cuts the concatenated key stream of all sequences into one equal piece per SM, so a sequence of
    average length is touched by about ``sm_count / batch`` pieces; twice that (plus one for a piece boundary)
    keeps the cut even when the longest sequence is twice the average.  The reference leaves this heuristic
    open ("0 to determine actual number by heuristic", fmha_fwd_split_kv_jinja.h:28-30)."""
    if rows_per_kv_head > 16:
        return int(min(max_splits, 16))
    return int(max(2, min(max_splits, -(-2 * sm_count // max(batch, 1)) + 1)))


def splitkv_workspace(q: torch.Tensor, dv: int, num_splits: int, cu_seqlens_q: Optional[torch.Tensor] = None):
    """Allocates ``(lse_acc, o_acc)`` in the reference's layout (fmha_fwd_split_kv_jinja.h:543-547):
    ``lse_acc [b, hq, S, sq]`` and ``o_acc [b, hq, S, sq, dv]`` fp32 (varlen: b = 1, sq = total_q)."""
    if cu_seqlens_q is not None:
        total_q, hq, _ = q.shape
        bs, rows = 1, total_q
    else:
        bs, rows, hq, _ = q.shape
    lse_acc = torch.empty((bs, hq, num_splits, rows), dtype=torch.float32, device=q.device)
    o_acc = torch.empty((bs, hq, num_splits, rows, dv), dtype=torch.float32, device=q.device)
    return lse_acc, o_acc


_OUT_CODES = {torch.float16: 3, torch.bfloat16: 4, torch.float32: 7}


def fmha_fwd_splitkv_combine(lse_acc: torch.Tensor, o_acc: torch.Tensor, dtype: torch.dtype, *,
                             varlen: bool = False, return_lse: bool = False, out: Optional[torch.Tensor] = None,
                             lse_out: Optional[torch.Tensor] = None):
    """LSE-weighted merge of split partials (C symbol ``FmhaFwdSplitKVCombine``).

    ``lse_acc [bs, hq, S, rows]``, ``o_acc [bs, hq, S, rows, dv]`` fp32 -> o ``[bs, rows, hq, dv]``
    (``[rows, hq, dv]`` when ``varlen``) in ``dtype`` and LSE ``[bs, hq, rows]`` (``[hq, rows]``).
    ``dtype=torch.float32`` keeps the merged partial in fp32 (what one rank contributes when the KV sequence is
    sharded over GPUs); ``out`` / ``lse_out`` receive the results in place."""
    _check_cuda("lse_acc", lse_acc, torch.float32)
    _check_cuda("o_acc", o_acc, torch.float32)
    if o_acc.dim() != 5 or lse_acc.shape != o_acc.shape[:4]:
        raise ValueError(f"bad workspace shapes lse_acc{tuple(lse_acc.shape)} o_acc{tuple(o_acc.shape)}")
    bs, hq, S, rows, dv = o_acc.shape
    if varlen and bs != 1:
        raise ValueError("varlen workspaces have a single batch row")
    code = _OUT_CODES.get(dtype)
    if code is None:
        raise TypeError(f"output dtype must be float16, bfloat16 or float32, got {dtype}")
    o = out if out is not None else torch.empty((bs, rows, hq, dv), dtype=dtype, device=o_acc.device)
    _check_cuda("out", o, dtype)
    lse = lse_out if lse_out is not None else (
        torch.empty((bs, hq, rows), dtype=torch.float32, device=o_acc.device) if return_lse else None)
    _check_cuda("lse_out", lse, torch.float32)
    with torch.cuda.device(o_acc.device):
        if dtype == torch.float32:
            ls = (ctypes.c_int64 * 4)(hq * S * rows, S * rows, rows, 1)
            os_ = (ctypes.c_int64 * 4)(hq * S * rows * dv, S * rows * dv, rows * dv, dv)
            rc = _lib.lib().FmhaFwdSplitKVCombineStrided(_ptr(lse_acc), _ptr(o_acc), _ptr(o), _ptr(lse), bs, rows, hq, dv,
                                                         S, ls, os_, code, _stream())
        else:
            # group mode is signalled by a non-null seqstart pointer; its contents are not needed by the combine
            marker = torch.zeros(1, dtype=torch.int64, device=o_acc.device) if varlen else None
            rc = _lib.lib().FmhaFwdSplitKVCombine(_ptr(lse_acc), _ptr(o_acc), _ptr(o), _ptr(marker), bs, rows, hq, dv,
                                                  rows, S, _stream(), _ptr(lse), code)
    _lib.check(rc, "FmhaFwdSplitKVCombine")
    if varlen and out is None:
        o = o[0]
        lse = lse[0] if lse is not None else None
    return (o, lse) if (return_lse or lse_out is not None) else o


def fmha_fwd_splitkv_combine_strided(buf: torch.Tensor, batch: int, rows: int, hq: int, dv: int, num_splits: int, *,
                                     lse_offset: int, lse_strides: Sequence[int], o_strides: Sequence[int],
                                     dtype: torch.dtype, return_lse: bool = False):
    """Merge of partials that sit in one fp32 buffer with arbitrary strides (C symbol
    ``FmhaFwdSplitKVCombineStrided``): the O partials start at element 0 of ``buf``, the LSE partials at element
    ``lse_offset``; strides are in elements for (batch, head, split, row).  Returns o ``[batch, rows, hq, dv]`` in
    ``dtype`` (and LSE ``[batch, hq, rows]``)."""
    _check_cuda("buf", buf, torch.float32)
    code = _OUT_CODES.get(dtype)
    if code is None:
        raise TypeError(f"output dtype must be float16, bfloat16 or float32, got {dtype}")
    o = torch.empty((batch, rows, hq, dv), dtype=dtype, device=buf.device)
    lse = torch.empty((batch, hq, rows), dtype=torch.float32, device=buf.device) if return_lse else None
    ls = (ctypes.c_int64 * 4)(*[int(x) for x in lse_strides])
    os_ = (ctypes.c_int64 * 4)(*[int(x) for x in o_strides])
    with torch.cuda.device(buf.device):
        rc = _lib.lib().FmhaFwdSplitKVCombineStrided(ctypes.c_void_p(buf.data_ptr() + 4 * int(lse_offset)), _ptr(buf),
                                                     _ptr(o), _ptr(lse), batch, rows, hq, dv, num_splits, ls, os_, code,
                                                     _stream())
    _lib.check(rc, "FmhaFwdSplitKVCombineStrided")
    return (o, lse) if return_lse else o


def fmha_fwd_splitkv(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *,
                     seqlen_k: Optional[torch.Tensor] = None, block_table: Optional[torch.Tensor] = None,
                     cache_batch_idx: Optional[torch.Tensor] = None, cu_seqlens_q: Optional[torch.Tensor] = None,
                     cu_seqlens_k: Optional[torch.Tensor] = None, max_seqlen_q: int = 0, num_splits: int = 0,
                     scale: Optional[float] = None, causal: bool = False, window_size: Sequence[int] = (-1, -1),
                     mask_type: Optional[int] = None, return_lse: bool = False,
                     workspace: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, combine: bool = True,
                     alibi_slopes: Optional[torch.Tensor] = None):
    """Split-KV attention (decode) over a contiguous or paged KV cache, followed by the combine.

    q ``[b, sq, hq, d]`` (or packed ``[total_q, hq, d]`` with ``cu_seqlens_q``).
    Paged: ``k_cache/v_cache [pages, page, hkv, *]`` + ``block_table`` int32 ``[b, pages_per_seq]`` +
    ``seqlen_k`` int32 ``[b]``.  Contiguous: ``[b_cache, sk, hkv, *]`` (+ optional ``seqlen_k``,
    ``cache_batch_idx``) or packed ``[total_k, hkv, *]`` with ``cu_seqlens_k``.
    ``combine=False`` returns the raw ``(lse_acc, o_acc)`` workspaces."""
    _check_cuda("q", q)
    _check_cuda("k_cache", k_cache, q.dtype)
    _check_cuda("v_cache", v_cache, q.dtype)
    group = cu_seqlens_q is not None
    cu_q = _as_i64("cu_seqlens_q", cu_seqlens_q) if group else None
    cu_k = _as_i64("cu_seqlens_k", cu_seqlens_k) if cu_seqlens_k is not None else None
    sl = _as_i32("seqlen_k", seqlen_k) if seqlen_k is not None else None
    bt = _as_i32("block_table", block_table) if block_table is not None else None
    cbi = _as_i64("cache_batch_idx", cache_batch_idx) if cache_batch_idx is not None else None
    if group:
        if q.dim() != 3:
            raise ValueError("varlen q must be [total_q, hq, d]")
        total_q, hq, d = q.shape
        batch = cu_q.numel() - 1
        shape_sq, max_sq = total_q, int(max_seqlen_q) or total_q
    else:
        if q.dim() != 4:
            raise ValueError("q must be [b, sq, hq, d]")
        batch, sq, hq, d = q.shape
        shape_sq, max_sq = sq, sq
    hkv, dv = k_cache.shape[-2], v_cache.shape[-1]
    if k_cache.shape[-1] != d:
        raise ValueError("k_cache hdim differs from q")
    if bt is not None:
        if sl is None:
            raise ValueError("paged K/V needs seqlen_k")
        if k_cache.dim() != 4 or bt.shape[0] != batch and cbi is None:
            raise ValueError("paged pools must be [pages, page, hkv, hdim] and block_table [batch, pages_per_seq]")
        page = k_cache.shape[1]
        # the reference passes batch * pages_per_seq and recovers the row stride by dividing (:318)
        max_pages = batch * bt.shape[1]
        shape_sk = 0
    else:
        page, max_pages = 0, 0
        shape_sk = k_cache.shape[0] if cu_k is not None else k_cache.shape[1]
    S = int(num_splits) if num_splits and num_splits > 0 else \
        default_num_splits(batch, rows_per_kv_head=max_sq * (hq // max(hkv, 1)))
    if workspace is None:
        lse_acc, o_acc = splitkv_workspace(q, dv, S, cu_q)
    else:
        lse_acc, o_acc = workspace
        S = o_acc.shape[2]
    mt, wl, wr = _mask(causal, window_size, mask_type)
    bias_ptr, bias_enum, bias_rank = _alibi_args(alibi_slopes, batch, hq)
    # pages of a paged pool, or rows of a contiguous cache (packed K/V: unused): where the K/V tensor maps end
    pool_extent = 0 if cu_k is not None else k_cache.shape[0]
    cap_k = bt.shape[1] * page if bt is not None else shape_sk
    with torch.cuda.device(q.device):
        rc = _launch_tuned(
            "fmha_fwd_split_kv", dict(dtype=_dtype_name(q), mode="group" if group else "batch", batch=batch, hq=hq, hkv=hkv,
                                      d=d, dv=dv, max_seqlen_q=max_sq, max_seqlen_k=int(cap_k), mask=_mask_name(mt, wl, wr),
                                      bias="alibi" if bias_enum else "none", paged=bt is not None, page=int(page)),
            lambda: _lib.lib().FmhaFwdSplitKVEx(_ptr(q), _ptr(k_cache), _ptr(v_cache), bias_ptr, _ptr(lse_acc), _ptr(o_acc),
                                                _ptr(cu_q), _ptr(cu_k), _ptr(sl), _ptr(bt), _ptr(cbi), batch, shape_sq,
                                                shape_sk, hq, hkv, d, dv, max_sq, S, max_pages, page, float(scale or 0.0),
                                                wl, wr, mt, _stream(), _dtype_code(q), bias_enum, bias_rank, pool_extent))
    _lib.check(rc, "FmhaFwdSplitKV")
    if not combine:
        return lse_acc, o_acc
    return fmha_fwd_splitkv_combine(lse_acc, o_acc, q.dtype, varlen=group, return_lse=return_lse)


# --------------------------------------------------------------------------------------------
# append-KV
# --------------------------------------------------------------------------------------------
def fmha_fwd_append_kv(q: Optional[torch.Tensor], k_cache: torch.Tensor, v_cache: torch.Tensor,
                       knew: torch.Tensor, vnew: torch.Tensor, seqlen_k: torch.Tensor,
                       rotary_cos: Optional[torch.Tensor] = None, rotary_sin: Optional[torch.Tensor] = None, *,
                       rope: int = RopeEnum.INTERLEAVED, rotary_dim: Optional[int] = None,
                       block_table: Optional[torch.Tensor] = None, cache_batch_idx: Optional[torch.Tensor] = None,
                       cu_seqlens_q: Optional[torch.Tensor] = None, cu_seqlens_knew: Optional[torch.Tensor] = None):
    """RoPE on ``q`` (in place) and on the new keys, then the K/V cache write (``fmha_fwd_appendkv``).

    ``seqlen_k`` int32 ``[b]`` is the cached length *before* the append; new token j of sequence b is written
    at position ``seqlen_k[b] + j`` and query i is rotated at ``seqlen_k[b] + n_new[b] - sq[b] + i``.
    Batch mode: q ``[b, sq, hq, d]``, knew ``[b, n, hkv, d]``, vnew ``[b, n, hkv, dv]``.  Varlen: packed
    tensors with ``cu_seqlens_q`` / ``cu_seqlens_knew`` (int64 ``[b+1]``).  Returns ``q`` (rotated)."""
    rope = int(rope)
    if rope != RopeEnum.NONE and (rotary_cos is None or rotary_sin is None):
        raise ValueError("rotary_cos / rotary_sin are required unless rope == RopeEnum.NONE")
    _check_cuda("k_cache", k_cache)
    dt = k_cache.dtype
    for n, t in (("q", q), ("v_cache", v_cache), ("knew", knew), ("vnew", vnew), ("rotary_cos", rotary_cos),
                 ("rotary_sin", rotary_sin)):
        _check_cuda(n, t, dt)
    sl = _as_i32("seqlen_k", seqlen_k)
    bt = _as_i32("block_table", block_table) if block_table is not None else None
    cbi = _as_i64("cache_batch_idx", cache_batch_idx) if cache_batch_idx is not None else None
    group = cu_seqlens_knew is not None
    batch = sl.numel()
    hkv, d = knew.shape[-2], knew.shape[-1]
    dv = vnew.shape[-1]
    if group:
        cu_n = _as_i64("cu_seqlens_knew", cu_seqlens_knew)
        if cu_seqlens_q is None:
            raise ValueError("varlen append needs cu_seqlens_q together with cu_seqlens_knew")
        cu_q = _as_i64("cu_seqlens_q", cu_seqlens_q)
        n_new = knew.shape[0]
        sq = q.shape[0] if q is not None else 0
    else:
        cu_n = cu_q = None
        n_new = knew.shape[1]
        sq = q.shape[1] if q is not None else 0
    hq = q.shape[-2] if q is not None else hkv
    if rotary_dim is None:
        rotary_dim = 2 * rotary_cos.shape[-1] if rope != RopeEnum.NONE else 0
    if bt is not None:
        page, max_pages, cap = k_cache.shape[1], batch * bt.shape[1], 0
    else:
        page, max_pages, cap = 0, 0, k_cache.shape[1]
    with torch.cuda.device(k_cache.device):
        rc = _lib.lib().FmhaFwdAppendKV(_ptr(q), _ptr(k_cache), _ptr(knew), _ptr(v_cache), _ptr(vnew), _ptr(sl),
                                        _ptr(cu_q), _ptr(cu_n), _ptr(rotary_cos), _ptr(rotary_sin), _ptr(bt),
                                        _ptr(cbi), batch, sq, cap, n_new, hq, hkv, d, dv, int(rotary_dim), rope,
                                        max_pages, page, _stream(), _dtype_code(k_cache))
    _lib.check(rc, "FmhaFwdAppendKV")
    return q
