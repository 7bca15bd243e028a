"""Functional operations (the reference's ``flash_ck.ops``), attention family only."""
from . import fmha
from .fmha import (batch_prefill, default_num_splits, fmha_fwd, fmha_fwd_append_kv, fmha_fwd_fp8,
                   fmha_fwd_paged_kv_prefill, fmha_fwd_splitkv, fmha_fwd_splitkv_combine,
                   fmha_fwd_splitkv_combine_strided, fmha_fwd_var_len, quantize_fp8, splitkv_workspace)

__all__ = [
    "fmha", "fmha_fwd", "fmha_fwd_var_len", "fmha_fwd_fp8", "quantize_fp8", "batch_prefill", "fmha_fwd_paged_kv_prefill", "fmha_fwd_splitkv",
    "fmha_fwd_splitkv_combine", "fmha_fwd_splitkv_combine_strided", "fmha_fwd_append_kv", "splitkv_workspace", "default_num_splits",
]
