"""flashck_b200 -- B200-native (sm_100a) attention path behind FlashCK's operator API.

Package layout follows the reference's ``flash_ck`` package (``flash_ck/__init__.py:8-35``): ``ops`` (functional
API), ``nn`` (modules) and ``utils`` (registry, enums).  The compute lives in ``libflashck_b200.so``
(``csrc/``, C ABI in ``include/flashck_b200.h``) and is reached through ``ctypes``; importing the package does
not load the library, the first operator call does -- and raises if it is missing.
"""
from . import nn, ops, utils
from .compat import install_as_flash_ck
from .ops import (batch_prefill, fmha_fwd, fmha_fwd_append_kv, fmha_fwd_paged_kv_prefill, fmha_fwd_splitkv,
                  fmha_fwd_splitkv_combine, fmha_fwd_var_len)
from .utils import (get_available_operations, get_flag_value, is_available, print_all_flags, print_flag_info,
                    register_flashck_functions, set_flag_value)

__version__ = "0.1.0"

# Fill the reference's `fmha` registry slot (flash_ck/utils/utils.py:50-59).
register_flashck_functions(utils.FlashCKOperationType.FMHA.value, {
    "forward": fmha_fwd,
    "forward_var_len": fmha_fwd_var_len,
    "batch_prefill": batch_prefill,
    "paged_kv_prefill": fmha_fwd_paged_kv_prefill,
    "forward_splitkv": fmha_fwd_splitkv,
    "splitkv_combine": fmha_fwd_splitkv_combine,
    "append_kv": fmha_fwd_append_kv,
})

__all__ = [
    "ops", "nn", "utils", "install_as_flash_ck", "fmha_fwd", "fmha_fwd_var_len", "batch_prefill", "fmha_fwd_paged_kv_prefill",
    "fmha_fwd_splitkv", "fmha_fwd_splitkv_combine", "fmha_fwd_append_kv", "is_available",
    "get_available_operations", "get_flag_value", "set_flag_value", "print_all_flags", "print_flag_info",
]
