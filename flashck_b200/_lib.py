"""ctypes binding of ``libflashck_b200.so`` -- the C ABI declared in ``include/flashck_b200.h``.

There is no fallback: if the library is missing or a call fails, a ``RuntimeError`` is raised.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libflashck_b200.so")
_LIB: Optional[ctypes.CDLL] = None

FLOAT8, BFLOAT8, FLOAT16, BFLOAT16 = 1, 2, 3, 4  # flashck::DataType values (core/utils/dtype.h:16-28)

_P, _I64, _F, _U32, _I = ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_uint32, ctypes.c_int

# name -> argtypes, in the order of include/flashck_b200.h
SIGNATURES = {
    "FlashckGetLastError": ([], ctypes.c_char_p),
    "FlashckVersion": ([], ctypes.c_char_p),
    "FlashckDeviceStatus": ([ctypes.POINTER(ctypes.c_int)], _I),
    "FmhaFwd": ([_P] * 8 + [_I64] * 8 + [_F, _I64, _I64, _U32, _P, _P, _I], _I),
    "FmhaFwdBias": ([_P] * 8 + [_I64] * 8 + [_F, _I64, _I64, _U32, _P, _P, _I, _I, _I, _F], _I),
    "FmhaFwdFp8": ([_P] * 6 + [_I64] * 8 + [_F, _F, _F, _I64, _I64, _U32, _P, _P, _I, _I], _I),
    "FmhaFwdBatchPrefill": ([_P] * 9 + [_I64] * 9 + [_F, _I64, _I64, _U32, _P, _P, _I], _I),
    "FmhaFwdPagedKVPrefill": ([_P] * 9 + [_I64] * 9 + [_F, _I64, _I64, _U32, _P, _P, _I], _I),
    "FmhaFwdSplitKV": ([_P] * 11 + [_I64] * 11 + [_F, _I64, _I64, _U32, _P, _I], _I),
    "FmhaFwdBatchPrefillEx": ([_P] * 9 + [_I64] * 9 + [_F, _I64, _I64, _U32, _P, _P, _I, _I, _I], _I),
    "FmhaFwdPagedKVPrefillEx": ([_P] * 9 + [_I64] * 9 + [_F, _I64, _I64, _U32, _P, _P, _I, _I, _I, _I64], _I),
    "FmhaFwdSplitKVEx": ([_P] * 11 + [_I64] * 11 + [_F, _I64, _I64, _U32, _P, _I, _I, _I, _I64], _I),
    "FmhaFwdSplitKVCombine": ([_P] * 4 + [_I64] * 6 + [_P, _P, _I], _I),
    "FmhaSplitKVCombine": ([_P] * 4 + [_I64] * 6 + [_P, _P, _I], _I),
    "FmhaFwdSplitKVCombineStrided": ([_P] * 4 + [_I64] * 5 + [ctypes.POINTER(_I64), ctypes.POINTER(_I64), _I, _P], _I),
    "FlashckShardExchangeBytes": ([_I64] * 4 + [_I], _I64),
    "FmhaFwdSplitKVShardedCombine": ([_P] * 5 + [_I, _I, _I] + [_I64] * 5 + [_I, _P], _I),
    "FlashckPeerBufferCreate": ([_I64, ctypes.POINTER(_P), _P], _I),
    "FlashckPeerBufferOpen": ([_P, ctypes.POINTER(_P)], _I),
    "FlashckPeerBufferClose": ([_P], _I),
    "FlashckPeerBufferFree": ([_P], _I),
    "FmhaFwdSplitKVStatic": ([_P] * 10 + [_I64] * 11 + [_F, _I64, _I64, _U32, _P, _I], _I),
    "FmhaFwdAppendKV": ([_P] * 12 + [_I64] * 9 + [_I, _I64, _I64, _P, _I], _I),
    "FlashckSetInstanceParam": ([_I, ctypes.c_char_p, _I64], _I),
    "FlashckGetInstanceParam": ([_I, ctypes.c_char_p, ctypes.POINTER(_I64)], _I),
}


def lib() -> ctypes.CDLL:
    """Loads the library once.  Raises if it has not been built (``python -m flashck_b200.build``)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m flashck_b200.build` "
                "(there is no CPU or PyTorch fallback for the attention path)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (argtypes, restype) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _LIB = handle
        apply_logging_flag()
    return _LIB


def apply_logging_flag() -> None:
    """FC_TUNING_LOG (core/utils/flags.cc:229) switches on the library's note on stderr whenever a forward call leaves
    the tcgen05 instance for the general one (the instance parameter ``log_fallback``).  No-op until the library is loaded."""
    if _LIB is None:
        return
    from .utils import flags
    _LIB.FlashckSetInstanceParam(0, b"log_fallback", 1 if flags.get_flag("FC_TUNING_LOG") else 0)


def last_error() -> str:
    return lib().FlashckGetLastError().decode()


def check(rc: int, what: str) -> None:
    if rc != 0:
        kind = {1: "invalid argument", 2: "unsupported problem", 3: "CUDA error", 4: "device timeout"}.get(rc, "error")
        raise RuntimeError(f"{what} failed ({kind}): {last_error()}")


def device_status() -> int:
    """Reads and clears the device status word (0: nothing to report; low 29 bits: a bounded device-side wait ran out;
    0x20000000: a work list overflowed; 0x40000000: append-KV skipped tokens that did not fit the cache)."""
    out = ctypes.c_int(0)
    rc = lib().FlashckDeviceStatus(ctypes.byref(out))
    if rc not in (0, 2, 4):  # 2 / 4: the word itself says what happened (skipped work / timeout)
        check(rc, "FlashckDeviceStatus")
    return out.value & 0xffffffff


def set_instance_param(family: int, key: str, value: int) -> None:
    check(lib().FlashckSetInstanceParam(family, key.encode(), int(value)), "FlashckSetInstanceParam")


def get_instance_param(family: int, key: str) -> int:
    out = _I64(0)
    check(lib().FlashckGetInstanceParam(family, key.encode(), ctypes.byref(out)), "FlashckGetInstanceParam")
    return out.value
