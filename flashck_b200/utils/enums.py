"""Enumerations of the attention path, with the reference's values.

``MaskEnum`` = ``GenericAttentionMaskEnum`` (core/profiling/attention/fmha_library.h:81-87),
``BiasEnum`` (fmha_library.h:121-126), ``RopeEnum`` (fmha_library.h:195-200), ``FmhaKind`` (fmha_library.h:17-25),
``DataType`` (core/utils/dtype.h:16-28; the reference exposes it to Python in core/pybind/pybind_helper.h:3-16).
"""
from enum import IntEnum

__all__ = ["MaskEnum", "BiasEnum", "RopeEnum", "FmhaKind", "DataType"]


class MaskEnum(IntEnum):
    NO_MASK = 0
    MASK_FROM_TOP_LEFT = 1
    MASK_FROM_BOTTOM_RIGHT = 2
    MASK_GENERIC = 3


class BiasEnum(IntEnum):
    NO_BIAS = 0
    ELEMENTWISE_BIAS = 1
    ALIBI = 2


class RopeEnum(IntEnum):
    NONE = 0
    INTERLEAVED = 1
    HALF_ROTATED = 2


class FmhaKind(IntEnum):
    Fwd = 0
    FwdAppendKV = 1
    FwdSplitKV = 2
    FwdSplitKVCombine = 3
    BatchPrefill = 4
    PagedKVPrefill = 5


class DataType(IntEnum):
    BOOL = 0
    FLOAT8 = 1
    BFLOAT8 = 2
    FLOAT16 = 3
    BFLOAT16 = 4
    UINT32 = 5
    INT32 = 6
    FLOAT32 = 7
    UINT64 = 8
    INT64 = 9
    FLOAT64 = 10
