"""Utilities of the attention path: operation registry, enums and seeded input generators."""
from .flags import get_flag_value, print_all_flags, print_flag_info, set_flag_value
from .enums import BiasEnum, DataType, FmhaKind, MaskEnum, RopeEnum
from .registry import (FlashCKOperationType, get_available_operations, get_flashck_functions,
                       get_operation_function, is_available, register_flashck_functions)

__all__ = [
    "FlashCKOperationType", "is_available", "get_flashck_functions", "register_flashck_functions",
    "get_available_operations", "get_operation_function",
    "get_flag_value", "set_flag_value", "print_all_flags", "print_flag_info",
    "MaskEnum", "BiasEnum", "RopeEnum", "FmhaKind", "DataType",
]
