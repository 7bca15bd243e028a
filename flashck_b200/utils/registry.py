"""Operation registry -- mirrors ``flash_ck/utils/utils.py`` of the reference (FlashCKOperationType :22-26,
``is_available`` :78-91, ``get_flashck_functions`` :94-107, ``register_flashck_functions`` :110-121,
``get_available_operations`` :124-131, ``get_operation_function`` :134-149).

The reference leaves the ``fmha`` slot as a commented placeholder (:50-59); here it is filled when the CUDA
library loads.  Unlike the norm operators there is no ``with_flashck_fallback``: the attention path never
falls back to PyTorch.
"""
from __future__ import annotations

from enum import Enum
from typing import Callable, Dict, Optional

__all__ = [
    "FlashCKOperationType",
    "is_available",
    "get_flashck_functions",
    "register_flashck_functions",
    "get_available_operations",
    "get_operation_function",
]


class FlashCKOperationType(Enum):
    """Operation families, with the reference's string values."""
    LAYER_NORM = "layer_norm"
    FMHA = "fmha"
    GEMM = "gemm"


_FLASHCK_FUNCTIONS: Dict[str, Dict[str, Callable]] = {}
_FLASHCK_AVAILABILITY: Dict[str, bool] = {t.value: False for t in FlashCKOperationType}


def is_available(operation_type: Optional[str] = None) -> bool:
    """True if the operation family (or, with ``None``, any family) has a registered backend."""
    if operation_type is None:
        return any(_FLASHCK_AVAILABILITY.values())
    return _FLASHCK_AVAILABILITY.get(operation_type, False)


def get_flashck_functions(operation_type: str) -> Optional[Dict[str, Callable]]:
    if not is_available(operation_type):
        return None
    return _FLASHCK_FUNCTIONS.get(operation_type)


def register_flashck_functions(operation_type: str, functions: Dict[str, Callable]) -> None:
    _FLASHCK_FUNCTIONS[operation_type] = dict(functions)
    _FLASHCK_AVAILABILITY[operation_type] = True


def get_available_operations() -> Dict[str, bool]:
    return _FLASHCK_AVAILABILITY.copy()


def get_operation_function(operation_type: str, function_name: str) -> Optional[Callable]:
    functions = get_flashck_functions(operation_type)
    if functions is None:
        return None
    return functions.get(function_name)
