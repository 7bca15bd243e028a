"""Modules (the reference's ``flash_ck.nn``), attention family only."""
from .attention import FlashAttention

__all__ = ["FlashAttention"]
