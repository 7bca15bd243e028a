"""``import flash_ck`` for code written against the reference's Python package.

The reference's package is ``flash_ck`` with sub-packages ``ops``, ``nn`` and ``utils`` (``flash_ck/__init__.py:8-35``).
:func:`install_as_flash_ck` registers this package under that name in ``sys.modules`` so that
``import flash_ck``, ``from flash_ck.ops import fmha_fwd`` or ``flash_ck.utils.is_available("fmha")`` resolve to the
B200 implementation.  It refuses to shadow a real ``flash_ck`` that is already imported.
"""
from __future__ import annotations

import sys

__all__ = ["install_as_flash_ck"]


def install_as_flash_ck(force: bool = False) -> None:
    import flashck_b200
    from flashck_b200 import nn, ops, utils

    existing = sys.modules.get("flash_ck")
    if existing is not None and existing is not flashck_b200 and not force:
        raise RuntimeError("a different 'flash_ck' module is already imported; pass force=True to replace it")
    sys.modules["flash_ck"] = flashck_b200
    sys.modules["flash_ck.ops"] = ops
    sys.modules["flash_ck.ops.fmha"] = ops.fmha
    sys.modules["flash_ck.nn"] = nn
    sys.modules["flash_ck.utils"] = utils
