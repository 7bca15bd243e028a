"""Seeded synthetic inputs for the attention path.

Restates the input generators embedded in FlashCK's profiler templates
(core/module/kernels/attention_kernels/fmha_common_jinja.h): ``to_seqstarts``
(:259-268), uniformly drawn sequence lengths (``randints`` :333-343), the block
table as a shuffled iota of physical page ids (``iota_shuffle`` :460-470, used at
fmha_fwd_split_kv/fmha_fwd_split_kv_jinja.h:550-551) and the rotary cos/sin tables
``[positions, rotary_dim/2]`` stored in the input dtype (:192-227).  Everything is
generated on the host with ``numpy`` / ``torch`` CPU generators so that the same
seed gives the same problem on every machine.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

__all__ = [
    "to_seqstarts",
    "uniform_seqlens",
    "iota_shuffle",
    "rotary_cos_sin",
    "random_rotary_cos_sin",
    "PagedCache",
    "make_paged_cache",
    "normal_tensor",
]


def to_seqstarts(seqlens: Sequence[int]) -> torch.Tensor:
    """Prefix sum with a leading zero, int64 ``[batch + 1]`` (fmha_common_jinja.h:259-268;
    the C ABI takes ``int64_t*`` seqstarts, fmha_fwd/fmha_fwd_call.h:14-16)."""
    out = np.zeros(len(seqlens) + 1, dtype=np.int64)
    np.cumsum(np.asarray(seqlens, dtype=np.int64), out=out[1:])
    return torch.from_numpy(out)


def uniform_seqlens(batch: int, low: int, high: int, seed: int) -> list[int]:
    """``batch`` integers uniform in ``[low, high]`` from a seeded generator."""
    rng = np.random.default_rng(seed)
    return [int(x) for x in rng.integers(low, high + 1, size=batch)]


def iota_shuffle(n: int, seed: int) -> torch.Tensor:
    """A seeded random permutation of ``0..n-1`` as int32 (fmha_common_jinja.h:460-470)."""
    rng = np.random.default_rng(seed)
    return torch.from_numpy(rng.permutation(n).astype(np.int32))


def rotary_cos_sin(max_pos: int, rotary_dim: int, dtype: torch.dtype, base: float = 10000.0):
    """RoPE tables ``[max_pos, rotary_dim/2]``: angle(pos, i) = pos * base**(-2i/rotary_dim),
    computed in fp32 on the host and stored in ``dtype`` like the reference's tables."""
    i = torch.arange(rotary_dim // 2, dtype=torch.float32)
    inv_freq = torch.pow(torch.tensor(base, dtype=torch.float32), -2.0 * i / rotary_dim)
    ang = torch.arange(max_pos, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)


def random_rotary_cos_sin(seqlen: int, rotary_dim: int, dtype: torch.dtype, seed: int):
    """The reference generator's tables: ``[2*seqlen, rotary_dim/2]`` of cos/sin of angles
    uniform in ``[0, 2*pi)`` (fmha_common_jinja.h:205-224)."""
    g = torch.Generator().manual_seed(seed)
    ang = torch.rand(2 * seqlen, rotary_dim // 2, generator=g, dtype=torch.float32) * (2 * math.pi)
    return torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)


def normal_tensor(shape, dtype: torch.dtype, seed: int) -> torch.Tensor:
    """N(0,1) values drawn in fp32 from a seeded CPU generator, then rounded to ``dtype``."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32).to(dtype)


@dataclass
class PagedCache:
    """A paged K/V pool and its block table in the reference's layout
    (fmha_fwd_split_kv_jinja.h:512-519,550): pools ``[num_pages, page, hkv, d]``,
    ``block_table`` int32 ``[batch, max_pages_per_seq]``, ``seqlen_k`` int32 ``[batch]``."""

    k: torch.Tensor
    v: torch.Tensor
    block_table: torch.Tensor
    seqlen_k: torch.Tensor
    page_block_size: int

    @property
    def max_num_page_blocks(self) -> int:
        # the reference passes batch * pages_per_seq and divides by batch for the row stride
        return int(self.block_table.shape[0] * self.block_table.shape[1])


def make_paged_cache(seqlens: Sequence[int], hkv: int, d: int, dv: int, page_block_size: int,
                     dtype: torch.dtype, seed: int, capacity: Optional[Sequence[int]] = None,
                     fill: bool = True) -> PagedCache:
    """Pool sized to the total page count; the block table is a seeded random permutation of the
    physical page ids, handed out row by row.  ``capacity`` (tokens per sequence, >= seqlens)
    reserves extra pages, e.g. for tokens appended later.  Unused table slots hold -1."""
    cap = list(capacity) if capacity is not None else list(seqlens)
    pages = [max(1, -(-c // page_block_size)) for c in cap]
    total = sum(pages)
    perm = iota_shuffle(total, seed)
    table = torch.full((len(seqlens), max(pages)), -1, dtype=torch.int32)
    off = 0
    for b, p in enumerate(pages):
        table[b, :p] = perm[off:off + p]
        off += p
    if fill:
        k = normal_tensor((total, page_block_size, hkv, d), dtype, seed + 1)
        v = normal_tensor((total, page_block_size, hkv, dv), dtype, seed + 2)
    else:
        k = torch.zeros((total, page_block_size, hkv, d), dtype=dtype)
        v = torch.zeros((total, page_block_size, hkv, dv), dtype=dtype)
    return PagedCache(k, v, table, torch.tensor(list(seqlens), dtype=torch.int32), page_block_size)
