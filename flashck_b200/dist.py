"""Multi-GPU use of the attention path: one process per GPU, ``torch.distributed`` for the plumbing.

The reference is single-GPU (no process groups, no collectives anywhere in its tree), so this module is new
design on top of the same operators:

* (batch, kv-head) units are independent, so prefill, append and ordinary decode shard *sequences* across the
  ranks with no collective on the data path (:func:`shard_sequences`).
* One long context is the exception: its KV pages are split contiguously over the ranks
  (:func:`shard_pages`); every rank runs the split-KV kernel on its pages and merges its own splits into an
  fp32 partial ``(O_r, LSE_r)``; one all-gather of ``b*hq*sq*(dv+1)`` floats per rank follows, and the same
  LSE-weighted merge with ``num_splits = world size`` yields O on every rank
  (:func:`sequence_sharded_decode`).  A rank whose shard is empty contributes ``LSE = -inf``.

The all-gather goes through ``torch.distributed`` (NCCL over NVLink on GPUs, gloo in the CPU tests); nothing here
issues TMA multicast or peer loads.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch

__all__ = [
    "shard_sequences",
    "shard_pages",
    "partial_numel",
    "split_partial_buffer",
    "gather_partials",
    "gathered_strides",
    "gathered_to_workspaces",
    "sequence_sharded_decode",
]


# ------------------------------------------------------------------------------------------------
# partitioning (pure host logic)
# ------------------------------------------------------------------------------------------------
def shard_sequences(seqlens: Sequence[int], rank: int, world: int) -> List[int]:
    """Indices of the sequences rank ``rank`` owns: longest-first greedy assignment to the least loaded rank
    (cost = length), so that ranks finish together; ties keep the input order.  Deterministic on every rank."""
    order = sorted(range(len(seqlens)), key=lambda i: (-int(seqlens[i]), i))
    load = [0] * world
    mine: List[int] = []
    for i in order:
        r = min(range(world), key=lambda x: (load[x], x))
        load[r] += int(seqlens[i])
        if r == rank:
            mine.append(i)
    return sorted(mine)


def shard_pages(seqlens: Sequence[int], block_table: torch.Tensor, page_block_size: int, rank: int,
                world: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Contiguous page shard of every sequence for ``rank``.

    Sequence b has ``P_b = ceil(len_b / page)`` pages; rank r owns pages ``[r*ceil(P_b/world), ...)`` (the last
    ranks may own none).  Returns ``(local_block_table [b, max_local_pages] int32, local_seqlen [b] int32)`` --
    page ids are unchanged, so the ranks can share one pool or hold only their own pages under the same ids."""
    rows, lens = [], []
    for b, n in enumerate(seqlens):
        pages = -(-int(n) // page_block_size)
        per = -(-pages // world) if pages else 0
        lo, hi = min(pages, rank * per), min(pages, (rank + 1) * per)
        rows.append(block_table[b, lo:hi])
        lens.append(max(0, min(int(n), hi * page_block_size) - lo * page_block_size))
    width = max(1, max(r.numel() for r in rows))
    out = torch.zeros((len(rows), width), dtype=torch.int32, device=block_table.device)
    for b, r in enumerate(rows):
        out[b, :r.numel()] = r
    return out, torch.tensor(lens, dtype=torch.int32, device=block_table.device)


# ------------------------------------------------------------------------------------------------
# the gathered buffer: per rank [ O_r fp32 (b, rows, hq, dv) | LSE_r fp32 (b, hq, rows) | pad ]
# ------------------------------------------------------------------------------------------------
def partial_numel(b: int, rows: int, hq: int, dv: int) -> int:
    """Floats one rank contributes, rounded up to a multiple of 4 (16-byte aligned slots)."""
    n = b * rows * hq * (dv + 1)
    return (n + 3) // 4 * 4


def split_partial_buffer(buf: torch.Tensor, b: int, rows: int, hq: int, dv: int):
    """Views ``(o_part [b, rows, hq, dv], lse_part [b, hq, rows])`` into one rank's flat slot."""
    no = b * rows * hq * dv
    return buf[:no].view(b, rows, hq, dv), buf[no:no + b * hq * rows].view(b, hq, rows)


def gather_partials(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gathers the flat per-rank slot; returns ``[world, n]``.  Without an initialised process group (one
    GPU) the result is the local slot alone."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local.view(1, -1)
    world = dist.get_world_size(group)
    out = torch.empty((world, local.numel()), dtype=local.dtype, device=local.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
    else:  # gloo (CPU tests) has no flat-tensor all-gather
        dist.all_gather([out[r] for r in range(world)], local.contiguous(), group=group)
    return out


def gathered_strides(n: int, rows: int, hq: int, dv: int):
    """Element strides (batch, head, split, row) of the O and LSE parts of a gathered ``[world, n]`` buffer, for
    ``FmhaFwdSplitKVCombineStrided`` (the split axis is the rank axis)."""
    return (hq * rows, rows, n, 1), (rows * hq * dv, dv, n, hq * dv)


def gathered_to_workspaces(gathered: torch.Tensor, b: int, rows: int, hq: int, dv: int):
    """The gathered buffer re-laid as the reference's workspaces ``lse_acc [b,hq,S,rows]``,
    ``o_acc [b,hq,S,rows,dv]`` (S = world).  Used by the CPU tests; the GPU path reads the buffer in place."""
    world = gathered.shape[0]
    no = b * rows * hq * dv
    o = gathered[:, :no].view(world, b, rows, hq, dv).permute(1, 3, 0, 2, 4).contiguous()
    lse = gathered[:, no:no + b * hq * rows].view(world, b, hq, rows).permute(1, 2, 0, 3).contiguous()
    return lse, o


# ------------------------------------------------------------------------------------------------
# sequence-sharded decode (GPU)
# ------------------------------------------------------------------------------------------------
def sequence_sharded_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                            local_block_table: torch.Tensor, local_seqlen_k: torch.Tensor, *, group=None,
                            num_splits: int = 0, scale: Optional[float] = None, return_lse: bool = False,
                            workspace=None, gather: Callable = gather_partials):
    """Decode (seqlen_q = 1 .. few) over a KV cache whose pages are sharded across the ranks of ``group``.

    ``q [b, sq, hq, d]`` is replicated; ``k_pool/v_pool`` hold (at least) this rank's pages;
    ``local_block_table`` / ``local_seqlen_k`` come from :func:`shard_pages`.  No mask is applied (a decode query
    sees the whole context).  Returns O ``[b, sq, hq, dv]`` in ``q.dtype`` (and LSE ``[b, hq, sq]``), identical on
    every rank."""
    from .ops import fmha as F

    b, sq, hq, _ = q.shape
    dv = v_pool.shape[-1]
    lse_acc, o_acc = F.fmha_fwd_splitkv(q, k_pool, v_pool, seqlen_k=local_seqlen_k, block_table=local_block_table,
                                        num_splits=num_splits, scale=scale, workspace=workspace, combine=False)
    n = partial_numel(b, sq, hq, dv)
    slot = torch.empty(n, dtype=torch.float32, device=q.device)
    if n > b * sq * hq * (dv + 1):
        slot[b * sq * hq * (dv + 1):].zero_()
    o_part, lse_part = split_partial_buffer(slot, b, sq, hq, dv)
    F.fmha_fwd_splitkv_combine(lse_acc, o_acc, torch.float32, out=o_part, lse_out=lse_part)  # local splits -> fp32
    gathered = gather(slot, group)
    world = gathered.shape[0]
    lse_strides, o_strides = gathered_strides(n, sq, hq, dv)
    return F.fmha_fwd_splitkv_combine_strided(gathered, b, sq, hq, dv, world, lse_offset=b * sq * hq * dv,
                                              lse_strides=lse_strides, o_strides=o_strides, dtype=q.dtype,
                                              return_lse=return_lse)
