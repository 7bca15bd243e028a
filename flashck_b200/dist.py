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

Two exchanges exist.  :func:`sequence_sharded_decode` uses ``torch.distributed`` (NCCL over NVLink on GPUs, gloo in
the CPU tests): local merge kernel, ``all_gather_into_tensor``, final merge kernel.  :class:`ShardedDecoder` -- the fast
path -- replaces those three steps by one kernel of this library (``FmhaFwdSplitKVShardedCombine``) that merges the
local splits, stores the partial into every rank's exchange buffer through CUDA-IPC mapped peer pointers (plain
stores, a flag in every 8 bytes) and merges the ranks; its buffers are preallocated, nothing is allocated per step,
and the two launches of a step can be captured in a CUDA graph.  Nothing here issues TMA multicast.
"""
from __future__ import annotations

import ctypes
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
    "ShardedDecoder",
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


# ------------------------------------------------------------------------------------------------
# the fused exchange: one kernel for local merge + peer stores + final merge
# ------------------------------------------------------------------------------------------------
class ShardedDecoder:
    """Decode over a KV cache sharded by pages across the ranks of ``group``, two kernel launches per step: the
    split-KV kernel on this rank's pages, then ``FmhaFwdSplitKVShardedCombine``.

    Construction is collective (every rank of the group must do it, with the same shapes): it allocates this rank's
    exchange buffer with ``FlashckPeerBufferCreate``, all-gathers the 64-byte CUDA-IPC handles through
    ``torch.distributed`` and maps the peers' buffers.  With one rank (or no process group) the buffer is local and no
    handle is exchanged.  ``__call__`` allocates nothing: the split workspaces and the outputs are created once here.

        dec = ShardedDecoder(q.shape, dv, q.dtype, q.device, group=group)
        o, lse = dec(q, k_pool, v_pool, local_block_table, local_seqlen_k)     # o, lse are the decoder's own buffers
        dec.capture(q, k_pool, v_pool, local_block_table, local_seqlen_k)       # optional: the step as a CUDA graph
        o, lse = dec.replay()                                                   # after updating the inputs in place

    Every rank must make the same sequence of calls (a step waits, with a bound of about a second, for the partials of
    all ranks).  Call :meth:`close` on every rank when done."""

    def __init__(self, q_shape: Sequence[int], dv: int, dtype: torch.dtype, device, *, group=None, num_splits: int = 0,
                 hkv: int = 0):
        import torch.distributed as dist
        from . import _lib
        from .ops import fmha as F
        self._lib, self._F = _lib, F
        self.device = torch.device(device)
        b, sq, hq, _ = [int(x) for x in q_shape]
        self.shape = (b, sq, hq, int(dv))
        self.dtype = dtype
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        if self.world > 8:
            raise ValueError("ShardedDecoder serves the GPUs of one node (at most 8 ranks)")
        self.num_splits = int(num_splits) if num_splits and num_splits > 0 else \
            F.default_num_splits(b, rows_per_kv_head=sq * (hq // hkv) if hkv else 1)
        self.lse_acc = torch.empty((b, hq, self.num_splits, sq), dtype=torch.float32, device=self.device)
        self.o_acc = torch.empty((b, hq, self.num_splits, sq, dv), dtype=torch.float32, device=self.device)
        self.o = torch.empty((b, sq, hq, dv), dtype=dtype, device=self.device)
        self.lse = torch.empty((b, hq, sq), dtype=torch.float32, device=self.device)
        self._out_code = {torch.float16: 3, torch.bfloat16: 4, torch.float32: 7}[dtype]
        self._graph = None
        self._own = None
        self._opened: List[int] = []
        lib = _lib.lib()
        nbytes = lib.FlashckShardExchangeBytes(b, sq, hq, dv, self.world)
        with torch.cuda.device(self.device):
            if self.world == 1:
                self._local = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
                ptrs = [self._local.data_ptr()]
            else:
                own = ctypes.c_void_p(0)
                handle = ctypes.create_string_buffer(64)
                _lib.check(lib.FlashckPeerBufferCreate(nbytes, ctypes.byref(own), handle), "FlashckPeerBufferCreate")
                self._own = own.value
                handles: List[Optional[bytes]] = [None] * self.world
                dist.all_gather_object(handles, handle.raw, group=group)
                ptrs = []
                for r, h in enumerate(handles):
                    if r == self.rank:
                        ptrs.append(self._own)
                        continue
                    p = ctypes.c_void_p(0)
                    _lib.check(lib.FlashckPeerBufferOpen(ctypes.create_string_buffer(h, 64), ctypes.byref(p)),
                               f"FlashckPeerBufferOpen(rank {r})")
                    self._opened.append(p.value)
                    ptrs.append(p.value)
                dist.barrier(group=group)  # every rank has mapped every buffer before the first step
        self._bufs = (ctypes.c_void_p * self.world)(*ptrs)
        self._one = lambda t: (ctypes.c_void_p * 1)(t.data_ptr())

    # -- one step: split-KV on the local pages, then merge + exchange + merge
    def __call__(self, q, k_pool, v_pool, local_block_table, local_seqlen_k, *, scale: Optional[float] = None):
        b, sq, hq, dv = self.shape
        if tuple(q.shape[:3]) != (b, sq, hq):
            raise ValueError(f"q must be [{b}, {sq}, {hq}, d], got {tuple(q.shape)}")
        self._F.fmha_fwd_splitkv(q, k_pool, v_pool, seqlen_k=local_seqlen_k, block_table=local_block_table,
                                 num_splits=self.num_splits, scale=scale, workspace=(self.lse_acc, self.o_acc),
                                 combine=False)
        with torch.cuda.device(self.device):
            rc = self._lib.lib().FmhaFwdSplitKVShardedCombine(
                self._one(self.lse_acc), self._one(self.o_acc), self._one(self.o), self._one(self.lse), self._bufs,
                self.rank, 1, self.world, b, sq, hq, dv, self.num_splits, self._out_code,
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        self._lib.check(rc, "FmhaFwdSplitKVShardedCombine")
        return self.o, self.lse

    def capture(self, q, k_pool, v_pool, local_block_table, local_seqlen_k, *, scale: Optional[float] = None):
        """Captures the step on these tensors as a CUDA graph (after one ordinary step, so that one-time set-up of the
        kernels is done outside the capture).  Update the tensors in place, then :meth:`replay`."""
        self(q, k_pool, v_pool, local_block_table, local_seqlen_k, scale=scale)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self(q, k_pool, v_pool, local_block_table, local_seqlen_k, scale=scale)
        self._graph = graph
        return self

    def replay(self):
        if self._graph is None:
            raise RuntimeError("capture() first")
        self._graph.replay()
        return self.o, self.lse

    def close(self) -> None:
        """Unmaps the peers' buffers and frees this rank's (collective: a buffer is freed after every rank unmapped it)."""
        if self._bufs is None:
            return
        torch.cuda.synchronize(self.device)
        self._graph = None
        lib = self._lib.lib()
        with torch.cuda.device(self.device):
            for p in self._opened:
                lib.FlashckPeerBufferClose(ctypes.c_void_p(p))
            self._opened = []
            if self.distributed:
                import torch.distributed as dist
                dist.barrier(group=self.group)
            if self._own is not None:
                lib.FlashckPeerBufferFree(ctypes.c_void_p(self._own))
                self._own = None
        self._bufs = None
