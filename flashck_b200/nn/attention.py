"""Core-attention module over the functional API.

The reference's ``flash_ck.nn`` holds one module family, ``LayerNorm`` (``flash_ck/nn/norm/layer_norm.py:20``): a
``torch.nn.Module`` that validates its configuration in ``__init__``, looks its backend up in the registry
(``get_flashck_functions``, ``flash_ck/utils/utils.py:94-107``) and forwards to the functional operator.  This module
has the same structure for the attention family, with the parameter set of the reference's C++ ``AttentionLayer``
constructor (``core/module/layers/attention_layers/attention_layer.h:13-33``: mask, window, scale, head counts,
head dims).  It has no weights: the projections around the core attention are ordinary ``torch.nn.Linear`` layers
of the caller.  There is no PyTorch fallback: without the CUDA library every call raises.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from ..utils import FlashCKOperationType, get_flashck_functions
from ..utils.enums import RopeEnum

__all__ = ["FlashAttention"]


class FlashAttention(torch.nn.Module):
    """Scaled-dot-product attention with GQA, masks and an optional paged KV cache.

    Args:
        num_heads: query heads.
        head_dim: head dimension of Q and K.
        num_kv_heads: key/value heads (default ``num_heads``); ``num_heads`` must be a multiple of it.
        head_dim_v: head dimension of V (default ``head_dim``).
        causal: causal mask (bottom-right aligned when queries are fewer than keys, as decode and append need).
        window_size: ``(left, right)`` sliding window, ``-1`` = unbounded.
        scale: softmax scale; ``None`` = ``1/sqrt(head_dim)``.

    Shapes follow the reference (BSHD): q ``[b, sq, hq, d]``, k ``[b, sk, hkv, d]``, v ``[b, sk, hkv, dv]``;
    packed (varlen) inputs drop the batch axis and come with ``cu_seqlens``.
    """

    def __init__(self, num_heads: int, head_dim: int, num_kv_heads: Optional[int] = None,
                 head_dim_v: Optional[int] = None, causal: bool = False, window_size: Sequence[int] = (-1, -1),
                 scale: Optional[float] = None) -> None:
        super().__init__()
        num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        if num_heads <= 0 or num_kv_heads <= 0 or num_heads % num_kv_heads != 0:
            raise ValueError(f"num_heads ({num_heads}) must be a positive multiple of num_kv_heads ({num_kv_heads})")
        if head_dim <= 0 or (head_dim_v is not None and head_dim_v <= 0):
            raise ValueError("head dims must be positive")
        if len(tuple(window_size)) != 2:
            raise ValueError("window_size must be (left, right)")
        if scale is not None and not scale > 0:
            raise ValueError("scale must be positive")
        self.num_heads, self.num_kv_heads = int(num_heads), int(num_kv_heads)
        self.head_dim, self.head_dim_v = int(head_dim), int(head_dim if head_dim_v is None else head_dim_v)
        self.causal, self.window_size, self.scale = bool(causal), tuple(int(w) for w in window_size), scale

    # the registry is read at call time, so a module built before the library was loaded still works
    @staticmethod
    def _fn(name: str):
        fns = get_flashck_functions(FlashCKOperationType.FMHA.value)
        if fns is None or name not in fns:
            raise RuntimeError(f"flashck attention backend '{name}' is not registered (the CUDA library is required; "
                               "there is no PyTorch fallback)")
        return fns[name]

    def _check_heads(self, q: torch.Tensor, k: torch.Tensor) -> None:
        if q.shape[-2] != self.num_heads or q.shape[-1] != self.head_dim:
            raise ValueError(f"q must end in [{self.num_heads}, {self.head_dim}], got {tuple(q.shape)}")
        if k.shape[-2] != self.num_kv_heads:
            raise ValueError(f"k/v must have {self.num_kv_heads} heads, got {tuple(k.shape)}")

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: Optional[torch.Tensor] = None,
                cu_seqlens_k: Optional[torch.Tensor] = None, max_seqlen_q: int = 0, max_seqlen_k: int = 0,
                return_lse: bool = False):
        """Dense (4-D inputs) or variable-length (3-D packed inputs + ``cu_seqlens``) attention."""
        self._check_heads(q, k)
        kw = dict(scale=self.scale, causal=self.causal, window_size=self.window_size, return_lse=return_lse)
        if q.dim() == 4:
            if cu_seqlens_q is not None or cu_seqlens_k is not None:
                raise ValueError("cu_seqlens go with packed [total, heads, hdim] inputs")
            return self._fn("forward")(q, k, v, **kw)
        if cu_seqlens_q is None or cu_seqlens_k is None:
            raise ValueError("packed inputs need cu_seqlens_q and cu_seqlens_k")
        return self._fn("forward_var_len")(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, **kw)

    def forward_paged(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                      seqlen_k: torch.Tensor, cu_seqlens_q: Optional[torch.Tensor] = None, max_seqlen_q: int = 0,
                      decode: Optional[bool] = None, num_splits: int = 0, return_lse: bool = False):
        """Attention over a paged KV cache ``[pages, page, hkv, *]`` behind ``block_table`` / ``seqlen_k``.

        ``decode`` picks the split-KV path (few query tokens against long contexts); by default it is chosen when
        no sequence has more than 64 query rows per kv head, the most the split-KV kernel serves in one pass."""
        self._check_heads(q, k_cache)
        sq = max_seqlen_q if cu_seqlens_q is not None else (q.shape[1] if q.dim() == 4 else 0)
        if decode is None:
            decode = 0 < sq * (self.num_heads // self.num_kv_heads) <= 64
        if decode:
            return self._fn("forward_splitkv")(q, k_cache, v_cache, seqlen_k=seqlen_k, block_table=block_table,
                                               cu_seqlens_q=cu_seqlens_q, max_seqlen_q=max_seqlen_q,
                                               num_splits=num_splits, scale=self.scale, causal=self.causal,
                                               window_size=self.window_size, return_lse=return_lse)
        return self._fn("paged_kv_prefill")(q, k_cache, v_cache, block_table, seqlen_k, cu_seqlens_q=cu_seqlens_q,
                                            max_seqlen_q=max_seqlen_q, scale=self.scale, causal=self.causal,
                                            window_size=self.window_size, return_lse=return_lse)

    def append_kv(self, q: Optional[torch.Tensor], k_cache: torch.Tensor, v_cache: torch.Tensor, knew: torch.Tensor,
                  vnew: torch.Tensor, seqlen_k: torch.Tensor, rotary: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                  rope: int = RopeEnum.INTERLEAVED, **kwargs):
        """Rotates ``q`` and the new keys and writes the new K/V into the cache (``fmha_fwd_appendkv``)."""
        cos, sin = rotary if rotary is not None else (None, None)
        return self._fn("append_kv")(q, k_cache, v_cache, knew, vnew, seqlen_k, cos, sin,
                                     rope=rope if rotary is not None else RopeEnum.NONE, **kwargs)

    def extra_repr(self) -> str:
        return (f"num_heads={self.num_heads}, num_kv_heads={self.num_kv_heads}, head_dim={self.head_dim}, "
                f"head_dim_v={self.head_dim_v}, causal={self.causal}, window_size={self.window_size}, scale={self.scale}")
