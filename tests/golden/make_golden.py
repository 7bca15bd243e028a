"""Generates the golden fixtures in this folder from the CPU oracle on seeded inputs.

The reference ships no golden vectors for its attention path (its FMHA test files are empty), so these
fixtures pin the oracle against itself over time ("parity unpinned" against the reference): a change in
the oracle's arithmetic or conventions shows up as a diff here.  Inputs are regenerated from the seeds, only
outputs are stored (fp16/bf16 payloads as int16 words).

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from flashck_b200.utils.inputs import make_paged_cache, normal_tensor, rotary_cos_sin, to_seqstarts  # noqa: E402
from oracle import cpu as oracle  # noqa: E402


def words(t):
    return t.contiguous().view(torch.int16).numpy()


def case_config1():
    """BASELINE config 1: fp16, b=2, h=8, s=128, hdim=64, causal, scale 1/8."""
    q, k, v = (normal_tensor((2, 128, 8, 64), torch.float16, 100 + i) for i in range(3))
    return q, k, v


def case_paged_decode():
    lens = [1, 15, 16, 17, 127, 129, 1000, 0]
    cache = make_paged_cache(lens, 2, 128, 128, 16, torch.bfloat16, seed=7)
    q = normal_tensor((len(lens), 1, 8, 128), torch.bfloat16, 41)
    return q, cache


def case_append():
    lens, new = [0, 5, 16, 31], [3, 16, 1, 2]
    cap = [a + b for a, b in zip(lens, new)]
    cache = make_paged_cache(lens, 2, 64, 64, 16, torch.bfloat16, seed=12, capacity=cap)
    cu = to_seqstarts(new)
    total = int(cu[-1])
    q = normal_tensor((total, 4, 64), torch.bfloat16, 81)
    knew = normal_tensor((total, 2, 64), torch.bfloat16, 82)
    vnew = normal_tensor((total, 2, 64), torch.bfloat16, 83)
    cos, sin = rotary_cos_sin(max(cap) + 1, 64, torch.bfloat16)
    return q, knew, vnew, cache, cu, cos, sin


def main():
    q, k, v = case_config1()
    o, lse = oracle.fmha_fwd(q, k, v, scale=0.125, mask_type=1, window=(-1, 0))
    np.savez_compressed(os.path.join(HERE, "config1_fp16_causal.npz"), o=words(o), lse=lse.numpy())

    q, cache = case_paged_decode()
    o, lse = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
    np.savez_compressed(os.path.join(HERE, "paged_decode_bf16.npz"), o=words(o), lse=lse.numpy())

    q, knew, vnew, cache, cu, cos, sin = case_append()
    oracle.fmha_fwd_appendkv(q, cache.k, knew, cache.v, vnew, cache.seqlen_k, cos, sin, rope_type=1,
                             block_table=cache.block_table, seqstart_q=cu, seqstart_knew=cu)
    np.savez_compressed(os.path.join(HERE, "appendkv_bf16_interleaved.npz"), q=words(q), k=words(cache.k),
                        v=words(cache.v))


if __name__ == "__main__":
    main()
