"""Multi-rank host logic on CPU: sequence / page sharding and the all-gather + merge of per-rank partials, run as
two gloo ranks.  The per-rank attention itself is played by the CPU oracle (the CUDA kernels need a GPU); what is
under test is the partitioning, the gathered-buffer layout and the collective plumbing of flashck_b200.dist."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashck_b200 import dist as fdist
from flashck_b200.utils.inputs import make_paged_cache, normal_tensor
from oracle import cpu as oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem():
    lens = [1000, 37, 0, 513, 64]
    hq, hkv, d, page = 8, 2, 64, 16
    cache = make_paged_cache(lens, hkv, d, d, page, torch.bfloat16, seed=3)
    q = normal_tensor((len(lens), 1, hq, d), torch.bfloat16, 4)
    return lens, cache, q, (hq, hkv, d, page)


def _rank_main(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lens, cache, q, (hq, hkv, d, page) = _problem()
        b = len(lens)
        table, local_len = fdist.shard_pages(lens, cache.block_table, page, rank, world)
        o_r, lse_r = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=local_len, block_table=table)
        n = fdist.partial_numel(b, 1, hq, d)
        slot = torch.zeros(n, dtype=torch.float32)
        o_part, lse_part = fdist.split_partial_buffer(slot, b, 1, hq, d)
        o_part.copy_(o_r.float())
        lse_part.copy_(lse_r)
        gathered = fdist.gather_partials(slot)
        assert gathered.shape == (world, n)
        lse_acc, o_acc = fdist.gathered_to_workspaces(gathered, b, 1, hq, d)
        o, lse = oracle.splitkv_combine(lse_acc, o_acc, torch.bfloat16)
        o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
        ok_o = bool(((o.float() - o_ref.float()).abs() <= 2e-2 + 2e-2 * o_ref.float().abs()).all())
        fin = ~torch.isinf(lse_ref)
        ok_l = bool(torch.equal(torch.isinf(lse), torch.isinf(lse_ref)) and
                    ((lse[fin] - lse_ref[fin]).abs() <= 1e-3).all())
        # strides advertised for the GPU merge address the same elements as the re-laid workspaces
        ls, os_ = fdist.gathered_strides(n, 1, hq, d)
        flat = gathered.reshape(-1)
        no = b * 1 * hq * d
        bb, hh, ss = 3, 5, world - 1
        ok_s = bool(flat[no + bb * ls[0] + hh * ls[1] + ss * ls[2]] == lse_acc[bb, hh, ss, 0]) and \
            bool(torch.equal(flat[bb * os_[0] + hh * os_[1] + ss * os_[2]: bb * os_[0] + hh * os_[1] + ss * os_[2] + d],
                             o_acc[bb, hh, ss, 0]))
        ret[rank] = (ok_o, ok_l, ok_s)
    finally:
        dist.destroy_process_group()


def test_sequence_sharded_decode_two_gloo_ranks():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {0: (True, True, True), 1: (True, True, True)}


def test_shard_pages_covers_every_page_once():
    lens = [1000, 37, 0, 513, 64, 16]
    page = 16
    cache = make_paged_cache(lens, 1, 64, 64, page, torch.bfloat16, seed=1)
    for world in (1, 2, 3, 8):
        seen = [[] for _ in lens]
        total = [0] * len(lens)
        for rank in range(world):
            table, local = fdist.shard_pages(lens, cache.block_table, page, rank, world)
            for b in range(len(lens)):
                npg = -(-int(local[b]) // page)
                seen[b] += table[b, :npg].tolist()
                total[b] += int(local[b])
        assert total == lens
        for b, n in enumerate(lens):
            assert seen[b] == cache.block_table[b, :-(-n // page)].tolist()


def test_shard_sequences_balances_and_partitions():
    lens = [4096, 512, 3000, 700, 2500, 2500, 900, 100]
    for world in (1, 2, 4, 8):
        parts = [fdist.shard_sequences(lens, r, world) for r in range(world)]
        assert sorted(sum(parts, [])) == list(range(len(lens)))
        loads = [sum(lens[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(lens)
