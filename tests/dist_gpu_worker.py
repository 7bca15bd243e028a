"""One rank of the multi-GPU check of ShardedDecoder (launched by tests/test_dist_gpu.py under torchrun, one process
per GPU, NCCL for the set-up collectives): a sequence-sharded decode over real peer buffers -- eager calls and CUDA-graph
replays -- compared on every rank with the CPU oracle on the unsharded cache, and with the torch.distributed path
(merge kernel, all-gather, merge kernel).  Prints one JSON line per rank."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from flashck_b200 import _lib  # noqa: E402
from flashck_b200 import dist as fdist  # noqa: E402
from flashck_b200.utils.inputs import make_paged_cache, normal_tensor  # noqa: E402
from helpers import assert_lse_close, assert_o_close  # noqa: E402
from oracle import cpu as oracle  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    result = {"rank": rank, "world": world, "ok": False}
    try:
        dtype, hq, hkv, d, page = torch.bfloat16, 64, 8, 128, 64
        lens = [8192 + 33, 64 * world - 1, 0, 4096, 100]   # one context shorter than a page per rank, one empty
        cache = make_paged_cache(lens, hkv, d, d, page, dtype, seed=81)
        table, local_len = fdist.shard_pages(lens, cache.block_table, page, rank, world)
        k, v, bt, sl = cache.k.to(dev), cache.v.to(dev), table.to(dev), local_len.to(dev)
        dec = fdist.ShardedDecoder((len(lens), 1, hq, d), d, dtype, dev, hkv=hkv)
        qd = torch.empty(len(lens), 1, hq, d, dtype=dtype, device=dev)
        for call in range(4):  # eager steps: both halves of the exchange buffers, twice
            q = normal_tensor((len(lens), 1, hq, d), dtype, 90 + call)
            qd.copy_(q.to(dev))
            o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
            o, lse = dec(qd, k, v, bt, sl)
            torch.cuda.synchronize()
            assert_o_close(o, o_ref, f"eager call {call}")
            assert_lse_close(lse, lse_ref, f"LSE, eager call {call}")
            o2, lse2 = fdist.sequence_sharded_decode(qd, k, v, bt, sl, return_lse=True)
            assert_o_close(o2, o_ref, f"all-gather path, call {call}")
            assert_lse_close(lse2, lse_ref, f"LSE, all-gather path, call {call}")
        dec.capture(qd, k, v, bt, sl)
        for call in range(3):  # graph replays on fresh inputs
            q = normal_tensor((len(lens), 1, hq, d), dtype, 95 + call)
            qd.copy_(q.to(dev))
            o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
            o, lse = dec.replay()
            torch.cuda.synchronize()
            assert_o_close(o, o_ref, f"graph replay {call}")
            assert_lse_close(lse, lse_ref, f"LSE, graph replay {call}")
        status = _lib.device_status()
        assert status == 0, f"device status {status:#x}"
        dec.close()
        result["ok"] = True
    except Exception as e:  # reported, not raised: the other ranks must reach the barrier below
        result["error"] = f"{type(e).__name__}: {e}"
    print(json.dumps(result), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if result["ok"] else 1)


if __name__ == "__main__":
    main()
