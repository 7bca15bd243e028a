#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload prefill|decode]

Headline workload (N=1): BASELINE config 2 -- varlen causal batch prefill, bf16, batch 16, 32 q heads / 8 kv
heads, hdim 128, lengths uniform in [512, 4096] from a seed.  `value` is causal-effective TFLOP/s
(4*d*hq*sum L(L+1)/2 FLOP per step) with inputs resident in HBM; `e2e` is the same metric through the public
API with pinned host buffers, host<->device copies inside the timed region.  The same run also measures
BASELINE config 3 (paged split-KV decode, HBM GB/s) and reports it under `extra.decode`.
With N > 1 (torchrun, one rank per GPU) every rank runs a batch of the same lengths with its own values (no
collective on the data path; weak scaling) and `extra.long_decode` runs BASELINE config 5: one long context sharded by pages across the ranks,
partial O/LSE merged after one NCCL all-gather.

`--impl reference` times the CPU statement of the same path (the oracle; the reference's own kernels need
ROCm + ck_tile and cannot run here) on the host cores, on a bounded sample of the same workload.
All inputs are synthetic (seeded N(0,1)), as the reference's own profiler generates them.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from flashck_b200.utils.inputs import iota_shuffle, to_seqstarts, uniform_seqlens  # noqa: E402

HQ, HKV, D = 32, 8, 128
# threads of the CPU baseline: all host cores, set explicitly (torchrun exports OMP_NUM_THREADS=1)
HOST_THREADS = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_traffic(key: str, scale: float = 1.0):
    """DRAM bytes per launch of a kernel from its committed ncu capture (`profiles/traffic.json`), or None when the
    kernel's source has changed since the capture (the record carries the SHA-256 of the source files it was taken
    from), so that a stale figure is never printed beside a fresh timing."""
    import hashlib
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f)[key]
        for rel, want in rec["source_sha256"].items():
            with open(os.path.join(ROOT, rel), "rb") as f:
                if hashlib.sha256(f.read()).hexdigest() != want:
                    return None
        return rec["dram_bytes_per_launch"] * scale
    except (OSError, KeyError, ValueError):
        return None


# ----------------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU every 200 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        med = sm[len(sm) // 2] if sm else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------------------------------
def make_prefill(seed: int, device, batch=16, lo=512, hi=4096, data_seed=None):
    """`seed` fixes the lengths (the same on every rank, so that the ranks of a weak-scaling run carry equal work);
    `data_seed` the values."""
    lens = uniform_seqlens(batch, lo, hi, seed)
    cu = to_seqstarts(lens)
    total = int(cu[-1])
    g = torch.Generator(device=device).manual_seed(seed if data_seed is None else data_seed)
    q = torch.randn(total, HQ, D, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn(total, HKV, D, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn(total, HKV, D, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    flops = 4.0 * D * HQ * sum(L * (L + 1) / 2 for L in lens)
    return {"lens": lens, "cu": cu.to(device), "q": q, "k": k, "v": v, "flops": flops, "total": total,
            "max_len": max(lens)}


def make_paged_prefill(w, page: int, seed: int, device):
    """The K/V of a packed prefill workload scattered into paged pools [pages, page, hkv, d] behind a shuffled block
    table (a `next` row: prefill reading K/V through the page table, as in a serving loop)."""
    lens = w["lens"]
    pages = [-(-L // page) for L in lens]
    perm = iota_shuffle(sum(pages), seed)
    table = torch.zeros((len(lens), max(pages)), dtype=torch.int32)
    slot = torch.empty(w["total"], dtype=torch.int64)
    off = tok = 0
    for b, (L, n) in enumerate(zip(lens, pages)):
        table[b, :n] = perm[off:off + n]
        j = torch.arange(L)
        slot[tok:tok + L] = perm[off:off + n].to(torch.int64)[j // page] * page + j % page
        off += n
        tok += L
    slot = slot.to(device)
    kpool = torch.zeros(sum(pages) * page, HKV, D, device=device, dtype=torch.bfloat16)
    vpool = torch.zeros_like(kpool)
    kpool[slot] = w["k"]
    vpool[slot] = w["v"]
    return {"k": kpool.view(-1, page, HKV, D), "v": vpool.view(-1, page, HKV, D), "table": table.to(device),
            "seqlen": torch.tensor(lens, dtype=torch.int32, device=device), "page": page}


def make_decode(seed: int, device, batch=64, lo=1024, hi=32768, page=16, hq=HQ, hkv=HKV, lens=None, data_seed=None):
    lens = lens or uniform_seqlens(batch, lo, hi, seed)
    batch = len(lens)
    pages = [-(-L // page) for L in lens]
    total_pages = sum(pages)
    data_seed = seed if data_seed is None else data_seed
    perm = iota_shuffle(total_pages, data_seed)
    table = torch.zeros((batch, max(pages)), dtype=torch.int32)
    off = 0
    for b, n in enumerate(pages):
        table[b, :n] = perm[off:off + n]
        off += n
    g = torch.Generator(device=device).manual_seed(data_seed + 1)
    kpool = torch.empty(total_pages, page, hkv, D, device=device, dtype=torch.bfloat16)
    vpool = torch.empty(total_pages, page, hkv, D, device=device, dtype=torch.bfloat16)
    chunk = max(1, (1 << 28) // (page * hkv * D))  # fill in pieces: fp32 randn of the whole pool would double memory
    for s in range(0, total_pages, chunk):
        e = min(total_pages, s + chunk)
        kpool[s:e] = torch.randn(e - s, page, hkv, D, generator=g, device=device, dtype=torch.float32)
        vpool[s:e] = torch.randn(e - s, page, hkv, D, generator=g, device=device, dtype=torch.float32)
    q = torch.randn(batch, 1, hq, D, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    kv_bytes = sum(lens) * hkv * 2 * D * 2
    algo_bytes = kv_bytes + q.numel() * 2 * 2 + 4 * total_pages  # K+V once, Q read, O write, block table
    return {"lens": lens, "q": q, "k": kpool, "v": vpool, "table": table.to(device),
            "seqlen": torch.tensor(lens, dtype=torch.int32, device=device), "bytes": float(algo_bytes),
            "page": page, "hq": hq, "hkv": hkv}


def make_append_decode(seed: int, device, batch=32, lo=2048, hi=16384, page=16, data_seed=None):
    """BASELINE config 4: a paged cache holding `ctx` tokens per sequence with room for 1..16 appended ones."""
    from flashck_b200.utils.inputs import rotary_cos_sin
    ctx = uniform_seqlens(batch, lo, hi, seed)
    new = uniform_seqlens(batch, 1, 16, seed + 1)
    cap = [c + n for c, n in zip(ctx, new)]
    data_seed = seed if data_seed is None else data_seed
    w = make_decode(seed + 2, device, lens=cap, page=page, data_seed=data_seed + 2)
    total = sum(new)
    g = torch.Generator(device=device).manual_seed(data_seed + 3)
    mk = lambda h: torch.randn(total, h, D, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    cos, sin = rotary_cos_sin(max(cap) + 1, D, torch.bfloat16)
    w.update({"ctx": ctx, "new": new, "qn": mk(HQ), "kn": mk(HKV), "vn": mk(HKV), "cu_new": to_seqstarts(new).to(device),
              "ctx_len": torch.tensor(ctx, dtype=torch.int32, device=device), "cos": cos.to(device), "sin": sin.to(device),
              "append_bytes": float(total * (2 * HKV * D * 2 * 2 + 2 * HQ * D * 2))})
    return w


def make_long_decode(seed: int, device, world: int, batch=4, ctx=524288, page=64, hq=64, hkv=8):
    """BASELINE config 5: this rank's contiguous page shard of `batch` contexts of `ctx` tokens (1/world of each)."""
    local = ctx // world
    w = make_decode(seed, device, lens=[local] * batch, page=page, hq=hq, hkv=hkv)
    w["total_bytes"] = float(batch * ctx * hkv * 2 * D * 2)
    return w


def sharded_decode_parity(fdist, ops, device, rank, world):
    """A small sequence-sharded decode (4 contexts of up to 8192 tokens, page 64, 64 q / 8 kv heads) through the code path
    the long-context leg times -- ShardedDecoder on every rank of the job, eager and replayed from a CUDA graph -- with
    rank 0's result checked against the CPU oracle on the unsharded cache."""
    from flashck_b200.utils.inputs import make_paged_cache, normal_tensor
    lens, hq, hkv, page = [8192, 4097, 64, 8000], 64, 8, 64
    cache = make_paged_cache(lens, hkv, D, D, page, torch.bfloat16, seed=55)  # the same cache on every rank
    q = normal_tensor((len(lens), 1, hq, D), torch.bfloat16, 56)
    table, local_len = fdist.shard_pages(lens, cache.block_table, page, rank, world)
    qd, kd, vd = q.to(device), cache.k.to(device), cache.v.to(device)
    dec = fdist.ShardedDecoder(qd.shape, D, torch.bfloat16, device, hkv=hkv)
    out = {}
    try:
        o, lse = dec(qd, kd, vd, table.to(device), local_len.to(device))
        res = {"eager": (o.float().cpu(), lse.cpu())}
        dec.capture(qd, kd, vd, table.to(device), local_len.to(device))
        o, lse = dec.replay()
        torch.cuda.synchronize()
        res["graph"] = (o.float().cpu(), lse.cpu())
        from flashck_b200 import _lib
        status = _lib.device_status()
        if rank == 0:
            from oracle import cpu as oracle  # the checker, on rank 0 only
            o_ref, lse_ref = oracle.fmha_fwd(q, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
            o_ref = o_ref.float()
            ok = status == 0
            for name, (o, lse) in res.items():
                eo = float(((o - o_ref).abs() - 2e-2 * o_ref.abs()).max())
                el = float((lse - lse_ref).abs().max())
                out[f"max_o_err_beyond_rel_{name}"] = eo
                out[f"max_lse_err_{name}"] = el
                ok = ok and eo <= 2e-2 and el <= 1e-3 and bool(torch.isfinite(o).all())
            out["parity_ok"] = bool(ok)
            out["device_status"] = status
            out["checked"] = f"rank 0 of {world}: O within 2e-2 abs/rel, LSE within 1e-3 of the oracle on the unsharded cache"
    finally:
        dec.close()
    return out


def library_prefill_baselines(w, steps):
    """The config 2 workload through the attention kernels that ship with the image, for context beside the roofline
    fraction: PyTorch's scaled_dot_product_attention on the cuDNN backend (NVIDIA's own Blackwell attention kernels; one
    call per sequence, no LSE) and flash_attn's varlen kernel (mma.sync).  Library code, not part of the product path."""
    out = {"note": "same seeded tensors and causal-effective FLOP count as the headline; rank 0 only"}
    try:
        import torch.nn.functional as F
        from torch.nn.attention import SDPBackend, sdpa_kernel
        cu = w["cu"].cpu().tolist()
        seqs = [tuple(w[n][cu[b]:cu[b + 1]].transpose(0, 1)[None].contiguous() for n in ("q", "k", "v"))
                for b in range(len(w["lens"]))]

        def run():
            for q, k, v in seqs:
                F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
            ms = time_steps(run, steps, 3) / steps
        out["torch_sdpa_cudnn"] = {"ms_per_step": ms, "tflops": w["flops"] / ms / 1e9, "launches_per_step": len(seqs)}
    except Exception as e:  # noqa: BLE001 -- a missing backend must not take the bench down
        out["torch_sdpa_cudnn"] = {"unavailable": f"{type(e).__name__}: {str(e)[:120]}"}
    try:
        # one batched call (4 x 4096 tokens, the head geometry of config 2): the library kernel without its 16 launches,
        # next to this repository's kernel on the same tensors
        import torch.nn.functional as F
        from torch.nn.attention import SDPBackend, sdpa_kernel
        from flashck_b200 import ops
        b, L = 4, 4096
        g = torch.Generator(device=w["q"].device).manual_seed(99)
        q, k, v = (torch.randn(b, L, h, D, generator=g, device=w["q"].device, dtype=torch.float32).to(torch.bfloat16)
                   for h in (HQ, HKV, HKV))
        qt, kt, vt = (x.transpose(1, 2) for x in (q, k, v))
        fl = 4.0 * D * HQ * b * L * (L + 1) / 2
        ms_own = time_steps(lambda: ops.fmha_fwd(q, k, v, causal=True, return_lse=True), steps, 3) / steps
        with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
            ms_lib = time_steps(lambda: F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=True), steps, 3) / steps
        out["batched_4x4096_causal"] = {"this_repo": {"ms": ms_own, "tflops": fl / ms_own / 1e9},
                                        "torch_sdpa_cudnn": {"ms": ms_lib, "tflops": fl / ms_lib / 1e9}}
        del q, k, v, qt, kt, vt
    except Exception as e:  # noqa: BLE001
        out["batched_4x4096_causal"] = {"unavailable": f"{type(e).__name__}: {str(e)[:120]}"}
    try:
        from flash_attn import flash_attn_varlen_func
        cu32 = w["cu"].to(torch.int32)

        def run_fa():
            flash_attn_varlen_func(w["q"], w["k"], w["v"], cu32, cu32, w["max_len"], w["max_len"], causal=True)
        ms = time_steps(run_fa, steps, 3) / steps
        out["flash_attn_varlen"] = {"ms_per_step": ms, "tflops": w["flops"] / ms / 1e9, "launches_per_step": 1}
    except Exception as e:  # noqa: BLE001
        out["flash_attn_varlen"] = {"unavailable": f"{type(e).__name__}: {str(e)[:120]}"}
    return out


def time_steps(fn, steps, warmup, barrier=None):
    """Device time of `steps` calls of fn, in ms (CUDA events on the current stream)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    beg.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return beg.elapsed_time(end)


# ----------------------------------------------------------------------------------------------------
# CPU baseline (the oracle) -- only this leg and the reference arm touch oracle/
# ----------------------------------------------------------------------------------------------------
def cpu_prefill_sample(w, budget_flops=1.5e12):
    from oracle import cpu as oracle
    lens, cu = w["lens"], w["cu"].cpu()
    chosen, fl = [], 0.0
    for b in sorted(range(len(lens)), key=lambda i: lens[i]):
        f = 4.0 * D * HQ * lens[b] * (lens[b] + 1) / 2
        if chosen and fl + f > budget_flops:
            break
        chosen.append(b)
        fl += f
    parts = [slice(int(cu[b]), int(cu[b + 1])) for b in chosen]
    q = torch.cat([w["q"][s] for s in parts]).cpu()
    k = torch.cat([w["k"][s] for s in parts]).cpu()
    v = torch.cat([w["v"][s] for s in parts]).cpu()
    cu_s = to_seqstarts([lens[b] for b in chosen])
    t0 = time.perf_counter()
    oracle.fmha_fwd(q, k, v, seqstart_q=cu_s, seqstart_k=cu_s, mask_type=1, window=(-1, 0), nthreads=HOST_THREADS)
    dt = time.perf_counter() - t0
    return {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": HOST_THREADS, "kind": "port",
            "sample": f"{len(chosen)} shortest of {len(lens)} sequences ({sum(lens[b] for b in chosen)} tokens, "
                      f"{fl:.3g} FLOP) in {dt:.2f} s", "seconds": dt}


def cpu_decode_sample(w, nseq=48):
    from oracle import cpu as oracle
    lens = w["lens"][:nseq]
    page = w["page"]
    # compact the pages of the sampled sequences into a small host pool
    table = w["table"][:nseq].cpu()
    npages = [-(-L // page) for L in lens]
    ids = torch.cat([table[b, :n] for b, n in enumerate(npages)]).long()
    kpool, vpool = w["k"][ids.to(w["k"].device)].cpu(), w["v"][ids.to(w["k"].device)].cpu()
    new_table = torch.zeros((nseq, max(npages)), dtype=torch.int32)
    off = 0
    for b, n in enumerate(npages):
        new_table[b, :n] = torch.arange(off, off + n, dtype=torch.int32)
        off += n
    q = w["q"][:nseq].cpu()
    sl = torch.tensor(lens, dtype=torch.int32)
    t0 = time.perf_counter()
    oracle.fmha_fwd(q, kpool, vpool, seqlen_k=sl, block_table=new_table, nthreads=HOST_THREADS)
    dt = time.perf_counter() - t0
    nbytes = sum(lens) * w["hkv"] * 2 * D * 2
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": HOST_THREADS, "kind": "port",
            "sample": f"first {nseq} of {len(w['lens'])} sequences ({sum(lens)} tokens) in {dt:.2f} s", "seconds": dt}


# ----------------------------------------------------------------------------------------------------
def run_reference(args, rank):
    """Reference arm: the CPU statement of the path on the host cores (rank 0 only), on the same workload as the GPU
    arm: every step is all 16 sequences of BASELINE config 2 (about 4 s on 16 cores)."""
    if rank != 0:
        return
    dev = torch.device("cpu")
    w = make_prefill(1234, dev)
    samples = []
    for _ in range(args.warmup):
        cpu_prefill_sample(w, budget_flops=float("inf"))
    t_all = 0.0
    for _ in range(args.steps):
        s = cpu_prefill_sample(w, budget_flops=float("inf"))
        samples.append(s)
        t_all += s["seconds"]
    val = w["flops"] * args.steps / t_all / 1e12
    line = {
        "impl": "reference", "metric": "prefill_fmha_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_all / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "varlen causal batch prefill (BASELINE config 2): batch 16, 32 q / 8 kv heads, "
                               "hdim 128, L~U[512,4096] from seed 1234",
                   "tokens_per_gpu": w["total"], "flops_per_gpu_step": w["flops"],
                   "flop_count": "causal-effective 4*d*hq*sum L(L+1)/2",
                   "note": "CPU statement of the path (oracle port) on the whole workload, all host threads; the "
                           "reference's own kernels need ROCm + ck_tile"},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": HOST_THREADS, "kind": "port",
                         "sample": samples[-1]["sample"]},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--small", action="store_true", help="reduced sizes (for profiler captures)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    from flashck_b200 import _lib, ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    peaks = load_peaks()
    steps, warmup = args.steps, max(args.warmup, 3)

    # ------------------------------------------------------------------ prefill (headline)
    if args.small:
        w = make_prefill(1234, device, batch=4, lo=512, hi=2048, data_seed=1234 + rank)
    else:
        w = make_prefill(1234, device, data_seed=1234 + rank)

    def prefill_step():
        return ops.fmha_fwd_var_len(w["q"], w["k"], w["v"], w["cu"], w["cu"], w["max_len"], causal=True,
                                    return_lse=True)

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = time_steps(prefill_step, steps, warmup, barrier)
    ms = max_over_ranks(ms)
    clocks = sampler.stop()
    total_flops = sum_over_ranks(w["flops"])
    value = total_flops * steps / (ms * 1e-3) / 1e12
    kernel_tflops = w["flops"] * steps / (ms * 1e-3) / 1e12  # per GPU; the step is one kernel launch

    # e2e: pinned host inputs -> device -> kernel -> host outputs, every step.  The three legs of a step run on a
    # stream each (copy in, compute, copy out) over two sets of device buffers, the way a serving loop feeds a GPU: the
    # copy of the next step's inputs and the read-back of the previous step's result overlap this step's kernel, and
    # the step time tends to the slowest leg instead of their sum.  Every step still moves all of its inputs and results.
    hq_, hk_, hv_ = (w[n].cpu().pin_memory() for n in ("q", "k", "v"))
    dbuf = [tuple(torch.empty_like(w[n]) for n in ("q", "k", "v")) for _ in range(2)]
    ho = [torch.empty_like(hq_).pin_memory() for _ in range(2)]
    hl = [torch.empty((HQ, w["total"]), dtype=torch.float32).pin_memory() for _ in range(2)]
    s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_run = [torch.cuda.Event() for _ in range(2)]
    e2e_count = [0]

    def prefill_e2e():
        i = e2e_count[0]
        e2e_count[0] += 1
        b = i & 1
        dq, dk, dv_ = dbuf[b]
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_run[b])   # the kernel that read this buffer set two steps ago is done
            dq.copy_(hq_, non_blocking=True)
            dk.copy_(hk_, non_blocking=True)
            dv_.copy_(hv_, non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_in[b])
            o, lse = ops.fmha_fwd_var_len(dq, dk, dv_, w["cu"], w["cu"], w["max_len"], causal=True, return_lse=True)
            ev_run[b].record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_run[b])
            ho[b].copy_(o, non_blocking=True)  # (same stream as two steps ago: that copy into ho[b] is over)
            hl[b].copy_(lse, non_blocking=True)
            o.record_stream(s_out)
            lse.record_stream(s_out)

    def e2e_region(n):
        """n pipelined steps between two events on the current stream; the side streams start after the first event and
        the second one waits for all of them."""
        cur = torch.cuda.current_stream()
        beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        beg.record(cur)
        for st in (s_in, s_run, s_out):
            st.wait_event(beg)
        for _ in range(n):
            prefill_e2e()
        for st in (s_in, s_run, s_out):
            done = torch.cuda.Event()
            done.record(st)
            cur.wait_event(done)
        end.record(cur)
        torch.cuda.synchronize()
        return beg.elapsed_time(end)

    e2e_steps = max(3, min(steps, 10))
    e2e_region(3)  # warm-up
    if barrier:
        barrier()
    torch.cuda.synchronize()
    ms_e2e = max_over_ranks(e2e_region(e2e_steps))
    if barrier:
        barrier()
    e2e_val = total_flops * e2e_steps / (ms_e2e * 1e-3) / 1e12
    h2d = (hq_.numel() + hk_.numel() + hv_.numel()) * 2
    d2h = ho[0].numel() * 2 + hl[0].numel() * 4
    del hq_, hk_, hv_, dbuf, ho, hl

    line = {
        "metric": "prefill_fmha_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "varlen causal batch prefill (BASELINE config 2): batch 16 per GPU, 32 q / 8 kv heads, "
                               "hdim 128, L~U[512,4096] from seed 1234 (the same lengths on every rank, values seeded per rank)" + (" [--small]" if args.small else ""),
                   "tokens_per_gpu": w["total"], "flops_per_gpu_step": w["flops"],
                   "flop_count": "causal-effective 4*d*hq*sum L(L+1)/2",
                   "l2": "inputs (q,k,v,o > 600 MB) larger than the 126 MB L2", "parallelism": f"dp{world}"},
        "roofline": {"bound": "tensor", "achieved": kernel_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": kernel_tflops / peaks["bf16_tflops"],
                     # DRAM bytes per launch from the committed ncu capture of this kernel on this workload
                     "traffic": None if args.small else load_traffic("prefill_config2"),
                     "algorithmic_bytes": 2.0 * w["total"] * (2 * HQ * D + 2 * HKV * D) + 4.0 * w["total"] * HQ,
                     "peak_source": peaks["source"] + " (burst bf16 GEMM)"},
        "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": steps,
        "clocks": clocks,
    }
    extra = {}

    # ------------------------------------------------------------------ prefill through the page table (next row)
    if not args.no_decode:
        wp = make_paged_prefill(w, 16, 99 + rank, device)

        def paged_prefill_step():
            return ops.fmha_fwd_paged_kv_prefill(w["q"], wp["k"], wp["v"], wp["table"], wp["seqlen"], cu_seqlens_q=w["cu"],
                                                 max_seqlen_q=w["max_len"], causal=True, return_lse=True)

        ms_p = max_over_ranks(time_steps(paged_prefill_step, steps, warmup, barrier))
        p_tflops = w["flops"] * steps / (ms_p * 1e-3) / 1e12
        extra["paged_prefill"] = {
            "metric": "paged_kv_prefill_tflops", "value": total_flops * steps / (ms_p * 1e-3) / 1e12, "unit": "TFLOP/s",
            "ms_per_step": ms_p / steps, "steps": steps,
            "config": {"workload": "the headline prefill with K/V read through a block table: pools [pages, 16, 8, 128], "
                                   "shuffled page ids, bottom-right causal (FmhaFwdPagedKVPrefill)", "page": 16},
            "roofline": {"bound": "tensor", "achieved": p_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": p_tflops / peaks["bf16_tflops"], "traffic": None, "peak_source": peaks["source"] + " (burst bf16 GEMM)"},
            "gpu_launches": steps,
        }
        del wp

    # ------------------------------------------------------------------ the same workload through library kernels (context)
    if not args.no_decode and rank == 0:
        extra["prefill_library_kernels"] = library_prefill_baselines(w, max(3, steps // 2))

    # ------------------------------------------------------------------ the headline prefill on 8-bit operands (next row)
    if not args.no_decode:
        (q8, dq), (k8, dk), (v8, dv8) = (ops.quantize_fp8(w[n], torch.float8_e4m3fn) for n in ("q", "k", "v"))
        sc_s, sc_p = dq * dk / D ** 0.5, 256.0

        def fp8_step():
            return ops.fmha_fwd_fp8(q8, k8, v8, scale_s=sc_s, scale_p=sc_p, scale_o=dv8 / sc_p, cu_seqlens_q=w["cu"],
                                    cu_seqlens_k=w["cu"], max_seqlen_q=w["max_len"], causal=True, out_dtype=torch.bfloat16,
                                    return_lse=True)

        n8 = max(3, steps // 2)
        ms_8 = max_over_ranks(time_steps(fp8_step, n8, 3, barrier))
        inst8 = _lib.get_instance_param(0, "last_instance")
        t8 = w["flops"] * n8 / (ms_8 * 1e-3) / 1e12
        extra["prefill_fp8"] = {
            "metric": "prefill_fmha_fp8_tflops", "value": total_flops * n8 / (ms_8 * 1e-3) / 1e12, "unit": "TFLOP/s",
            "ms_per_step": ms_8 / n8, "steps": n8, "dtype": "f8e4m3",
            "config": {"workload": "the headline prefill with Q, K, V quantised to E4M3 (static per-tensor scales), P rounded "
                                   "to E4M3 into TMEM, O in bf16 (FmhaFwdFp8): the kind::f8f6f4 instance of the tcgen05 kernel",
                       "instance": "tcgen05 kind::f8f6f4" if inst8 == 1 else "general (mma.sync on widened halves)"},
            "roofline": {"bound": "tensor", "achieved": t8, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": t8 / peaks["bf16_tflops"], "traffic": None,
                         "peak_source": peaks["source"] + " (burst bf16 GEMM; no 8-bit peak was measured on this pool)"},
            "gpu_launches": n8,
        }
        del q8, k8, v8

    # ------------------------------------------------------------------ decode (config 3)
    if not args.no_decode:
        if args.small:
            wd = make_decode(4321, device, batch=16, lo=1024, hi=16384, data_seed=4321 + rank)
        else:
            wd = make_decode(4321, device, data_seed=4321 + rank)
        S = ops.default_num_splits(len(wd["lens"]))
        ws = ops.splitkv_workspace(wd["q"], D, S)

        def decode_step():
            return ops.fmha_fwd_splitkv(wd["q"], wd["k"], wd["v"], seqlen_k=wd["seqlen"], block_table=wd["table"],
                                        num_splits=S, workspace=ws, return_lse=True)

        sampler = ClockSampler(local_rank)
        sampler.start()
        dsteps = max(steps, 20)
        ms_d = max_over_ranks(time_steps(decode_step, dsteps, warmup, barrier))
        dclocks = sampler.stop()
        tot_bytes = sum_over_ranks(wd["bytes"])
        gbs = tot_bytes * dsteps / (ms_d * 1e-3) / 1e9
        gbs_gpu = wd["bytes"] * dsteps / (ms_d * 1e-3) / 1e9
        # e2e decode step: the cache is resident state; the step's inputs are q, lengths and block table
        hq2 = wd["q"].cpu().pin_memory()
        hs, ht = wd["seqlen"].cpu().pin_memory(), wd["table"].cpu().pin_memory()
        dq2, ds, dt_ = torch.empty_like(wd["q"]), torch.empty_like(wd["seqlen"]), torch.empty_like(wd["table"])
        ho2 = torch.empty_like(hq2).pin_memory()

        def decode_e2e():
            dq2.copy_(hq2, non_blocking=True)
            ds.copy_(hs, non_blocking=True)
            dt_.copy_(ht, non_blocking=True)
            o, _ = ops.fmha_fwd_splitkv(dq2, wd["k"], wd["v"], seqlen_k=ds, block_table=dt_, num_splits=S,
                                        workspace=ws, return_lse=True)
            ho2.copy_(o, non_blocking=True)

        ms_de = max_over_ranks(time_steps(decode_e2e, dsteps, 3, barrier))
        extra["decode"] = {
            "metric": "paged_splitkv_decode_hbm_gbs", "value": gbs, "unit": "GB/s", "ms_per_step": ms_d / dsteps,
            "steps": dsteps,
            "config": {"workload": "paged split-KV decode (BASELINE config 3): batch 64 per GPU, seqlen_q 1, 32/8 heads, "
                                   "hdim 128, ctx~U[1024,32768], page 16, shuffled block table"
                                   + (" [--small]" if args.small else ""),
                       "tokens_per_gpu": sum(wd["lens"]), "algorithmic_bytes_per_gpu_step": wd["bytes"],
                       "num_splits": S, "l2": "K/V pool (GBs) larger than L2"},
            "roofline": {"bound": "hbm", "achieved": gbs_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs_gpu / peaks["hbm_gbs"],
                         # DRAM bytes of the split-KV launch: the record is a capture of the reduced workload, stored per cached
                         # token (the kernel reads every K/V byte once, so its traffic grows with the token count)
                         "traffic": load_traffic("decode_config3", scale=float(sum(wd["lens"]))), "peak_source": peaks["source"],
                         "note": "split-KV kernel + combine kernel timed together"},
            "e2e": {"value": tot_bytes * dsteps / (ms_de * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": hq2.numel() * 2 + hs.numel() * 4 + ht.numel() * 4,
                    "d2h_bytes_per_step": ho2.numel() * 2,
                    "note": "KV cache is resident state; q, lengths and block table are the step's inputs"},
            "gpu_launches": 2 * dsteps, "clocks": dclocks,
        }
        if rank == 0 and not args.no_cpu_baseline:
            extra["decode"]["cpu_baseline"] = cpu_decode_sample(wd)
        del wd, ws

    # ------------------------------------------------------------------ append + decode (config 4)
    if not args.no_decode and not args.small:
        wa = make_append_decode(777, device, data_seed=777 + rank)
        S4 = ops.default_num_splits(len(wa["lens"]), rows_per_kv_head=max(wa["new"]) * (HQ // HKV))
        cu_n, max_new = wa["cu_new"], max(wa["new"])
        ws4 = ops.splitkv_workspace(wa["qn"], D, S4, cu_n)

        def append_decode_step():
            ops.fmha_fwd_append_kv(wa["qn"], wa["k"], wa["v"], wa["kn"], wa["vn"], wa["ctx_len"], wa["cos"], wa["sin"],
                                   block_table=wa["table"], cu_seqlens_q=cu_n, cu_seqlens_knew=cu_n)
            return ops.fmha_fwd_splitkv(wa["qn"], wa["k"], wa["v"], seqlen_k=wa["seqlen"], block_table=wa["table"],
                                        cu_seqlens_q=cu_n, max_seqlen_q=max_new, num_splits=S4, causal=True,
                                        workspace=ws4, return_lse=True)

        asteps = max(steps, 20)
        ms_a = max_over_ranks(time_steps(append_decode_step, asteps, warmup, barrier))
        a_bytes = wa["bytes"] + wa["append_bytes"]
        extra["append_decode"] = {
            "metric": "appendkv_plus_splitkv_decode_hbm_gbs", "value": sum_over_ranks(a_bytes) * asteps / (ms_a * 1e-3) / 1e9,
            "unit": "GB/s", "ms_per_step": ms_a / asteps, "steps": asteps,
            "config": {"workload": "append 1-16 tokens with interleaved RoPE, then split-KV decode (BASELINE config 4): batch 32 "
                                   "per GPU, 32/8 heads, hdim 128, ctx~U[2048,16384], page 16",
                       "tokens_per_gpu": sum(wa["lens"]), "new_tokens_per_gpu": sum(wa["new"]),
                       "algorithmic_bytes_per_gpu_step": a_bytes, "num_splits": S4},
            "roofline": {"bound": "hbm", "achieved": a_bytes * asteps / (ms_a * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": a_bytes * asteps / (ms_a * 1e-3) / 1e9 / peaks["hbm_gbs"],
                         # DRAM bytes of the split-KV launch: the record is an ncu capture of 8 sequences, stored per cached
                         # token (the kernel reads every K/V byte once, so its traffic grows with the token count)
                         "traffic": load_traffic("append_decode_config4_per_token", scale=float(sum(wa["lens"]))),
                         "peak_source": peaks["source"], "note": "append-KV + split-KV + combine kernels timed together"},
            "gpu_launches": 3 * asteps,
        }
        del wa, ws4

    # ------------------------------------------------------------------ sequence-sharded long-context decode (config 5)
    if not args.no_decode and not args.small:
        from flashck_b200 import dist as fdist
        parity = sharded_decode_parity(fdist, ops, device, rank, world)  # small problem, same code path, against the oracle
        wl = make_long_decode(999 + rank, device, world)
        if dist is not None:  # q is replicated
            dist.broadcast(wl["q"], src=0)
        dec = fdist.ShardedDecoder(wl["q"].shape, D, torch.bfloat16, device, hkv=wl["hkv"])
        S5 = dec.num_splits
        lsteps = max(steps, 20)

        def long_decode_step():
            return dec(wl["q"], wl["k"], wl["v"], wl["table"], wl["seqlen"])

        ms_eager = max_over_ranks(time_steps(long_decode_step, lsteps, warmup, barrier))
        dec.capture(wl["q"], wl["k"], wl["v"], wl["table"], wl["seqlen"])
        ms_l = max_over_ranks(time_steps(dec.replay, lsteps, warmup, barrier))
        # stages, each timed alone over the same number of calls on every rank (the exchange kernel waits for its peers,
        # so its figure includes the skew between the ranks)
        def split_only():
            ops.fmha_fwd_splitkv(wl["q"], wl["k"], wl["v"], seqlen_k=wl["seqlen"], block_table=wl["table"],
                                 num_splits=S5, workspace=(dec.lse_acc, dec.o_acc), combine=False)

        def exchange_only():
            one = dec._one
            _lib.check(_lib.lib().FmhaFwdSplitKVShardedCombine(
                one(dec.lse_acc), one(dec.o_acc), one(dec.o), one(dec.lse), dec._bufs, dec.rank, 1, dec.world,
                *dec.shape, S5, 4, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "FmhaFwdSplitKVShardedCombine")

        ms_split = max_over_ranks(time_steps(split_only, lsteps, warmup, barrier))
        ms_exch = max_over_ranks(time_steps(exchange_only, lsteps, warmup, barrier))
        # the same step through torch.distributed: merge kernel, NCCL all-gather, merge kernel (the library-call baseline)
        ws5 = (dec.lse_acc, dec.o_acc)

        def nccl_step():
            return fdist.sequence_sharded_decode(wl["q"], wl["k"], wl["v"], wl["table"], wl["seqlen"], num_splits=S5,
                                                 workspace=ws5, return_lse=True)

        ms_nccl = max_over_ranks(time_steps(nccl_step, lsteps, warmup, barrier))
        gbs_l = wl["total_bytes"] * lsteps / (ms_l * 1e-3) / 1e9
        extra["long_decode"] = {
            "metric": "sequence_sharded_decode_hbm_gbs", "value": gbs_l, "unit": "GB/s", "ms_per_step": ms_l / lsteps,
            "steps": lsteps, "scaling": "strong",
            "config": {"workload": "long-context decode (BASELINE config 5): batch 4, seqlen_q 1, 64/8 heads, hdim 128, "
                                   "ctx 524288 per sequence, page 64, KV pages sharded contiguously over the GPUs; per "
                                   "step the split-KV kernel, then one kernel that merges the local splits, stores the "
                                   "partial into every rank's buffer over NVLink and merges the ranks; the two launches "
                                   "replayed from a CUDA graph (ShardedDecoder.capture / replay)",
                       "total_kv_bytes": wl["total_bytes"], "num_splits": S5,
                       "exchange_bytes_per_rank_pair": 4 * 64 * (D + 2) * 8, "parallelism": f"sp{world}"},
            "stages_ms": {"split_kv_kernel": ms_split / lsteps, "merge_exchange_merge_kernel": ms_exch / lsteps,
                          "step_eager_launches": ms_eager / lsteps, "step_cuda_graph": ms_l / lsteps,
                          "step_nccl_all_gather_path": ms_nccl / lsteps},
            "parity": parity,
            "roofline": {"bound": "hbm", "achieved": gbs_l / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs_l / world / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
                         "note": "per GPU; split-KV kernel and the merge + exchange + merge kernel timed together"},
            "gpu_launches": 2 * lsteps,
        }
        dec.close()
        del wl, ws5, dec

    if rank == 0 and not args.no_cpu_baseline:
        cb = cpu_prefill_sample(w)
        line["cpu_baseline"] = cb
    line["extra"] = extra
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
