"""The tuner on the GPU: real CUDA-event timing of every valid instance on a small prefill and a small decode problem,
the winner cached in flash_ck.db, applied, and served from the cache on the next call -- through the functional API
(FC_TUNING_MODE 1 + FC_TUNING_DB_DIR arm the in-call tuner) and through Tuner.tune directly."""
import os
import sqlite3

import pytest
import torch

import flashck_b200 as fck
from flashck_b200 import _lib, ops
from flashck_b200 import instances as I
from flashck_b200 import tuner as T
from flashck_b200.utils.inputs import make_paged_cache, normal_tensor, to_seqstarts
from helpers import assert_lse_close, assert_o_close
from oracle import cpu as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture
def tuning_flags(tmp_path):
    names = ("FC_TUNING_MODE", "FC_TUNING_DB_DIR", "FC_TUNING_NUM_COLD_ITERATION", "FC_TUNING_NUM_REPEATS",
             "FC_FORCE_PROFILING_DB", "FC_TUNING_METRIC")
    old = {n: fck.get_flag_value(n) for n in names}
    fck.set_flag_value("FC_TUNING_MODE", 1)
    fck.set_flag_value("FC_TUNING_DB_DIR", str(tmp_path))
    fck.set_flag_value("FC_TUNING_NUM_COLD_ITERATION", 2)
    fck.set_flag_value("FC_TUNING_NUM_REPEATS", 5)
    fck.set_flag_value("FC_FORCE_PROFILING_DB", True)   # use cached results when there are some
    fck.set_flag_value("FC_TUNING_METRIC", 0)
    defaults = {(f, k): _lib.get_instance_param(f, k) for f, k in
                ((0, "use_sm100"), (0, "exp_mode"), (2, "use_sm100_splitkv"), (2, "stages"), (2, "ctas_per_sm_x100"),
                 (2, "heads_per_cta"), (2, "row_tiles"), (2, "exp_mode_splitkv"), (2, "split_item_cost"))}
    yield str(tmp_path)
    for n, v in old.items():
        fck.set_flag_value(n, v)
    for (f, k), v in defaults.items():
        _lib.set_instance_param(f, k, v)
    T._DEFAULT_TUNER = None


def _rows(db_dir):
    conn = sqlite3.connect(os.path.join(db_dir, "flash_ck.db"))
    rows = conn.execute("SELECT instance_name, latency, tflops, bandwidth FROM fmha").fetchall()
    conn.close()
    return rows


def test_in_call_tuning_of_a_small_prefill_and_a_small_decode(tuning_flags):
    dtype = torch.bfloat16
    # ---- prefill: 7 valid instances at hdim 128 (six tcgen05 softmax variants and the general instance)
    lens = [700, 130, 1025, 512]
    cu = to_seqstarts(lens)
    q = normal_tensor((sum(lens), 8, 128), dtype, 5)
    k = normal_tensor((sum(lens), 2, 128), dtype, 6)
    v = normal_tensor((sum(lens), 2, 128), dtype, 7)
    o_ref, lse_ref = oracle.fmha_fwd(q, k, v, seqstart_q=cu, seqstart_k=cu, mask_type=1, window=(-1, 0))
    args = (q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV), cu.to(DEV), max(lens))
    o, lse = ops.fmha_fwd_var_len(*args, causal=True, return_lse=True)
    tn = T._DEFAULT_TUNER
    assert tn is not None and len(tn.log) == 7 and all(r.get("latency", 0) > 0 for r in tn.log)  # every candidate timed
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)
    rows = _rows(tuning_flags)
    assert len(rows) == 1 and rows[0][0].startswith("fmha_fwd_bf16_group_") and rows[0][1] > 0
    winner = min(tn.log, key=lambda r: r["latency"])
    assert rows[0][0] == winner["instance_name"]
    inst = I.from_config("fmha_fwd", winner["instance"])
    assert _lib.get_instance_param(0, "use_sm100") == inst.pipeline            # the winner is what is applied
    assert _lib.get_instance_param(0, "exp_mode") == inst.exp_mode
    # the next call of the same problem is served from the cache: nothing is timed, the same instance runs
    tn.log = []
    _lib.set_instance_param(0, "exp_mode", 0 if inst.exp_mode else 11)         # disturb; the cache must put it back
    o2, lse2 = ops.fmha_fwd_var_len(*args, causal=True, return_lse=True)
    assert tn.log == [] and len(_rows(tuning_flags)) == 1
    assert _lib.get_instance_param(0, "exp_mode") == inst.exp_mode
    assert_o_close(o2, o_ref)
    assert_lse_close(lse2, lse_ref)

    # ---- decode: one query token per sequence, page 16 (the gather kernel's ring depth, CTAs per SM, heads per CTA)
    lens_k = [3000, 64, 9000, 1500, 17, 4097]
    cache = make_paged_cache(lens_k, 8, 128, 128, 16, dtype, seed=9)
    qd = normal_tensor((len(lens_k), 1, 32, 128), dtype, 10)
    o_ref, lse_ref = oracle.fmha_fwd(qd, cache.k, cache.v, seqlen_k=cache.seqlen_k, block_table=cache.block_table)
    dargs = (qd.to(DEV), cache.k.to(DEV), cache.v.to(DEV))
    dkw = dict(seqlen_k=cache.seqlen_k.to(DEV), block_table=cache.block_table.to(DEV), return_lse=True)
    o, lse = ops.fmha_fwd_splitkv(*dargs, **dkw)
    assert len(tn.log) == 12 and all(r.get("latency", 0) > 0 for r in tn.log)
    assert_o_close(o, o_ref)
    assert_lse_close(lse, lse_ref)
    rows = _rows(tuning_flags)
    assert len(rows) == 2 and rows[1][0].startswith("fmha_fwd_splitkv_bf16_batch_")
    tn.log = []
    o, lse = ops.fmha_fwd_splitkv(*dargs, **dkw)
    assert tn.log == [] and len(_rows(tuning_flags)) == 2
    assert_o_close(o, o_ref)
    assert _lib.device_status() == 0


def test_tuner_metrics_on_the_gpu(tuning_flags):
    """Tuner.tune with the bandwidth metric on a decode workload: GB/s is recorded and is what picks the winner."""
    family, prob, run, flops, nbytes = T._workload("decode_small")
    flags = T.TuningFlags(FC_TUNING_MODE=2, FC_TUNING_METRIC=2, FC_TUNING_NUM_COLD_ITERATION=2, FC_TUNING_NUM_REPEATS=5)
    tn = T.Tuner(flags=flags)
    best = tn.tune(family, prob, run, flops, nbytes)
    assert best["bandwidth"] == max(r["bandwidth"] for r in tn.log) and best["bandwidth"] > 1000.0  # GB/s on a B200
    again = tn.tune(family, prob, run, flops, nbytes)
    assert again["from_cache"] and again["instance_name"] == best["instance_name"]
