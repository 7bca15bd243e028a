"""Tuner host logic (no GPU): search-space expansion in the reference's JSON form, selection by metric, and the
SQLite cache round trip."""
import dataclasses
import os

import pytest

from flashck_b200 import instances as I
from flashck_b200 import tuner as T


def test_param_forms_and_cartesian_product():
    assert T.expand_param({"values": [1, 4]}) == [1, 4]
    assert T.expand_param({"min": 2, "max": 8, "step": 2, "exclude": [6]}) == [2, 4, 8]
    assert T.expand_param({}) == []
    combos = T.cartesian_product({"b": [1, 2], "a": [7]})
    assert combos == [{"a": 7, "b": 1}, {"a": 7, "b": 2}]


def test_shipped_search_spaces_load():
    fwd = T.load_search_space("fmha_fwd")
    assert fwd["block_m"] == [128, 64] and fwd["pipeline"] == [1, 0] and 0 in fwd["exp_mode"]
    dec = T.load_search_space("fmha_fwd_split_kv")
    assert dec["stages"] == [0, 2, 3] and 100 in dec["ctas_per_sm_x100"] and dec["tokens_per_tile"] == [16, 128]
    assert T.load_search_space("fmha_fwd_split_kv", section="strategy")["num_splits"] == [0]


def _prefill_problem(**kw):
    base = dict(family="fmha_fwd", dtype="bf16", mode="group", batch=16, hq=32, hkv=8, d=128, dv=128, max_seqlen_q=4096,
                max_seqlen_k=4096, mask="causal")
    base.update(kw)
    return I.FmhaProblem(**base)


def test_instances_validity_names_and_heuristics():
    cands = T.load_candidates("fmha_fwd")
    assert len(cands) == len(set(cands)) and len(cands) > 20  # the Cartesian product, canonical, without duplicates
    p = _prefill_problem()
    valid = [t for t in cands if I.is_valid(t, p)]
    names = [t.name() for t in valid]
    assert "fmha_fwd_128x128x128_s2_wg2_x0_tc05_384_1" in names and "fmha_fwd_64x64x128_s2_wg2_x0_mma_128_1" in names
    assert len(valid) == 7 and len(set(names)) == 7
    # what cannot work says why
    assert "128 x 128" in I.why_invalid(I.FmhaFwdInstance(block_m=64), p)
    assert "exp2 unit" in I.why_invalid(I.FmhaFwdInstance(head_dim=64, exp_mode=1), _prefill_problem(d=64, dv=64))
    assert I.why_invalid(I.FmhaFwdInstance(), p) is None
    assert "head_dim" in I.why_invalid(I.FmhaFwdInstance(head_dim=64), p)
    assert "positive" in I.why_invalid(I.FmhaFwdInstance(kv_stages=0), p)
    # hdim 64 has one tcgen05 instance and the general one; a bias tensor has a tcgen05 instance at hdim 128 only
    assert sorted(t.pipeline for t in cands if I.is_valid(t, _prefill_problem(d=64, dv=64))) == [0, 1]
    assert sorted((t.pipeline, t.exp_mode) for t in cands if I.is_valid(t, _prefill_problem(bias="elementwise"))) == [(0, 0), (1, 0)]
    assert [t.pipeline for t in cands if I.is_valid(t, _prefill_problem(d=64, dv=64, bias="elementwise"))] == [0]
    # 8-bit operands: the kind::f8f6f4 instance (plain exp2 unit, hdim 128, contiguous) and the general one
    p8 = dataclasses.replace(p, dtype="fp8")
    v8 = [t for t in cands if I.is_valid(t, p8)]
    assert sorted((t.pipeline, t.exp_mode) for t in v8) == [(0, 0), (1, 0)]
    assert "f8f6f4" in I.why_invalid(I.FmhaFwdInstance(exp_mode=11), p8)
    assert [t.pipeline for t in cands if I.is_valid(t, dataclasses.replace(p8, paged=True, page=16))] == [0]
    assert "no bias" in I.why_invalid(I.FmhaFwdInstance(), dataclasses.replace(p8, bias="alibi"))
    # rules of thumb: tensor-memory pipeline with the plain exp2 unit first
    kept = I.heuristic_filter(valid, p)
    assert kept[0].pipeline == 1 and kept[0].exp_mode == 0 and all(t.pipeline == 1 for t in kept)
    # the problem is part of the full name, and the cache key buckets lengths
    assert valid[0].name(p).startswith("fmha_fwd_bf16_group_b16_h32x8_d128x128_sq4096_sk4096_causal_none_128x128x128")
    assert _prefill_problem(max_seqlen_q=3000).key() == _prefill_problem(max_seqlen_q=4096).key()
    # split-KV: one query row per sequence runs on the gather kernel only, many rows also on the tcgen05 split modes
    dec = T.load_candidates("fmha_fwd_split_kv")
    p3 = I.FmhaProblem("fmha_fwd_split_kv", "bf16", "batch", 64, 32, 8, 128, 128, 1, 32768, "none", paged=True, page=16)
    assert {t.pipeline for t in dec if I.is_valid(t, p3)} == {0}
    p4 = I.FmhaProblem("fmha_fwd_split_kv", "bf16", "group", 32, 32, 8, 128, 128, 16, 16400, "causal", paged=True, page=16)
    v4 = [t for t in dec if I.is_valid(t, p4)]
    assert {t.pipeline for t in v4} == {0, 1} and all(t.pipeline == 1 for t in I.heuristic_filter(v4, p4))
    assert "multiple of tokens_per_tile" in I.why_invalid(
        I.FmhaFwdSplitKVInstance(pipeline=0), I.FmhaProblem("fmha_fwd_split_kv", "bf16", "batch", 1, 8, 8, 128, 128, 1, 64,
                                                            paged=True, page=8))
    with pytest.raises(KeyError):
        I.from_config("fmha_fwd", {"block_q": 128})


def test_tune_picks_best_and_caches(tmp_path):
    applied = []
    cost = {0: 3.0, 1: 1.5, 11: 2.0, 12: 2.5, 13: 2.6}
    state = {"exp_mode": None, "use_sm100": None, "timed": 0}

    def apply(fam, key, value):
        applied.append((fam, key, value))
        state[key] = value

    def timer(run, cold, repeats, flush):
        state["timed"] += 1
        if state["use_sm100"] == 0:
            raise RuntimeError("refused")  # a candidate the library refuses is skipped, not picked
        return cost[state["exp_mode"]]

    flags = T.TuningFlags(FC_TUNING_DB_DIR=str(tmp_path), FC_TUNING_METRIC=1, FC_TUNING_MODE=1, FC_FORCE_PROFILING=False)
    env = {"cuda_version": "12.9", "device_name": "fake B200"}
    tn = T.Tuner(flags=flags, db=T.ProfilingDB(os.path.join(str(tmp_path), "flash_ck.db")), timer=timer, apply=apply, env=env)
    problem = _prefill_problem()
    best = tn.tune("fmha_fwd", problem, run=lambda: None, flops=1e12)
    assert best["instance"]["exp_mode"] == 1 and state["exp_mode"] == 1 and state["timed"] == 7
    assert len(tn.log) == 7 and sum("error" in r for r in tn.log) == 1
    assert abs(best["tflops"] - 1e12 / 1.5 / 1e9) < 1e-6 and best["instance_name"].endswith("x1r200_tc05_384_1")
    # second call: served from the cache, nothing is timed again, the winner is re-applied
    state.update(timed=0, exp_mode=None)
    again = tn.tune("fmha_fwd", problem, run=lambda: None, flops=1e12)
    assert again["instance"] == best["instance"] and again["from_cache"] and state["timed"] == 0 and state["exp_mode"] == 1
    # another problem is a cache miss; heuristic mode takes the first candidate without a sweep
    tn.flags.FC_TUNING_MODE = 0
    other = tn.tune("fmha_fwd", _prefill_problem(hq=64), run=lambda: None, flops=1e12)
    assert state["timed"] == 1 and other["instance"]["exp_mode"] == 0 and other["instance"]["pipeline"] == 1
    # equal TFLOP/s: the candidate that keeps the tensor pipe busier wins
    tn.flags.FC_TUNING_MODE = 1
    tn.utilisation = lambda inst: {0: 40.0, 11: 55.0}.get(inst.exp_mode, 10.0)
    cost.update({0: 2.0, 1: 2.5, 11: 2.01})
    tied = tn.tune("fmha_fwd", _prefill_problem(hq=16), run=lambda: None, flops=1e12)
    assert tied["instance"]["exp_mode"] == 11 and tied["tensor_pipe_pct"] == 55.0
    tn.db.flush()
    assert tn.db.query(env, tn.setting(), problem.key()) is None


def test_flag_api_has_the_reference_names_types_and_errors(capsys):
    import flashck_b200 as fck
    from flashck_b200.utils import flags
    # defaults of core/utils/flags.cc, values as strings like the reference's binding returns them
    assert fck.get_flag_value("FC_TUNING_NUM_REPEATS") == "64"
    assert fck.get_flag_value("FC_TUNING_FLUSH_CACHE") == "true"
    assert fck.get_flag_value("FC_TUNING_DB_DIR") == ""
    try:
        fck.set_flag_value("FC_TUNING_NUM_REPEATS", "8")
        fck.set_flag_value("FC_TUNING_FLUSH_CACHE", "false")
        assert flags.get_flag("FC_TUNING_NUM_REPEATS") == 8 and flags.get_flag("FC_TUNING_FLUSH_CACHE") is False
        t = T.Tuner(timer=lambda run, cold, rep, flush: 1.0)
        assert t.flags.FC_TUNING_NUM_REPEATS == 8 and t.flags.FC_TUNING_FLUSH_CACHE is False  # a new tuner sees them
        with pytest.raises(RuntimeError):
            fck.set_flag_value("FC_TUNING_NUM_REPEATS", "many")
        with pytest.raises(RuntimeError):
            fck.set_flag_value("FC_ROCM_PATH", "/opt/rocm")     # HIP build pipeline flag: not registered here
        with pytest.raises(RuntimeError):
            fck.get_flag_value("FC_NO_SUCH_FLAG")
    finally:
        fck.set_flag_value("FC_TUNING_NUM_REPEATS", "64")
        fck.set_flag_value("FC_TUNING_FLUSH_CACHE", "true")
    fck.print_flag_info("FC_TUNING_METRIC")
    fck.print_all_flags()
    out = capsys.readouterr().out
    assert "FC_TUNING_METRIC (int) = 0" in out and "FC_CALL_STACK_LEVEL" in out
