"""Tuner host logic (no GPU): search-space expansion in the reference's JSON form, selection by metric, and the
SQLite cache round trip."""
import os

import pytest

from flashck_b200 import tuner as T


def test_param_forms_and_cartesian_product():
    assert T.expand_param({"values": [1, 4]}) == [1, 4]
    assert T.expand_param({"min": 2, "max": 8, "step": 2, "exclude": [6]}) == [2, 4, 8]
    assert T.expand_param({}) == []
    combos = T.cartesian_product({"b": [1, 2], "a": [7]})
    assert combos == [{"a": 7, "b": 1}, {"a": 7, "b": 2}]


def test_shipped_search_spaces_load():
    fwd = T.load_search_space("fmha_fwd")
    assert fwd["use_sm100"] == [1] and 0 in fwd["poly8"]
    dec = T.load_search_space("fmha_fwd_split_kv")
    assert dec["stages"] == [2, 3] and 100 in dec["ctas_per_sm_x100"]
    assert T.load_search_space("fmha_fwd_split_kv", section="strategy")["num_splits"] == [0]


def test_tune_picks_best_and_caches(tmp_path):
    applied = []
    cost = {0: 3.0, 3: 1.5}
    state = {"poly8": None, "timed": 0}

    def apply(fam, key, value):
        applied.append((fam, key, value))
        state[key] = value

    def timer(run, cold, repeats, flush):
        state["timed"] += 1
        return cost[state["poly8"]]

    flags = T.TuningFlags(FC_TUNING_DB_DIR=str(tmp_path), FC_TUNING_METRIC=1)
    env = {"cuda_version": "12.9", "device_name": "fake B200"}
    tn = T.Tuner(flags=flags, db=T.ProfilingDB(os.path.join(str(tmp_path), "flash_ck.db")), timer=timer, apply=apply, env=env)
    problem = {"dtype": "bf16", "hq": 32, "hkv": 8, "d": 128, "mask": "causal", "mode": "group"}
    best = tn.tune("fmha_fwd", problem, run=lambda: None, flops=1e12)
    assert best["instance"]["poly8"] == 3 and state["poly8"] == 3 and state["timed"] == 2
    assert abs(best["tflops"] - 1e12 / 1.5 / 1e9) < 1e-6
    # second call: served from the cache, nothing is timed again, the winner is re-applied
    state["timed"] = 0
    again = tn.tune("fmha_fwd", problem, run=lambda: None, flops=1e12)
    assert again["instance"] == best["instance"] and state["timed"] == 0 and state["poly8"] == 3
    # another problem is a cache miss; heuristic mode takes the first candidate without a sweep
    tn.flags.FC_TUNING_MODE = 0
    other = tn.tune("fmha_fwd", dict(problem, hq=64), run=lambda: None, flops=1e12)
    assert state["timed"] == 1 and other["instance"]["poly8"] == 0
    tn.db.flush()
    assert tn.db.query(env, tn.setting(), problem) is None


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
