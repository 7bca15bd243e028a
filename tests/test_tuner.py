"""Tuner host logic (no GPU): search-space expansion in the reference's JSON form, selection by metric, and the
SQLite cache round trip."""
import os

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
    cost = {0: 3.0, 2: 1.5, 3: 2.0}
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
    assert best["instance"]["poly8"] == 2 and state["poly8"] == 2 and state["timed"] == 3
    assert abs(best["tflops"] - 1e12 / 1.5 / 1e9) < 1e-6
    # second call: served from the cache, nothing is timed again, the winner is re-applied
    state["timed"] = 0
    again = tn.tune("fmha_fwd", problem, run=lambda: None, flops=1e12)
    assert again["instance"] == best["instance"] and state["timed"] == 0 and state["poly8"] == 2
    # another problem is a cache miss; heuristic mode takes the first candidate without a sweep
    tn.flags.FC_TUNING_MODE = 0
    other = tn.tune("fmha_fwd", dict(problem, hq=64), run=lambda: None, flops=1e12)
    assert state["timed"] == 1 and other["instance"]["poly8"] == 0
    tn.db.flush()
    assert tn.db.query(env, tn.setting(), problem) is None
