"""Instance tuner for the attention kernels.

In the reference, tuning means: expand a JSON search space into ck_tile instances
(``core/profiling/attention/fmha_fwd/fmha_fwd_emitter.cc:132-323``), compile and time each one in a subprocess
(``core/profiling/gpu_profiling_runner.cc:99-156``), keep the best by ``FC_TUNING_METRIC`` and cache it in SQLite
keyed by environment, settings and problem (``core/profiling/profiling_db.cc:22-40,59-286``).  Here the instances
are prebuilt and selected through ``FlashckSetInstanceParam``, so the tuner keeps the same three pieces without
the JIT:

* the search space files use the reference's parameter form -- ``{"values": [...]}`` or
  ``{"min", "max", "step", "exclude"}`` (``core/utils/json_config.h:15-52``) -- under
  ``flashck_b200/configs/attention/<family>/default_config.json``;
* candidates are timed in-process with CUDA events after warm-up, with an L2 flush between repeats, using the
  reference's knobs and defaults (``FC_TUNING_NUM_COLD_ITERATION`` 16, ``FC_TUNING_NUM_REPEATS`` 64,
  ``FC_TUNING_FLUSH_CACHE`` true; ``core/utils/flags.cc:213-233``); the metric is latency (0), TFLOP/s (1) or
  GB/s (2) like ``FC_TUNING_METRIC``;
* winners are cached in ``flash_ck.db`` with the reference's table columns (``cuda_version`` in place of
  ``rocm_version``).
"""
from __future__ import annotations

import itertools
import json
import os
import sqlite3
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, Iterable, List, Optional

__all__ = ["TuningFlags", "load_search_space", "load_candidates", "expand_param", "cartesian_product", "ProfilingDB",
           "Tuner", "FAMILY_IDS", "select_instance", "tuning_enabled", "ncu_tensor_pipe_pct"]

_HERE = os.path.dirname(os.path.abspath(__file__))
FAMILY_IDS = {"fmha_fwd": 0, "fmha_fwd_split_kv": 2}  # FmhaKind values (fmha_library.h:17-25)


def _flag(name: str):
    from .utils import flags
    return flags.get_flag(name)


@dataclass
class TuningFlags:
    """The reference's tuning flags (core/utils/flags.cc:201-233).  The defaults are read from the flag registry
    (``flashck_b200.utils.flags``: ``set_flag_value`` / ``FC_*`` environment variables) when a tuner is built."""
    FC_TUNING_MODE: int = field(default_factory=lambda: _flag("FC_TUNING_MODE"))    # 0 heuristic, 1 autotuning, 2 hybrid
    FC_TUNING_METRIC: int = field(default_factory=lambda: _flag("FC_TUNING_METRIC"))  # 0 latency, 1 TFLOP/s, 2 bandwidth
    FC_TUNING_NUM_COLD_ITERATION: int = field(default_factory=lambda: _flag("FC_TUNING_NUM_COLD_ITERATION"))
    FC_TUNING_NUM_REPEATS: int = field(default_factory=lambda: _flag("FC_TUNING_NUM_REPEATS"))
    FC_TUNING_FLUSH_CACHE: bool = field(default_factory=lambda: _flag("FC_TUNING_FLUSH_CACHE"))
    FC_TUNING_SEED: int = field(default_factory=lambda: _flag("FC_TUNING_SEED"))
    # Re-time even if the cache has an entry.  The reference defaults both FC_FORCE_PROFILING and FC_FORCE_PROFILING_DB
    # to true, which contradict each other; here a cached result is used unless FC_FORCE_PROFILING_DB is switched off.
    FC_FORCE_PROFILING: bool = field(default_factory=lambda: not _flag("FC_FORCE_PROFILING_DB"))
    FC_TUNING_DB_DIR: str = field(default_factory=lambda: _flag("FC_TUNING_DB_DIR"))
    FC_CONFIG_JSON_PATH: str = field(default_factory=lambda: _flag("FC_CONFIG_JSON_PATH") or os.path.join(_HERE, "configs"))


def expand_param(node: dict) -> List[int]:
    """Values of one parameter node (core/utils/json_config.h:19-40)."""
    if isinstance(node.get("values"), list):
        return [int(v) for v in node["values"]]
    if "min" in node and "max" in node:
        step = int(node.get("step", 1))
        excl = set(node.get("exclude", []))
        return [v for v in range(int(node["min"]), int(node["max"]) + 1, step) if v not in excl]
    return []


def load_search_space(family: str, config_root: Optional[str] = None, section: str = "instance") -> Dict[str, List[int]]:
    """``{param: [values]}`` of one section of ``<root>/attention/<family>/default_config.json``."""
    root = config_root or TuningFlags().FC_CONFIG_JSON_PATH
    with open(os.path.join(root, "attention", family, "default_config.json")) as f:
        doc = json.load(f)
    return {k: expand_param(v) for k, v in doc.get(section, {}).items()}


def cartesian_product(space: Dict[str, List[int]]) -> List[Dict[str, int]]:
    """All combinations, in a stable order (the reference's ``CartesianProduct``, json_config.h)."""
    keys = sorted(space)
    return [dict(zip(keys, combo)) for combo in itertools.product(*(space[k] for k in keys))]


def load_candidates(family: str, config_root: Optional[str] = None) -> List:
    """Every instance of the family's search space (sections ``instance``, ``launch`` and ``strategy`` of its JSON file
    multiplied out, core/profiling/attention/fmha_fwd/fmha_fwd_emitter.cc:132-323), in canonical form, without
    duplicates, in a stable order."""
    from . import instances as I
    space: Dict[str, List[int]] = {}
    for section in ("instance", "launch", "strategy"):
        space.update(load_search_space(family, config_root, section))
    seen, out = set(), []
    for cfg in cartesian_product(space):
        inst = I.from_config(family, cfg).canonical()
        if inst not in seen:
            seen.add(inst)
            out.append(inst)
    return out


class ProfilingDB:
    """SQLite cache of tuning results; columns follow core/profiling/profiling_db.cc:28-40."""

    def __init__(self, path: str):
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self.conn = sqlite3.connect(path)
        self.conn.execute("PRAGMA journal_mode = WAL")
        self.conn.execute(
            "CREATE TABLE IF NOT EXISTS fmha ("
            "id INTEGER PRIMARY KEY AUTOINCREMENT, cuda_version TEXT NOT NULL, device_name TEXT NOT NULL,"
            "setting TEXT NOT NULL, problem TEXT NOT NULL, instance_name TEXT NOT NULL, instance TEXT NOT NULL,"
            "split_k INTEGER NOT NULL DEFAULT -1, latency REAL, tflops REAL, bandwidth REAL, tensor_pipe_pct REAL)")
        cols = [r[1] for r in self.conn.execute("PRAGMA table_info(fmha)")]
        if "tensor_pipe_pct" not in cols:  # a database written before the column existed
            self.conn.execute("ALTER TABLE fmha ADD COLUMN tensor_pipe_pct REAL")
        self.conn.commit()

    @staticmethod
    def _key(d: dict) -> str:
        return json.dumps(d, sort_keys=True)

    def query(self, env: dict, setting: dict, problem: dict) -> Optional[dict]:
        row = self.conn.execute(
            "SELECT instance_name, instance, latency, tflops, bandwidth, tensor_pipe_pct, split_k FROM fmha WHERE cuda_version=? AND device_name=? "
            "AND setting=? AND problem=? ORDER BY id DESC LIMIT 1",
            (env["cuda_version"], env["device_name"], self._key(setting), self._key(problem))).fetchone()
        if row is None:
            return None
        return {"instance_name": row[0], "instance": json.loads(row[1]), "latency": row[2], "tflops": row[3],
                "bandwidth": row[4], "tensor_pipe_pct": row[5], "split_k": row[6]}

    def insert(self, env: dict, setting: dict, problem: dict, name: str, instance: dict, latency: float,
               tflops: Optional[float], bandwidth: Optional[float], tensor_pipe_pct: Optional[float] = None,
               split_k: int = -1) -> None:
        self.conn.execute(
            "INSERT INTO fmha (cuda_version, device_name, setting, problem, instance_name, instance, split_k, latency, "
            "tflops, bandwidth, tensor_pipe_pct) VALUES (?,?,?,?,?,?,?,?,?,?,?)",
            (env["cuda_version"], env["device_name"], self._key(setting), self._key(problem), name,
             json.dumps(instance, sort_keys=True), split_k, latency, tflops, bandwidth, tensor_pipe_pct))
        self.conn.commit()

    def flush(self) -> None:
        """FC_FLUSH_PROFILING_DB: drop every cached result."""
        self.conn.execute("DELETE FROM fmha")
        self.conn.commit()


@dataclass
class Tuner:
    """Times the valid instances of one family on a caller-supplied workload and applies the winner.

    ``timer(run, cold, repeats, flush)`` returns milliseconds per call; the default uses CUDA events.  ``apply`` sets
    one instance parameter (default: ``FlashckSetInstanceParam``).  ``utilisation(instance)`` (optional) returns the
    tensor-pipe busy percentage of a candidate, e.g. from an ncu capture of a small case
    (:func:`ncu_tensor_pipe_pct`); it is stored beside the timing, and with ``FC_TUNING_METRIC`` 1 it breaks ties
    between candidates whose TFLOP/s differ by less than 1 %.  All three are injectable so that the selection logic is
    testable without a GPU."""
    flags: TuningFlags = field(default_factory=TuningFlags)
    db: Optional[ProfilingDB] = None
    timer: Optional[Callable] = None
    apply: Optional[Callable[[int, str, int], None]] = None
    env: Optional[dict] = None
    utilisation: Optional[Callable] = None
    log: List[dict] = field(default_factory=list)  # every candidate timed by the last sweep

    def __post_init__(self):
        if self.db is None:
            d = self.flags.FC_TUNING_DB_DIR or os.path.join(os.path.expanduser("~"), ".flashck")
            self.db = ProfilingDB(os.path.join(d, "flash_ck.db"))
        if self.timer is None:
            self.timer = _cuda_event_timer
        if self.apply is None:
            from . import _lib
            self.apply = _lib.set_instance_param
        if self.env is None:
            self.env = _environment()

    def setting(self) -> dict:
        f = self.flags
        return {"metric": f.FC_TUNING_METRIC, "cold": f.FC_TUNING_NUM_COLD_ITERATION, "repeats": f.FC_TUNING_NUM_REPEATS,
                "flush_cache": bool(f.FC_TUNING_FLUSH_CACHE)}

    def candidates(self, family: str, problem) -> List:
        """Valid instances for the problem, narrowed as FC_TUNING_MODE says: 0 (heuristic) the first survivor of the
        rules of thumb, 2 (hybrid) all survivors, 1 (autotuning) every valid instance
        (fmha_fwd_emitter.cc:325-466 applies the same three modes)."""
        from . import instances as I
        valid = [t for t in load_candidates(family, self.flags.FC_CONFIG_JSON_PATH) if I.is_valid(t, problem)]
        if not valid:
            raise RuntimeError(f"no instance of {family} can run {problem.name()}")
        mode = self.flags.FC_TUNING_MODE
        if mode == 1:
            return valid
        kept = I.heuristic_filter(valid, problem)
        return kept[:1] if mode == 0 else kept

    def _score(self, rec: dict) -> float:
        m = self.flags.FC_TUNING_METRIC
        if m == 1 and rec["tflops"]:
            return rec["tflops"]
        if m == 2 and rec["bandwidth"]:
            return rec["bandwidth"]
        return -rec["latency"]

    def _better(self, a: dict, b: Optional[dict]) -> bool:
        if b is None:
            return True
        sa, sb = self._score(a), self._score(b)
        if self.flags.FC_TUNING_METRIC == 1 and a.get("tensor_pipe_pct") and b.get("tensor_pipe_pct") \
                and abs(sa - sb) <= 0.01 * max(abs(sa), abs(sb)):
            return a["tensor_pipe_pct"] > b["tensor_pipe_pct"]
        return sa > sb

    def _apply(self, fam: int, params: Dict[str, int]) -> None:
        for k, v in params.items():
            self.apply(fam, k, v)

    def tune(self, family: str, problem, run: Callable[[], object], flops: Optional[float] = None,
             nbytes: Optional[float] = None) -> dict:
        """Returns the winning record (served from the cache when there is one) and leaves its parameters applied.
        ``problem`` is an :class:`flashck_b200.instances.FmhaProblem`."""
        from . import instances as I
        fam = FAMILY_IDS[family]
        key = problem.key()
        cached = None if self.flags.FC_FORCE_PROFILING else self.db.query(self.env, self.setting(), key)
        if cached is not None:
            self._apply(fam, I.from_config(family, cached["instance"]).params())
            cached["from_cache"] = True
            return cached
        best, self.log = None, []
        for inst in self.candidates(family, problem):
            self._apply(fam, inst.params())
            try:
                ms = float(self.timer(run, self.flags.FC_TUNING_NUM_COLD_ITERATION, self.flags.FC_TUNING_NUM_REPEATS,
                                      self.flags.FC_TUNING_FLUSH_CACHE))
            except RuntimeError as e:  # the library refused the problem on this instance: not a candidate
                self.log.append({"instance_name": inst.name(problem), "instance": asdict(inst), "error": str(e)})
                continue
            rec = {"instance_name": inst.name(problem), "instance": asdict(inst), "latency": ms,
                   "tflops": flops / ms / 1e9 if flops else None, "bandwidth": nbytes / ms / 1e6 if nbytes else None,
                   "tensor_pipe_pct": float(self.utilisation(inst)) if self.utilisation else None,
                   "split_k": int(getattr(inst, "num_splits", -1) or -1), "from_cache": False}
            self.log.append(rec)
            if self._better(rec, best):
                best = rec
        if best is None:
            raise RuntimeError(f"every candidate of {family} failed on {problem.name()}: {self.log}")
        self._apply(fam, I.from_config(family, best["instance"]).params())
        self.db.insert(self.env, self.setting(), key, best["instance_name"], best["instance"], best["latency"],
                       best["tflops"], best["bandwidth"], best["tensor_pipe_pct"], best["split_k"])
        return best


# The tuner the functional API consults when FC_TUNING_MODE is not 0 (one per process, created on first use).
_DEFAULT_TUNER: Optional[Tuner] = None


def tuning_enabled() -> bool:
    """The functional API tunes in-call when the mode is not 0 (heuristic) and a cache directory is set
    (``FC_TUNING_DB_DIR``, empty by default as in the reference): without a place to keep the winners every process
    would repeat the sweep, so the prebuilt default instances run instead."""
    return int(_flag("FC_TUNING_MODE")) != 0 and bool(_flag("FC_TUNING_DB_DIR"))


def select_instance(family: str, problem, run: Callable[[], object], flops: Optional[float] = None,
                    nbytes: Optional[float] = None) -> dict:
    """What ``flashck_b200.ops`` calls before a launch when tuning is on: applies the cached winner for the problem,
    or -- on a miss -- times the candidates on the caller's own tensors (``run`` launches the call) and caches the
    winner.  The instance parameters are process-wide, like the reference's single ProfilingEngine
    (core/profiling/profiling_engine.cc:70-74)."""
    global _DEFAULT_TUNER
    if _DEFAULT_TUNER is None or _DEFAULT_TUNER.flags.FC_TUNING_MODE != int(_flag("FC_TUNING_MODE")) \
            or _DEFAULT_TUNER.flags.FC_TUNING_DB_DIR != _flag("FC_TUNING_DB_DIR"):
        _DEFAULT_TUNER = Tuner()
    return _DEFAULT_TUNER.tune(family, problem, run, flops, nbytes)


def ncu_tensor_pipe_pct(family: str, params: Dict[str, int], workload: str = "small") -> Optional[float]:
    """sm__pipe_tensor_cycles_active (% of peak) of one candidate, from a one-metric ncu capture of a single launch of
    the small probe workload (``python -m flashck_b200.tuner --probe``) in a child process; None when ncu is missing or
    refuses to profile (then the CUDA-event TFLOP/s alone decides)."""
    import csv
    import io
    import shutil
    import subprocess
    import sys
    ncu = shutil.which("ncu")
    if ncu is None:
        return None
    kernel = "regex:fmha_fwd_sm100|fmha_fwd_generic" if family == "fmha_fwd" else "regex:splitkv_decode|fmha_fwd_sm100"
    cmd = [ncu, "--metrics", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "--clock-control", "none",
           "-k", kernel, "-s", "2", "-c", "1", "--csv", sys.executable, "-m", "flashck_b200.tuner", "--probe", family,
           "--workload", workload, "--params", json.dumps(params)]
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    except (OSError, subprocess.TimeoutExpired):
        return None
    rows = [l for l in r.stdout.splitlines() if l.startswith('"')]
    for row in csv.DictReader(io.StringIO("\n".join(rows))):
        if row.get("Metric Name", "").startswith("sm__pipe_tensor_cycles_active"):
            try:
                return float(row["Metric Value"].replace(",", ""))
            except ValueError:
                return None
    return None


def _environment() -> dict:
    import torch
    name = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
    return {"cuda_version": str(torch.version.cuda), "device_name": name}


def _cuda_event_timer(run: Callable[[], object], cold: int, repeats: int, flush: bool) -> float:
    """Mean milliseconds per call: `cold` untimed calls, then `repeats` timed ones; with `flush`, a buffer larger
    than the 126 MB L2 is rewritten before each timed call and each call is timed on its own."""
    import torch
    for _ in range(cold):
        run()
    torch.cuda.synchronize()
    if not flush:
        beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        beg.record()
        for _ in range(repeats):
            run()
        end.record()
        torch.cuda.synchronize()
        return beg.elapsed_time(end) / repeats
    scratch = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")
    total = 0.0
    for _ in range(repeats):
        scratch.fill_(1)
        beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        beg.record()
        run()
        end.record()
        torch.cuda.synchronize()
        total += beg.elapsed_time(end)
    return total / repeats


# --------------------------------------------------------------------------------------------------------------
# command line: tune the shipped workloads on this GPU, or run one candidate a few times for a profiler
# --------------------------------------------------------------------------------------------------------------
def _workload(name: str):
    """(family, problem, run, flops, bytes) of a seeded synthetic workload: ``small`` / ``config2`` (varlen causal
    prefill, 32/8 heads, hdim 128), ``decode_small`` / ``config3`` (paged decode, page 16), ``config4`` (1-16 query
    tokens per sequence over a paged cache, causal)."""
    import torch
    from . import ops
    from .instances import FmhaProblem
    from .utils.inputs import make_paged_cache, normal_tensor, to_seqstarts, uniform_seqlens
    dev, dt, hq, hkv, d = "cuda", torch.bfloat16, 32, 8, 128
    if name in ("small", "config2"):
        lens = uniform_seqlens(4, 512, 2048, 1234) if name == "small" else uniform_seqlens(16, 512, 4096, 1234)
        cu = to_seqstarts(lens).to(dev)
        total = sum(lens)
        q, k, v = (normal_tensor((total, h, d), dt, 1 + i).to(dev) for i, h in enumerate((hq, hkv, hkv)))
        flops = 4.0 * d * hq * sum(L * (L + 1) / 2 for L in lens)
        prob = FmhaProblem("fmha_fwd", "bf16", "group", len(lens), hq, hkv, d, d, max(lens), max(lens), "causal")
        run = lambda: ops.fmha_fwd_var_len(q, k, v, cu, cu, max(lens), causal=True, return_lse=True)
        return "fmha_fwd", prob, run, flops, None
    if name in ("decode_small", "config3"):
        lens = uniform_seqlens(16, 1024, 16384, 4321) if name == "decode_small" else uniform_seqlens(64, 1024, 32768, 4321)
        cache = make_paged_cache(lens, hkv, d, d, 16, dt, seed=5)
        k, v, bt, sl = cache.k.to(dev), cache.v.to(dev), cache.block_table.to(dev), cache.seqlen_k.to(dev)
        q = normal_tensor((len(lens), 1, hq, d), dt, 6).to(dev)
        S = ops.default_num_splits(len(lens))
        ws = ops.splitkv_workspace(q, d, S)
        prob = FmhaProblem("fmha_fwd_split_kv", "bf16", "batch", len(lens), hq, hkv, d, d, 1, bt.shape[1] * 16, "none",
                           paged=True, page=16)
        run = lambda: ops.fmha_fwd_splitkv(q, k, v, seqlen_k=sl, block_table=bt, num_splits=S, workspace=ws)
        return "fmha_fwd_split_kv", prob, run, None, float(sum(lens) * hkv * 2 * d * 2)
    if name == "config4":
        lens = uniform_seqlens(32, 2048 + 16, 16384 + 16, 777)
        new = uniform_seqlens(32, 1, 16, 778)
        cache = make_paged_cache(lens, hkv, d, d, 16, dt, seed=7)
        k, v, bt, sl = cache.k.to(dev), cache.v.to(dev), cache.block_table.to(dev), cache.seqlen_k.to(dev)
        cu = to_seqstarts(new).to(dev)
        q = normal_tensor((sum(new), hq, d), dt, 8).to(dev)
        S = ops.default_num_splits(len(lens), rows_per_kv_head=max(new) * (hq // hkv))
        ws = ops.splitkv_workspace(q, d, S, cu)
        prob = FmhaProblem("fmha_fwd_split_kv", "bf16", "group", len(lens), hq, hkv, d, d, max(new), bt.shape[1] * 16,
                           "causal", paged=True, page=16)
        run = lambda: ops.fmha_fwd_splitkv(q, k, v, seqlen_k=sl, block_table=bt, cu_seqlens_q=cu, max_seqlen_q=max(new),
                                           num_splits=S, causal=True, workspace=ws)
        return "fmha_fwd_split_kv", prob, run, None, float(sum(lens) * hkv * 2 * d * 2)
    raise SystemExit(f"unknown workload {name}")


def main(argv=None) -> None:
    import argparse
    ap = argparse.ArgumentParser(prog="python -m flashck_b200.tuner", description=__doc__.splitlines()[0])
    ap.add_argument("--tune", nargs="+", metavar="WORKLOAD", help="small, config2, decode_small, config3, config4")
    ap.add_argument("--mode", type=int, default=1, help="FC_TUNING_MODE for --tune (1 every valid instance, 2 hybrid)")
    ap.add_argument("--with-ncu", action="store_true", help="tensor-pipe %% of every prefill candidate from ncu (small case)")
    ap.add_argument("--db-dir", default=None)
    ap.add_argument("--probe", metavar="FAMILY", help="run one candidate a few times (for a profiler) and exit")
    ap.add_argument("--workload", default="small")
    ap.add_argument("--params", default="{}")
    args = ap.parse_args(argv)
    import torch
    from . import _lib
    if args.probe:
        fam = FAMILY_IDS[args.probe]
        for k, v in json.loads(args.params).items():
            _lib.set_instance_param(fam, k, int(v))
        _, _, run, _, _ = _workload(args.workload if args.probe == "fmha_fwd" or args.workload != "small" else "decode_small")
        for _ in range(4):
            run()
        torch.cuda.synchronize()
        return
    flags = TuningFlags(FC_TUNING_MODE=args.mode, FC_FORCE_PROFILING=True)
    if args.db_dir:
        flags.FC_TUNING_DB_DIR = args.db_dir
    for name in args.tune or []:
        family, prob, run, flops, nbytes = _workload(name)
        flags.FC_TUNING_METRIC = 1 if flops else 2
        util = None
        if args.with_ncu and family == "fmha_fwd":
            util = lambda inst: ncu_tensor_pipe_pct("fmha_fwd", inst.params(), "small")
        tn = Tuner(flags=flags, utilisation=util)
        best = tn.tune(family, prob, run, flops, nbytes)
        print(json.dumps({"workload": name, "problem": prob.name(), "winner": best, "candidates": tn.log}), flush=True)
        del run
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
