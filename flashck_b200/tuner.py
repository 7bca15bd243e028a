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
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional

__all__ = ["TuningFlags", "load_search_space", "expand_param", "cartesian_product", "ProfilingDB", "Tuner",
           "FAMILY_IDS"]

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


def instance_name(family: str, cfg: Dict[str, int]) -> str:
    return family + "_" + "_".join(f"{k}{v}" for k, v in sorted(cfg.items()))


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
            "split_k INTEGER NOT NULL DEFAULT -1, latency REAL, tflops REAL, bandwidth REAL)")
        self.conn.commit()

    @staticmethod
    def _key(d: dict) -> str:
        return json.dumps(d, sort_keys=True)

    def query(self, env: dict, setting: dict, problem: dict) -> Optional[dict]:
        row = self.conn.execute(
            "SELECT instance_name, instance, latency, tflops, bandwidth FROM fmha WHERE cuda_version=? AND device_name=? "
            "AND setting=? AND problem=? ORDER BY id DESC LIMIT 1",
            (env["cuda_version"], env["device_name"], self._key(setting), self._key(problem))).fetchone()
        if row is None:
            return None
        return {"instance_name": row[0], "instance": json.loads(row[1]), "latency": row[2], "tflops": row[3],
                "bandwidth": row[4]}

    def insert(self, env: dict, setting: dict, problem: dict, name: str, instance: dict, latency: float,
               tflops: Optional[float], bandwidth: Optional[float]) -> None:
        self.conn.execute(
            "INSERT INTO fmha (cuda_version, device_name, setting, problem, instance_name, instance, latency, tflops, "
            "bandwidth) VALUES (?,?,?,?,?,?,?,?,?)",
            (env["cuda_version"], env["device_name"], self._key(setting), self._key(problem), name,
             json.dumps(instance, sort_keys=True), latency, tflops, bandwidth))
        self.conn.commit()

    def flush(self) -> None:
        """FC_FLUSH_PROFILING_DB: drop every cached result."""
        self.conn.execute("DELETE FROM fmha")
        self.conn.commit()


@dataclass
class Tuner:
    """Times the candidates of one family on a caller-supplied workload and applies the winner.

    ``timer(run, cold, repeats, flush)`` returns milliseconds per call; the default uses CUDA events.  ``apply`` sets
    one instance parameter (default: ``FlashckSetInstanceParam``).  Both are injectable so that the selection logic
    is testable without a GPU."""
    flags: TuningFlags = field(default_factory=TuningFlags)
    db: Optional[ProfilingDB] = None
    timer: Optional[Callable] = None
    apply: Optional[Callable[[int, str, int], None]] = None
    env: Optional[dict] = None

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

    def candidates(self, family: str) -> List[Dict[str, int]]:
        cands = cartesian_product(load_search_space(family, self.flags.FC_CONFIG_JSON_PATH))
        return cands[:1] if self.flags.FC_TUNING_MODE == 0 else cands

    def _score(self, ms: float, flops: Optional[float], nbytes: Optional[float]) -> float:
        m = self.flags.FC_TUNING_METRIC
        if m == 1 and flops:
            return flops / ms
        if m == 2 and nbytes:
            return nbytes / ms
        return -ms

    def tune(self, family: str, problem: dict, run: Callable[[], object], flops: Optional[float] = None,
             nbytes: Optional[float] = None) -> dict:
        """Returns the winning record and leaves its parameters applied."""
        fam = FAMILY_IDS[family]
        cached = None if self.flags.FC_FORCE_PROFILING else self.db.query(self.env, self.setting(), problem)
        if cached is not None:
            for k, v in cached["instance"].items():
                self.apply(fam, k, v)
            return cached
        best = None
        for cfg in self.candidates(family):
            for k, v in cfg.items():
                self.apply(fam, k, v)
            ms = float(self.timer(run, self.flags.FC_TUNING_NUM_COLD_ITERATION, self.flags.FC_TUNING_NUM_REPEATS,
                                  self.flags.FC_TUNING_FLUSH_CACHE))
            rec = {"instance_name": instance_name(family, cfg), "instance": cfg, "latency": ms,
                   "tflops": flops / ms / 1e9 if flops else None, "bandwidth": nbytes / ms / 1e6 if nbytes else None}
            if best is None or self._score(ms, flops, nbytes) > self._score(best["latency"], flops, nbytes):
                best = rec
        if best is None:
            raise RuntimeError(f"no candidate instance for family {family}")
        for k, v in best["instance"].items():
            self.apply(fam, k, v)
        self.db.insert(self.env, self.setting(), problem, best["instance_name"], best["instance"], best["latency"],
                       best["tflops"], best["bandwidth"])
        return best


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
