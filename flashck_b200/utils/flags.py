"""The reference's flag API for the flags that matter on this path.

The reference registers its flags with ``FC_DEFINE_EXPORTED_*`` (``core/utils/flags.cc:153-239``) and exposes them to
Python through four functions of its extension module (``core/pybind/pybind.cc:21-45``): ``get_flag_value(name)``
(value as a string), ``set_flag_value(name, value)`` (string, parsed by the flag's type), ``print_all_flags`` and
``print_flag_info``.  Scripts written against FlashCK set e.g. ``FC_TUNING_NUM_REPEATS`` that way; the same calls
work here, with the same names, types and defaults.  Flags of the HIP build pipeline (ROCm path, builder counts,
compiler options) have no meaning for a prebuilt CUDA library and are not registered: setting one raises, as the
reference does for an unknown flag.  A flag's initial value is taken from the environment variable of the same name
when it is set.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Dict

__all__ = ["get_flag_value", "set_flag_value", "get_flag", "print_all_flags", "print_flag_info", "flag_names"]


@dataclass
class _Flag:
    name: str
    type: type
    default: Any
    doc: str
    value: Any = None


def _parse(kind: type, text: str, name: str):
    if kind is bool:
        low = text.strip().lower()
        if low in ("1", "true", "yes", "on"):
            return True
        if low in ("0", "false", "no", "off"):
            return False
        raise RuntimeError(f"Failed to set flag: {name} (not a boolean: {text!r})")
    try:
        return kind(text)
    except ValueError:
        raise RuntimeError(f"Failed to set flag: {name} (not {kind.__name__}: {text!r})") from None


_FLAGS: Dict[str, _Flag] = {}


def _define(name: str, kind: type, default, doc: str) -> None:
    flag = _Flag(name, kind, default, doc, default)
    env = os.environ.get(name)
    if env is not None:
        flag.value = _parse(kind, env, name)
    _FLAGS[name] = flag


# names, types, defaults and texts of core/utils/flags.cc (line numbers there)
_define("FC_TUNING_DB_DIR", str, "", "Directory for profiler cache storage")                                   # :157
_define("FC_CONFIG_JSON_PATH", str, "", "Path to the JSON configuration file")                                 # :159
_define("FC_FORCE_PROFILING_DB", bool, True, "Force the profiler to use cached results")                       # :201
_define("FC_FORCE_PROFILING", bool, True, "Force profiling even if cached results exist")                      # :203
_define("FC_FLUSH_PROFILING_DB", bool, False, "Flush profile cache database on startup")                       # :205
_define("FC_ENABLE_DEFAULT_JSON", bool, False, "Enable default JSON configuration")                            # :207
_define("FC_ENABLE_USER_JSON", bool, True, "Enable user JSON configuration")                                   # :209
_define("FC_TUNING_MODE", int, 1, "Tuning mode: 0=heuristic, 1=autotuning, 2=hybrid")                          # :213
_define("FC_TUNING_METRIC", int, 0, "Profiling metric: 0=latency, 1=throughput(TFLOPS), 2=bandwidth")          # :215
_define("FC_TUNING_NUM_COLD_ITERATION", int, 16, "Number of warm-up iterations for profiling")                 # :217
_define("FC_TUNING_NUM_REPEATS", int, 64, "Number of profiling iterations for measurements")                   # :219
_define("FC_TUNING_GPU_TIMER", bool, True, "Enable GPU timer for accurate profiling")                          # :221
_define("FC_TUNING_SEED", int, 42, "Random seed for tuning")                                                   # :225
_define("FC_TUNING_LOG", bool, False, "Enable detailed tuning logs")                                           # :229
_define("FC_TUNING_FLUSH_CACHE", bool, True, "Flush cache before profiling measurements")                      # :231
_define("FC_TUNING_ROTATING_COUNT", int, 1, "Number of rotating profiling runs")                               # :233
_define("FC_CALL_STACK_LEVEL", int, 1, "Error call stack detail level: 0=summary, 1=+Python, 2=+C++")          # :239


def flag_names():
    return sorted(_FLAGS)


def _lookup(name: str) -> _Flag:
    flag = _FLAGS.get(name)
    if flag is None:
        raise RuntimeError(f"Flag not found: {name}")
    return flag


def get_flag(name: str):
    """The flag's value in its own type."""
    return _lookup(name).value


def get_flag_value(name: str) -> str:
    """The flag's value as a string (booleans as ``true`` / ``false``), like the reference's binding."""
    value = _lookup(name).value
    return ("true" if value else "false") if isinstance(value, bool) else str(value)


def set_flag_value(name: str, value) -> None:
    """Sets a flag from a string (or a value of the flag's type).  Unknown flag or unparsable text raises."""
    flag = _FLAGS.get(name)
    if flag is None:
        raise RuntimeError(f"Failed to set flag: {name}")
    flag.value = value if isinstance(value, flag.type) and not (flag.type is int and isinstance(value, bool)) \
        else _parse(flag.type, str(value), name)
    if name == "FC_TUNING_LOG":  # detailed logs include the library's own: which instance a call ran on, and why
        from .. import _lib
        _lib.apply_logging_flag()


def print_flag_info(name: str) -> None:
    f = _lookup(name)
    print(f"{f.name} ({f.type.__name__}) = {get_flag_value(name)}  [default {f.default!r}]  {f.doc}")


def print_all_flags(writable_only: bool = False) -> None:
    for name in flag_names():  # every flag here is writable
        print_flag_info(name)
