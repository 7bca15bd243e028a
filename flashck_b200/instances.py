"""Kernel-instance schema of the attention families: what the tuner enumerates, checks and names.

In the reference an instance is a ck_tile tile shape ``{m0,n0,k0,n1,k1,k0max, warps, warp tiles}`` plus traits,
pipeline and launch bounds (``core/profiling/attention/fmha_fwd/fmha_fwd_codegen.h:20-112``,
``fmha_fwd_split_kv/fmha_fwd_split_kv_codegen.h:17-121``); its emitter expands the JSON search space into a Cartesian
product, drops shapes that cannot work (``IsValidTile``, ``fmha_fwd_emitter.cc:15-67``), optionally narrows the rest by
rules of thumb (``HeuristicFilter``, ``:74-130``) and names every survivor (``fmha_fwd_codegen.cc:5-27,60-81``) -- the
name is the key of the tuning cache.

On B200 the quantities that matter are different, so the schema is: query / key tile (``block_m`` x ``block_n`` rows of
tcgen05.mma or mma.sync), ``head_dim``, depth of the K/V shared-memory ring (``kv_stages``), softmax warpgroups, the
pipeline (tcgen05 + TMEM + TMA, or the general mma.sync instance), how the softmax takes its exponentials, and for
split-KV the page gather (``tokens_per_tile``, ``heads_per_cta``, ``row_tiles``), the work cut and the split count.
Parameters that are template constants of the compiled library appear in the JSON with the single value that is
built; :func:`is_valid` rejects the rest, so widening the library widens the search space without touching the tuner.

Everything here is host logic (no CUDA): it runs in the CPU test suite.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional

SMEM_PER_CTA = 227 * 1024  # bytes a CTA can have on sm_100a
TMEM_COLUMNS = 512         # 32-bit columns of tensor memory per SM
MAX_WARPS_DECODE = 8       # consumer warps of the split-KV decode kernel


# --------------------------------------------------------------------------------------------------------------
# problems
# --------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class FmhaProblem:
    """What the tuning cache is keyed by -- the fields of the reference's FmhaFwdProblem / FmhaFwdSplitKVProblem that
    select or size an instance (``fmha_fwd_problem.h:59-95``, ``fmha_fwd_split_kv_problem.h``).  Lengths are bucketed to
    powers of two so that neighbouring problems share a record."""
    family: str            # "fmha_fwd" | "fmha_fwd_split_kv"
    dtype: str             # "fp16" | "bf16" | "fp8" (E4M3) | "bf8" (E5M2)
    mode: str              # "batch" | "group"
    batch: int
    hq: int
    hkv: int
    d: int
    dv: int
    max_seqlen_q: int
    max_seqlen_k: int
    mask: str = "none"     # "none" | "causal" | "window"
    bias: str = "none"     # "none" | "elementwise" | "alibi"
    soft_cap: bool = False
    paged: bool = False
    page: int = 0

    def name(self) -> str:
        return (f"{self.dtype}_{self.mode}_b{self.batch}_h{self.hq}x{self.hkv}_d{self.d}x{self.dv}_"
                f"sq{self.max_seqlen_q}_sk{self.max_seqlen_k}_{self.mask}_{self.bias}{'_cap' if self.soft_cap else ''}"
                f"{'_p' + str(self.page) if self.paged else ''}")

    def key(self) -> dict:
        d = asdict(self)
        d["max_seqlen_q"] = _bucket(self.max_seqlen_q)
        d["max_seqlen_k"] = _bucket(self.max_seqlen_k)
        d["batch"] = _bucket(self.batch)
        return d


def _bucket(n: int) -> int:
    n = max(int(n), 1)
    return 1 << (n - 1).bit_length()


# --------------------------------------------------------------------------------------------------------------
# instances
# --------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class FmhaFwdInstance:
    """One forward / prefill instance.  ``pipeline``: 1 = tcgen05 (TMEM accumulators, TMA-staged tiles, warp-specialised),
    0 = general (mma.sync, cp.async).  ``exp_mode``: 0 fp32 exp2 unit, 1 packed f16x2 exp2 unit, 11/12/13 fp32 with
    1/2/3 of every 8 column pairs on an FMA-pipe polynomial.  ``rescale_log2_x100``: lazy-rescale threshold of the
    packed-exp2 softmax."""
    block_m: int = 128
    block_n: int = 128
    head_dim: int = 128
    kv_stages: int = 2
    softmax_wgs: int = 2
    pipeline: int = 1
    exp_mode: int = 0
    rescale_log2_x100: int = 200
    max_thread_per_block: int = 384
    min_block_per_cu: int = 1

    def canonical(self) -> "FmhaFwdInstance":
        """The same instance with the parameters it does not read at their defaults (so that combinations of the search
        space that differ only there collapse into one candidate)."""
        from dataclasses import replace
        t = self if self.exp_mode == 1 else replace(self, rescale_log2_x100=200)
        return replace(t, max_thread_per_block=384 if t.pipeline else 128)

    def params(self) -> Dict[str, int]:
        """The run-time instance parameters of family 0 that select this instance (FlashckSetInstanceParam)."""
        out = {"use_sm100": self.pipeline, "exp_mode": self.exp_mode}
        if self.exp_mode == 1:
            out["rescale_log2_x100"] = self.rescale_log2_x100
        return out

    def name(self, problem: Optional[FmhaProblem] = None) -> str:
        # fmha_fwd_{problem}_{tile}_{trait}_{pipeline}_{launch}, the reference's order (fmha_fwd_codegen.cc:60-81)
        tile = f"{self.block_m}x{self.block_n}x{self.head_dim}_s{self.kv_stages}_wg{self.softmax_wgs}"
        trait = f"x{self.exp_mode}" + (f"r{self.rescale_log2_x100}" if self.exp_mode == 1 else "")
        pipe = "tc05" if self.pipeline else "mma"
        launch = f"{self.max_thread_per_block}_{self.min_block_per_cu}"
        return "_".join(x for x in ("fmha_fwd", problem.name() if problem else "", tile, trait, pipe, launch) if x)


@dataclass(frozen=True)
class FmhaFwdSplitKVInstance:
    """One split-KV instance.  ``pipeline`` 0: the TMA-gather decode kernel (mma.sync, ``tokens_per_tile`` = 16 keys per
    ring stage, ``heads_per_cta`` kv heads and ``row_tiles`` 16-row query tiles per CTA); 1: the tcgen05 kernel's split
    modes (128 keys per stage) for more than 16 query rows per kv head.  ``num_splits`` 0 = the library's default."""
    tokens_per_tile: int = 16
    heads_per_cta: int = 0
    row_tiles: int = 0
    stages: int = 0
    ctas_per_sm_x100: int = 100
    pipeline: int = 1
    exp_mode: int = 0
    split_item_cost: int = 6
    split_min_piece_tiles: int = 8
    num_splits: int = 0

    def canonical(self) -> "FmhaFwdSplitKVInstance":
        from dataclasses import replace
        if self.pipeline:
            return replace(self, heads_per_cta=0, row_tiles=0, stages=0, ctas_per_sm_x100=100)
        return replace(self, exp_mode=0, split_item_cost=6, split_min_piece_tiles=8)

    def params(self) -> Dict[str, int]:
        return {"use_sm100_splitkv": self.pipeline, "stages": self.stages, "ctas_per_sm_x100": self.ctas_per_sm_x100,
                "heads_per_cta": self.heads_per_cta, "row_tiles": self.row_tiles, "exp_mode_splitkv": self.exp_mode,
                "split_item_cost": self.split_item_cost, "split_min_piece_tiles": self.split_min_piece_tiles}

    def name(self, problem: Optional[FmhaProblem] = None) -> str:
        tile = f"t{self.tokens_per_tile}_hk{self.heads_per_cta}_mt{self.row_tiles}_s{self.stages}"
        cut = f"c{self.ctas_per_sm_x100}_ic{self.split_item_cost}_mp{self.split_min_piece_tiles}_ns{self.num_splits}"
        pipe = ("tc05" if self.pipeline else "mma") + f"_x{self.exp_mode}"
        return "_".join(x for x in ("fmha_fwd_splitkv", problem.name() if problem else "", tile, cut, pipe) if x)


FAMILY_INSTANCE = {"fmha_fwd": FmhaFwdInstance, "fmha_fwd_split_kv": FmhaFwdSplitKVInstance}


def from_config(family: str, cfg: Dict[str, int]):
    """Instance from one combination of the JSON search space (unknown keys are an error, missing ones default)."""
    cls = FAMILY_INSTANCE[family]
    fields = set(cls.__dataclass_fields__)
    unknown = set(cfg) - fields
    if unknown:
        raise KeyError(f"{family}: unknown instance parameter(s) {sorted(unknown)}")
    return cls(**{k: int(v) for k, v in cfg.items()})


# --------------------------------------------------------------------------------------------------------------
# validity (the reference's IsValidTile) and rules of thumb (its HeuristicFilter)
# --------------------------------------------------------------------------------------------------------------
def why_invalid(inst, problem: FmhaProblem) -> Optional[str]:
    """None when the compiled library has this instance and it can run the problem; else the reason."""
    if isinstance(inst, FmhaFwdInstance):
        return _why_invalid_fwd(inst, problem)
    return _why_invalid_split(inst, problem)


def is_valid(inst, problem: FmhaProblem) -> bool:
    return why_invalid(inst, problem) is None


def _why_invalid_fwd(t: FmhaFwdInstance, p: FmhaProblem) -> Optional[str]:
    if min(t.block_m, t.block_n, t.head_dim, t.kv_stages, t.softmax_wgs, t.max_thread_per_block, t.min_block_per_cu) <= 0:
        return "tile parameters must be positive"
    if t.head_dim != p.d or p.d != p.dv:
        return f"head_dim {t.head_dim} does not match the problem ({p.d}/{p.dv})"
    if t.exp_mode not in (0, 1, 11, 12, 13):
        return f"exp_mode {t.exp_mode} is not built"
    if not 0 <= t.rescale_log2_x100 <= 1400:
        return "rescale_log2_x100 outside [0, 1400]"
    f8 = p.dtype in ("fp8", "bf8")
    esize = 1 if f8 else 2
    if f8 and (p.bias != "none" or p.soft_cap):
        return "the 8-bit element types take no bias and no soft cap"
    if t.pipeline == 1:
        if (t.block_m, t.block_n) != (128, 128) or t.head_dim not in (64, 128):
            return "the tcgen05 instance is built for 128 x 128 tiles at head_dim 128 or 64"
        if f8 and (t.head_dim != 128 or p.paged or t.exp_mode != 0):
            return "the kind::f8f6f4 tcgen05 instances: head_dim 128, contiguous K/V, fp32 exponentials on the exp2 unit"
        if t.head_dim == 64 and t.exp_mode != 0:
            return "the hdim-64 tcgen05 instances take their exponentials in fp32 on the exp2 unit"
        if t.kv_stages != 2 or t.softmax_wgs != 2 or t.min_block_per_cu != 1:
            return "the tcgen05 instance is built with a 2-slot K/V ring, 2 softmax warpgroups, 384 threads, 1 CTA per SM"
        # S and O accumulators of two Q tiles: fp32 columns of tensor memory
        if 2 * t.block_n + 2 * t.head_dim > TMEM_COLUMNS:
            return "S and O accumulators of two query tiles exceed the 512 TMEM columns"
        # two Q tiles, the K and V rings, 8 x 2 KB of O staging, alignment slack, the on-chip schedule (17 KB)
        smem = (2 * t.block_m + 2 * t.kv_stages * t.block_n) * t.head_dim * esize + 16 * 1024 + 1024 + 17 * 1024
        if smem > SMEM_PER_CTA:
            return f"tiles, staging and schedule need {smem} bytes of shared memory"
        if p.bias == "elementwise" and (t.head_dim != 128 or p.paged or t.exp_mode != 0):
            return "the elementwise-bias tcgen05 instances: head_dim 128, contiguous K/V, fp32 exponentials on the exp2 unit"
        if (p.bias != "none" or p.soft_cap) and t.exp_mode != 0:
            return "the score-addition instances (ALiBi, soft cap) take their exponentials in fp32 on the exp2 unit"
        if p.batch > 256 or (p.max_seqlen_q + 127) // 128 > 512 or p.hq > 1023:
            return "beyond the on-chip schedule (256 sequences, 512 row blocks, 1023 heads)"
        if p.paged and (p.page < 16 or not (128 % p.page == 0 or p.page % 128 == 0)):
            return "paged K/V needs pages of 16..128 tokens dividing 128, or multiples of 128"
    else:
        if (t.block_m, t.block_n) != (64, 64) or t.head_dim not in (64, 128):
            return "the general instance is built for 64 x 64 tiles at head_dim 64 or 128"
        if t.kv_stages != 2 or t.exp_mode != 0:
            return "the general instance has a double buffer and fp32 exponentials"
        if (t.block_m + 2 * t.kv_stages * t.block_n) * t.head_dim * esize > SMEM_PER_CTA:
            return "tiles exceed shared memory"
    return None


def _why_invalid_split(t: FmhaFwdSplitKVInstance, p: FmhaProblem) -> Optional[str]:
    if min(t.tokens_per_tile, t.ctas_per_sm_x100, t.split_item_cost, t.split_min_piece_tiles) <= 0 or \
            min(t.heads_per_cta, t.row_tiles, t.stages, t.num_splits) < 0:
        return "negative or zero tile parameter"
    if p.d != p.dv or p.d not in (64, 128):
        return "hdim_q == hdim_v in {64, 128} required"
    group = p.hq // max(p.hkv, 1)
    rows = p.max_seqlen_q * group
    if t.num_splits > 1024:
        return "num_splits above 1024"
    if t.pipeline == 1:
        if t.tokens_per_tile != 128:
            return "the tcgen05 split modes read 128 keys per stage"
        if p.d != 128 or rows <= 16 or (rows + 127) // 128 > 16 or group > 128 or 128 % max(group, 1) != 0:
            return "the tcgen05 split modes serve head_dim 128 with 17..2048 query rows per kv head"
        if p.mask == "window" or p.bias != "none" or p.batch > 256:
            return "no window, bias or batches above 256 on the tcgen05 split modes"
        if p.paged and (p.page < 16 or not (128 % p.page == 0 or p.page % 128 == 0)):
            return "pages of 16..128 tokens dividing 128, or multiples of 128"
        if t.exp_mode not in (0, 1) or not 1 <= t.split_item_cost <= 64 or t.split_min_piece_tiles > 4096:
            return "exp_mode_splitkv in {0, 1}, split_item_cost in [1, 64], split_min_piece_tiles <= 4096"
        if t.num_splits > 255:
            return "at most 255 splits on the tcgen05 split modes"
        return None
    if t.tokens_per_tile != 16:
        return "the decode kernel reads 16 keys per stage"
    if p.paged and p.page % t.tokens_per_tile != 0:
        return "page_block_size must be a multiple of tokens_per_tile"
    if t.heads_per_cta not in (0, 1, 2, 4, 8) or t.row_tiles not in (0, 1, 2, 4):
        return "heads_per_cta in {0,1,2,4,8}, row_tiles in {0,1,2,4}"
    hk = t.heads_per_cta or 8
    mt = t.row_tiles or (1 if rows <= 16 else 2 if rows <= 32 else 4)
    if t.heads_per_cta and (p.hkv % hk != 0 or hk * mt > MAX_WARPS_DECODE):
        return "heads_per_cta must divide nhead_k and heads_per_cta * row_tiles fit 8 warps"
    if t.exp_mode != 0:
        return "the decode kernel has fp32 exponentials"
    if p.batch > 8192:
        return "batch above 8192"
    tile_bytes = t.tokens_per_tile * min(hk, p.hkv) * p.d * 2
    need = 2 if t.stages == 0 else t.stages
    if need < 2 or need > 12:
        return "stages in [2, 12] (0 = as many as fit)"
    if 1024 + (2 * p.batch + 5) * 4 + need * (2 * tile_bytes + 24) > SMEM_PER_CTA:
        return "the K/V ring does not fit shared memory"
    return None


def heuristic_filter(instances: List, problem: FmhaProblem) -> List:
    """Rules of thumb that narrow the valid instances before timing (FC_TUNING_MODE 0 takes the first survivor, 2 times
    the survivors, 1 times every valid instance).  Never returns an empty list when given a non-empty one."""
    keep = []
    group = problem.hq // max(problem.hkv, 1)
    for t in instances:
        if isinstance(t, FmhaFwdInstance):
            # tensor memory pipeline whenever it is built for the problem; the polynomial shares and the packed exp2 form
            # only ever lost to the plain exp2 unit on hdim 128 (they cost issue slots of the softmax warps)
            if t.pipeline == 0 and any(isinstance(u, FmhaFwdInstance) and u.pipeline == 1 for u in instances):
                continue
            if t.exp_mode != 0:
                continue  # (the packed exp2 form also trades LSE accuracy: up to 1e-3 on rows that one key dominates)
        else:
            rows = problem.max_seqlen_q * group
            if rows > 16 and t.pipeline == 0 and any(u.pipeline == 1 for u in instances):
                continue  # several row tiles per kv head: the decode kernel is latency-bound there
            if t.pipeline == 0 and t.stages not in (0, 3):
                continue  # three 64 KB stages keep the HBM pipe full; deeper rings do not fit at 8 heads x hdim 128
            if t.ctas_per_sm_x100 != 100:
                continue  # the equal-piece work cut assumes one CTA per SM
        keep.append(t)
    return keep or instances[: min(len(instances), 10)]
