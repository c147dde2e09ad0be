"""Analytical choice of the grid for seed-only decode on B200.

Same surface as the reference's ``stream_attention/seed_autotune.py`` (shape /
candidate / result records :17-160, ``seed_kernel_candidates`` :166-283,
``autotune_seed_kernel_mode`` :298-330, ``seed_shape_from_policy`` :333-354),
re-derived for this package's kernel.

The reference ranks three Triton kernel modes (one CTA per query head reading its
own copy of the seed K/V, the same split into chunks, and a GQA-shared variant
that it does not ship).  Here there is one kernel: it always reads a seed token
once per KV head and shares it among the query heads of the group, so the only
thing left to choose is how many CTAs work on one (row, KV head) pair.  A
candidate is therefore "``seed_chunks`` CTAs per pair"; its cost comes from a
latency model of the kernel fitted to a sweep on a B200 (batch 1-8, 128-1024 seed
tokens, 1-16 CTAs per pair; the model's grid is the fastest measured one, or within
4 % of it, on every cell of that sweep):

``t = T0 + rounds * T_ROUND + tiles_per_cta * T_TILE + straddle(chunks) + merge(chunks)``

* a CTA has 8 warps with one 16 KB K+V tile in flight each, so it needs
  ``rounds = ceil(tiles_per_cta / 8)`` trips to HBM (``T_ROUND`` each) and moves
  its tiles at about 110 GB/s per SM (``T_TILE`` per tile);
* with two or three CTAs per pair the kernel cuts the tile list into equal slices,
  and unless a pair's tiles divide evenly one CTA then straddles two pairs and
  flushes its state twice (``STRADDLE_US``); from four CTAs per pair on, the slices
  are snapped to pair boundaries.  Either way the partition is worked out before
  the launch's dependency wait, i.e. while the previous kernel of the stream drains,
  and costs nothing in a decode loop;
* more than one CTA per pair adds the in-launch merge of their split states by the
  pair's first CTA: one round trip to L2 for the states (the merging CTA asks for 3, 6 or 10
  states per thread, whichever covers the pair; more states take further round
  trips), the output store.

Few seed tokens are served fastest by ONE CTA per pair (no merge at all); from
about 12 tiles per pair on, splitting the pair over several CTAs wins.
"""

from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import Iterable, List, Optional, Tuple

B200_SM_COUNT = 148
TILE_BYTES = 16384          # one K tile + one V tile of the streaming kernel
WARPS_PER_CTA = 8
# Fitted constants, microseconds (B200, SM clock 1965 MHz, programmatic dependent launch on).
T0_US = 3.0                 # launch, what is left of the set-up after the dependency wait, output store
T_ROUND_US = 0.9            # one more dependent trip to HBM for a warp
T_TILE_US = 0.15            # 16 KB through one SM
ALIGNED_CHUNKS = 4          # CTAs per pair from which the slices are snapped to pair boundaries
STRADDLE_US = 3.5           # equal slices that do not end on pair boundaries: a CTA flushes twice
MERGE_TIERS_US = ((3, 1.8), (6, 2.2), (10, 2.75))  # (states per thread the batch covers, cost)
MERGE_EXTRA_PASS_US = 2.2   # per further batch of split states the merging CTA has to request
MERGE_STATES_PER_THREAD = MERGE_TIERS_US[-1][0]


@dataclass(frozen=True)
class SeedKernelShape:
    """Shape and seed schedule of a seed-only decode call (fields as in the reference)."""

    batch: int
    q_heads: int
    kv_heads: int
    kv_len: int
    dim: int
    block_size: int
    sink_blocks: int
    recent_blocks: int
    middle_seed_blocks: int
    dtype_bytes: int = 2

    def __post_init__(self) -> None:
        for name in ("batch", "q_heads", "kv_heads", "kv_len", "dim", "block_size", "dtype_bytes"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive")
        if self.q_heads % self.kv_heads != 0:
            raise ValueError("q_heads must be divisible by kv_heads for true GQA")
        for name in ("sink_blocks", "recent_blocks", "middle_seed_blocks"):
            if getattr(self, name) < 0:
                raise ValueError(f"{name} must be non-negative")

    # Derived quantities (names and values as in the reference's record, whose to_dict() is the
    # interchange format).  Byte counts are K plus V over `heads` heads and `tokens` tokens.

    def _kv_bytes(self, heads: int, tokens: int) -> int:
        return 2 * self.batch * heads * tokens * self.dim * self.dtype_bytes

    group_size = property(lambda self: self.q_heads // self.kv_heads, doc="query heads per KV head")
    seed_blocks = property(lambda self: self.sink_blocks + self.recent_blocks + self.middle_seed_blocks)
    seed_tokens = property(lambda self: min(self.kv_len, self.seed_blocks * self.block_size),
                           doc="tokens the seed schedule reads (the cache length at most)")
    seed_token_ratio = property(lambda self: self.seed_tokens / float(self.kv_len))
    head_private_kv_byte_ratio = property(
        lambda self: self.group_size * self.seed_token_ratio,
        doc="seed K/V bytes over exact K/V bytes if every query head reloaded the seed K/V")
    gqa_shared_kv_byte_ratio = property(
        lambda self: self.seed_token_ratio,
        doc="seed K/V bytes over exact K/V bytes with K/V shared inside a group (what the kernel does)")
    exact_kv_bytes = property(lambda self: self._kv_bytes(self.kv_heads, self.kv_len))
    head_private_seed_kv_bytes = property(lambda self: self._kv_bytes(self.q_heads, self.seed_tokens))
    gqa_shared_seed_kv_bytes = property(lambda self: self._kv_bytes(self.kv_heads, self.seed_tokens))

    # -- what the streaming kernel makes of the shape ---------------------------------------

    @property
    def pairs(self) -> int:
        """(row, KV head) pairs: the units the kernel's CTAs are dealt to."""

        return self.batch * self.kv_heads

    @property
    def tile_tokens(self) -> int:
        return max(1, TILE_BYTES // 2 // (self.dim * self.dtype_bytes))

    @property
    def tiles_per_pair(self) -> int:
        return max(1, math.ceil(self.seed_tokens / self.tile_tokens))

    def to_dict(self) -> dict:
        data = asdict(self)
        for name in ("group_size", "seed_blocks", "seed_tokens", "seed_token_ratio", "head_private_kv_byte_ratio",
                     "gqa_shared_kv_byte_ratio", "exact_kv_bytes", "head_private_seed_kv_bytes",
                     "gqa_shared_seed_kv_bytes"):
            data[name] = getattr(self, name)
        return data


@dataclass(frozen=True)
class SeedKernelCandidate:
    """One grid for the seed-only kernel: ``seed_chunks`` CTAs per (row, KV head) pair."""

    mode: str
    seed_tile_tokens: int            # seed tokens one CTA reads
    seed_chunks: int                 # CTAs per pair (1: no merge)
    cta_count: int
    occupancy_threshold_ctas: int    # grids up to this size run as one wave
    kv_byte_ratio_vs_exact: float
    row_work_ratio_vs_exact: float
    duplicate_kv_across_q_heads: bool
    viable_duplication: bool
    viable_occupancy: bool
    recommendation_score: float      # minus the predicted microseconds: higher is better
    predicted_us: float = 0.0

    @property
    def viable(self) -> bool:
        return self.viable_duplication and self.viable_occupancy

    def to_dict(self) -> dict:
        data = asdict(self)
        data["viable"] = self.viable
        return data


@dataclass(frozen=True)
class SeedKernelAutotuneResult:
    """Outcome of :func:`autotune_seed_kernel_mode`."""

    shape: SeedKernelShape
    sm_count: int
    target_waves: float
    duplication_byte_budget: float
    occupancy_threshold_ctas: int
    candidates: Tuple[SeedKernelCandidate, ...]
    recommended_mode: str
    recommended_seed_tile_tokens: int
    decision: str
    recommended_num_ctas: int = 0
    predicted_us: float = 0.0

    def to_dict(self) -> dict:
        return {
            "schema": "streamattn_b200.seed_kernel_grid_autotune.v1",
            "shape": self.shape.to_dict(),
            "sm_count": self.sm_count,
            "target_waves": self.target_waves,
            "duplication_byte_budget": self.duplication_byte_budget,
            "occupancy_threshold_ctas": self.occupancy_threshold_ctas,
            "candidates": [candidate.to_dict() for candidate in self.candidates],
            "recommended_mode": self.recommended_mode,
            "recommended_seed_tile_tokens": self.recommended_seed_tile_tokens,
            "recommended_num_ctas": self.recommended_num_ctas,
            "predicted_us": self.predicted_us,
            "decision": self.decision,
        }


def predicted_seed_decode_us(shape: SeedKernelShape, chunks: int) -> float:
    """Latency model of the seed-only launch with ``chunks`` CTAs per (row, KV head) pair."""

    if chunks <= 0:
        raise ValueError("chunks must be positive")
    tiles_per_cta = math.ceil(shape.tiles_per_pair / chunks)
    rounds = math.ceil(tiles_per_cta / WARPS_PER_CTA)
    t = T0_US + rounds * T_ROUND_US + tiles_per_cta * T_TILE_US
    if chunks > 1:
        if chunks < ALIGNED_CHUNKS and shape.tiles_per_pair % chunks:
            t += STRADDLE_US
        # 256 threads share the (head row, 4 columns) work items of the group; each requests the
        # states of its item in batches sized to the pair.
        items = shape.group_size * max(1, shape.dim // 4)
        threads_per_item = max(1, (WARPS_PER_CTA * 32) // items)
        per_thread = math.ceil(chunks / threads_per_item)
        passes = math.ceil(per_thread / MERGE_STATES_PER_THREAD)
        t += next((cost for covers, cost in MERGE_TIERS_US if per_thread <= covers), MERGE_TIERS_US[-1][1])
        t += (passes - 1) * MERGE_EXTRA_PASS_US
    return t


def _chunk_counts(shape: SeedKernelShape, sm_count: int, seed_tile_tokens: Optional[Iterable[int]]) -> List[int]:
    most = max(1, min(shape.tiles_per_pair, sm_count // shape.pairs if shape.pairs <= sm_count else 1))
    counts = set(range(1, min(most, 16) + 1))
    counts.update(c for c in (24, 32, 48, 64) if c <= most)
    for tokens in seed_tile_tokens or ():  # the reference's knob: tokens per CTA
        if int(tokens) > 0:
            counts.add(max(1, min(most, math.ceil(shape.seed_tokens / int(tokens)))))
    return sorted(counts)


def seed_kernel_candidates(shape: SeedKernelShape, *, sm_count: int = B200_SM_COUNT, target_waves: float = 1.0,
                           seed_tile_tokens: Optional[Iterable[int]] = None,
                           duplication_byte_budget: float = 0.15) -> List[SeedKernelCandidate]:
    """Candidate grids, best first.

    ``seed_tile_tokens`` adds grids by "seed tokens per CTA" (the reference's way of naming a
    split).  ``target_waves`` bounds the grid: candidates larger than ``sm_count * target_waves``
    CTAs are listed as not viable.  ``duplication_byte_budget`` is accepted for signature
    compatibility: this kernel never duplicates K/V reads across query heads.
    """

    if sm_count <= 0:
        raise ValueError("sm_count must be positive")
    if target_waves <= 0.0:
        raise ValueError("target_waves must be positive")
    if duplication_byte_budget <= 0.0:
        raise ValueError("duplication_byte_budget must be positive")
    threshold = max(1, math.floor(float(sm_count) * float(target_waves)))
    candidates = []
    for chunks in _chunk_counts(shape, sm_count, seed_tile_tokens):
        predicted = predicted_seed_decode_us(shape, chunks)
        ctas = shape.pairs * chunks
        candidates.append(SeedKernelCandidate(
            mode="gqa_shared_seed", seed_tile_tokens=math.ceil(shape.seed_tokens / chunks), seed_chunks=chunks,
            cta_count=ctas, occupancy_threshold_ctas=threshold,
            kv_byte_ratio_vs_exact=shape.gqa_shared_kv_byte_ratio, row_work_ratio_vs_exact=shape.seed_token_ratio,
            duplicate_kv_across_q_heads=False, viable_duplication=True,
            viable_occupancy=ctas <= threshold or chunks == 1, recommendation_score=-predicted,
            predicted_us=predicted))
    # Best first; ties go to the smaller grid.
    return sorted(candidates, key=lambda c: (not c.viable, c.predicted_us, c.cta_count))


def autotune_seed_kernel_mode(shape: SeedKernelShape, *, sm_count: int = B200_SM_COUNT, target_waves: float = 1.0,
                              seed_tile_tokens: Optional[Iterable[int]] = None,
                              duplication_byte_budget: float = 0.15) -> SeedKernelAutotuneResult:
    """Pick the grid of a seed-only route; ``recommended_num_ctas`` is what a plan should be built with."""

    candidates = seed_kernel_candidates(shape, sm_count=sm_count, target_waves=target_waves,
                                        seed_tile_tokens=seed_tile_tokens,
                                        duplication_byte_budget=duplication_byte_budget)
    best = candidates[0]
    return SeedKernelAutotuneResult(
        shape=shape, sm_count=sm_count, target_waves=target_waves, duplication_byte_budget=duplication_byte_budget,
        occupancy_threshold_ctas=best.occupancy_threshold_ctas, candidates=tuple(candidates),
        recommended_mode=best.mode, recommended_seed_tile_tokens=best.seed_tile_tokens,
        decision="seed_only_native_candidate", recommended_num_ctas=best.cta_count, predicted_us=best.predicted_us)


def seed_shape_from_policy(policy, *, batch: Optional[int] = None, dtype_bytes: int = 2) -> SeedKernelShape:
    """Shape record of a seed-only policy-like object (``batch`` overrides the policy's own)."""

    if batch is None:
        batch = getattr(policy, "batch", None)
    if batch is None:
        batch = getattr(policy, "min_batch")
    return SeedKernelShape(
        batch=int(batch), q_heads=int(getattr(policy, "heads")), kv_heads=int(getattr(policy, "kv_heads")),
        kv_len=int(getattr(policy, "kv_len_bucket")), dim=int(getattr(policy, "dim")),
        block_size=int(getattr(policy, "block_size")), sink_blocks=int(getattr(policy, "sink_blocks")),
        recent_blocks=int(getattr(policy, "recent_blocks")),
        middle_seed_blocks=int(getattr(policy, "middle_seed_blocks")), dtype_bytes=int(dtype_bytes))


__all__ = ["SeedKernelAutotuneResult", "SeedKernelCandidate", "SeedKernelShape", "autotune_seed_kernel_mode",
           "predicted_seed_decode_us", "seed_kernel_candidates", "seed_shape_from_policy"]
