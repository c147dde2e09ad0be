"""Seeded input builders shared by the golden-vector generator and the tests.

Inputs are always drawn on the CPU in float32 from ``torch.Generator`` with a
fixed seed and only then cast, so the oracle, the reference and the CUDA path
all see identical bits.  Nothing here touches the reference.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    return g


@dataclass(frozen=True)
class ExactCase:
    name: str
    seed: int
    batch: int
    q_heads: int
    kv_heads: int
    dim: int
    kv_len: int


EXACT_CASES: Dict[str, ExactCase] = {
    c.name: c
    for c in [
        # BASELINE config 1: the reference's own CPU-runnable case.
        ExactCase("c1_b2_h16_kv2_d64_n4096", 0, 2, 16, 2, 64, 4096),
        ExactCase("g8_d64_n300", 1, 2, 16, 2, 64, 300),
        ExactCase("g4_d128_n257", 2, 1, 32, 8, 128, 257),
        ExactCase("g1_d64_n64", 3, 3, 4, 4, 64, 64),
        ExactCase("g2_d8_n32", 4, 2, 4, 2, 8, 32),
        ExactCase("g7_d64_n1000", 5, 2, 14, 2, 64, 1000),
        ExactCase("g16_d32_n129", 6, 1, 16, 1, 32, 129),
    ]
}


def exact_inputs(case: ExactCase) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """q [B,1,Hq,D], k/v [B,N,Hkv,D] float32 N(0,1)."""

    g = _gen(case.seed)
    q = torch.randn(case.batch, 1, case.q_heads, case.dim, generator=g)
    k = torch.randn(case.batch, case.kv_len, case.kv_heads, case.dim, generator=g)
    v = torch.randn(case.batch, case.kv_len, case.kv_heads, case.dim, generator=g)
    return q, k, v


@dataclass(frozen=True)
class PagedCase:
    name: str
    seed: int
    batch: int
    q_heads: int
    kv_heads: int
    dim: int
    page_size: int
    max_pages: int
    min_len: int
    max_len: int
    extra_pages: int = 0


PAGED_CASES: Dict[str, PagedCase] = {
    c.name: c
    for c in [
        PagedCase("p16_g8_d64", 17, 3, 16, 2, 64, 16, 24, 100, 384),
        PagedCase("p64_g8_d64", 18, 2, 16, 2, 64, 64, 6, 65, 384),
        PagedCase("p16_g4_d128", 19, 2, 32, 8, 128, 16, 10, 1, 160, 3),
        PagedCase("p4_g2_d8", 20, 2, 4, 2, 8, 4, 5, 1, 20, 2),
        PagedCase("p32_g7_d64", 21, 2, 14, 2, 64, 32, 9, 33, 288),
        PagedCase("p128_g8_d64", 22, 2, 16, 2, 64, 128, 3, 130, 384),
    ]
}


def paged_inputs(case: PagedCase, *, layout: str = "HND"):
    """Page pool (random physical order), page table with -1 tails, ragged lengths.

    Mirrors how the reference's paged profiler lays a cache out
    (``benchmarks/profile_paged_exact_decode.py:191-235``): the pool has exactly
    the pages the table can name (plus ``extra_pages`` spare ones), the table is
    a random permutation of physical pages, and slots past a row's last active
    page are -1.
    """

    g = _gen(case.seed)
    num_pages = case.batch * case.max_pages + case.extra_pages
    q = torch.randn(case.batch, 1, case.q_heads, case.dim, generator=g)
    k_nhd = torch.randn(num_pages, case.page_size, case.kv_heads, case.dim, generator=g)
    v_nhd = torch.randn(num_pages, case.page_size, case.kv_heads, case.dim, generator=g)
    perm = torch.randperm(num_pages, generator=g)[: case.batch * case.max_pages]
    table = perm.to(torch.int32).view(case.batch, case.max_pages).clone()
    lengths = torch.randint(case.min_len, case.max_len + 1, (case.batch,), generator=g).to(torch.int32)
    lengths[0] = case.max_len  # one row always fills its table
    for b in range(case.batch):
        active = -(-int(lengths[b]) // case.page_size)
        table[b, active:] = -1
    if layout.upper() == "HND":
        k = k_nhd.permute(0, 2, 1, 3).contiguous()
        v = v_nhd.permute(0, 2, 1, 3).contiguous()
    else:
        k, v = k_nhd, v_nhd
    return q, k, v, table, lengths


def reference_paged_fixture(*, layout: str = "NHD"):
    """The reference's own paged fixture (tests/test_paged_decode.py:25-52)."""

    torch.manual_seed(17)
    q = torch.randn(2, 1, 4, 8)
    k_nhd = torch.randn(5, 4, 2, 8)
    v_nhd = torch.randn_like(k_nhd)
    table = torch.tensor([[3, 0, -1], [1, 4, 2]], dtype=torch.int32)
    lengths = torch.tensor([7, 10], dtype=torch.int32)
    if layout.upper() == "HND":
        return q, k_nhd.permute(0, 2, 1, 3).contiguous(), v_nhd.permute(0, 2, 1, 3).contiguous(), table, lengths
    return q, k_nhd, v_nhd, table, lengths


@dataclass(frozen=True)
class SeedCase:
    name: str
    seed: int
    batch: int
    q_heads: int
    kv_heads: int
    dim: int
    kv_len: int
    block_size: int
    sink_blocks: int
    recent_blocks: int
    middle_seed_blocks: int
    block_order: str


SEED_CASES: Dict[str, SeedCase] = {
    c.name: c
    for c in [
        SeedCase("s_bs32_d128", 30, 2, 16, 2, 128, 1000, 32, 2, 2, 8, "recent_first"),
        SeedCase("s_bs16_d64", 31, 2, 14, 2, 64, 777, 16, 1, 3, 4, "sequential"),
        SeedCase("s_bs8_d8", 32, 2, 4, 2, 8, 100, 8, 1, 1, 2, "sink_recent_first"),
        SeedCase("s_bs64_d64", 33, 1, 16, 2, 64, 2048, 64, 1, 1, 2, "recent_first"),
    ]
}

# Run-time seed selection (one KV head per query head, so the reference's per-head selection and
# the per-(row, KV head) selection of the kernels coincide): reuses SeedCase with q_heads == kv_heads.
SELECT_CASES: Dict[str, SeedCase] = {
    c.name: c
    for c in [
        SeedCase("sel_bs32_d128", 40, 2, 3, 3, 128, 1000, 32, 2, 2, 8, "recent_first"),
        SeedCase("sel_bs16_d64", 41, 1, 4, 4, 64, 777, 16, 1, 3, 4, "sequential"),
        SeedCase("sel_bs8_d64_short", 42, 2, 2, 2, 64, 50, 8, 1, 1, 3, "recent_first"),
    ]
}
SELECTORS = ("qk_block_max", "block_mean_proxy")


def select_inputs(case: SeedCase):
    """q, k rounded to bf16 (returned as float32) so CPU reference and GPU kernels see the same values."""

    g = _gen(case.seed)
    q = torch.randn(case.batch, 1, case.q_heads, case.dim, generator=g).bfloat16().float()
    k = torch.randn(case.batch, case.kv_len, case.kv_heads, case.dim, generator=g).bfloat16().float()
    return q, k


# Parameter grid for the integer seed-set goldens:
# (seq_len, block_size, sink, recent, middle, order)
SEED_INDEX_GRID: List[Tuple[int, int, int, int, int, str]] = [
    (320, 32, 1, 1, 2, "recent_first"),       # reference test vector
    (320, 32, 1, 1, 2, "sequential"),
    (32768, 32, 2, 2, 8, "recent_first"),     # packaged 3B schedule at 32K
    (32768, 32, 2, 3, 8, "recent_first"),
    (32768, 32, 2, 6, 12, "recent_first"),
    (32768, 16, 4, 16, 4, "sequential"),
    (1000, 32, 2, 2, 8, "recent_first"),      # ragged last block
    (100, 32, 2, 2, 8, "recent_first"),       # overlapping sink/recent/middle
    (100, 32, 2, 2, 8, "sequential"),
    (33, 32, 1, 1, 1, "sink_recent_first"),
    (10, 4, 1, 1, 0, "sequential"),
    (1, 32, 2, 2, 8, "recent_first"),
    (777, 16, 1, 3, 4, "sequential"),
    (2048, 64, 1, 1, 2, "recent_first"),
    (65536, 32, 2, 2, 8, "sink_recent_first"),
]


def seed_inputs(case: SeedCase):
    g = _gen(case.seed)
    q = torch.randn(case.batch, 1, case.q_heads, case.dim, generator=g)
    k = torch.randn(case.batch, case.kv_len, case.kv_heads, case.dim, generator=g)
    v = torch.randn(case.batch, case.kv_len, case.kv_heads, case.dim, generator=g)
    return q, k, v


def tensor_checksum(t: torch.Tensor) -> float:
    """Order-sensitive float64 checksum used to detect generator drift."""

    flat = t.detach().to(torch.float64).reshape(-1)
    weights = torch.arange(1, flat.numel() + 1, dtype=torch.float64) % 251 + 1.0
    return float((flat * weights).sum())


# ---- KV-cache update (rotary embedding + append) --------------------------------------------

@dataclass(frozen=True)
class RopeAppendCase:
    batch: int
    q_heads: int
    kv_heads: int
    dim: int
    max_seq: int
    positions: Tuple[int, ...]   # one entry (shared) or one per row
    shared_cos: bool
    dtype: str                   # "bf16" | "fp16" | "fp32"
    seed: int


ROPE_APPEND_CASES: Dict[str, RopeAppendCase] = {
    "qwen_bf16_shared_pos": RopeAppendCase(4, 16, 2, 128, 96, (37,), False, "bf16", 11),
    "qwen_fp16_shared_cos": RopeAppendCase(2, 8, 2, 64, 64, (63,), True, "fp16", 12),
    "rows_bf16_d64": RopeAppendCase(3, 8, 4, 64, 80, (0, 41, 79), False, "bf16", 13),
    "rows_fp32_d32": RopeAppendCase(2, 4, 4, 32, 40, (5, 17), True, "fp32", 14),
}

ROPE_DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def rope_append_inputs(case: RopeAppendCase):
    """(q_raw [B,Hq,1,D], k_raw, v_raw [B,Hkv,1,D], cos, sin [B or 1,1,D], k_cache, v_cache [B,Hkv,N,D]).

    Same recipe as the reference's parity script (scaled randn, angles ~ N(0,1) duplicated over
    the two halves), generated on the CPU in float32 and cast to the case's dtype.
    """

    g = _gen(case.seed)
    dtype = ROPE_DTYPES[case.dtype]
    scale = 1.0 / (case.dim ** 0.5)
    q_raw = (torch.randn(case.batch, case.q_heads, 1, case.dim, generator=g) * scale).to(dtype)
    k_raw = (torch.randn(case.batch, case.kv_heads, 1, case.dim, generator=g) * scale).to(dtype)
    v_raw = torch.randn(case.batch, case.kv_heads, 1, case.dim, generator=g).to(dtype)
    k_cache = (torch.randn(case.batch, case.kv_heads, case.max_seq, case.dim, generator=g) * scale).to(dtype)
    v_cache = torch.randn(case.batch, case.kv_heads, case.max_seq, case.dim, generator=g).to(dtype)
    angles = torch.randn(1 if case.shared_cos else case.batch, 1, case.dim // 2, generator=g)
    emb = torch.cat((angles, angles), dim=-1)
    return q_raw, k_raw, v_raw, emb.cos().to(dtype), emb.sin().to(dtype), k_cache, v_cache
