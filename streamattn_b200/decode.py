"""Decode routing, policies and fixed-buffer runners (host side of the hot path).

Mirrors the decode surface of the reference's ``stream_attention/decode.py``:
the public modes and their aliases, the seed-only policy cells and their
mismatch reasons, the serving telemetry record, the direct runners, the planned
``dense`` vs ``gate0_seed_only_batched`` decision and the fail-closed service.
Names, argument meaning, reason strings and error messages follow the
reference so callers and tests read the same; what executes is different:

* every launch goes to the sm_100a kernels behind ``streamattn_b200.native``;
* there is no Triton, no SDPA and no CPU execution path - running on non-CUDA
  tensors raises unless the caller injected its own ``dense_fallback``;
* the Gate-1 / fused-hybrid research routes of the reference are not part of
  this package; their arguments are accepted only as ``None``.
"""

from __future__ import annotations

import json
import math
import re
from dataclasses import asdict, dataclass, fields
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Union

import torch

from . import native
from .seed_selectors import policy_seed_blocks

DenseFallbackFn = Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor]

STREAMATTN_EXACT_NATIVE_BACKEND = "streamattn_exact_native"
STREAMATTN_MODE_EXACT_NATIVE = "exact_native"
STREAMATTN_MODE_SEED_ONLY_NATIVE = "seed_only_native"
STREAMATTN_MODE_VERIFIED_AUTO = "verified_auto"
STREAMATTN_NATIVE_MODES = frozenset(
    {STREAMATTN_MODE_EXACT_NATIVE, STREAMATTN_MODE_SEED_ONLY_NATIVE, STREAMATTN_MODE_VERIFIED_AUTO}
)
DEFAULT_GATE0_SEED_ONLY_BATCHED_POLICY = "qwen25_05b_l8_32k_seed_only_batched"
SEED_ONLY_BACKEND = "gate0_seed_only_batched"
_CELLS_FILE = Path(__file__).resolve().parent / "policies" / "seed_only_cells.json"
_MODE_ALIASES = {"auto": STREAMATTN_MODE_VERIFIED_AUTO, "dense": STREAMATTN_MODE_EXACT_NATIVE}


def normalize_stream_attn_mode(mode: str) -> str:
    """Public mode names plus the retained aliases (reference decode.py:53-64)."""

    text = str(mode)
    text = _MODE_ALIASES.get(text, text)
    if text not in STREAMATTN_NATIVE_MODES:
        raise ValueError("mode must be one of: " + ", ".join(sorted(STREAMATTN_NATIVE_MODES)))
    return text


def seq_bucket(seq_len: int) -> int:
    """Power-of-two bucket of a sequence length (reference telemetry.py:17-22)."""

    if seq_len <= 0:
        raise ValueError("seq_len must be positive")
    return 1 << (int(seq_len) - 1).bit_length()


def normalize_device_class(device_name: str) -> str:
    """Stable device class from a CUDA display name (reference router.py:14-29)."""

    raw = (device_name or "").lower()
    for needle, label in (("b200", "sm100_b200"), ("sm100", "sm100_b200"), ("h100", "sm90_h100"),
                          ("sm90", "sm90_h100"), ("a100", "sm80_a100"), ("sm80", "sm80_a100")):
        if needle in raw:
            return label
    if raw in {"cpu", "mps"}:
        return raw
    return re.sub(r"[^a-z0-9]+", "_", raw).strip("_") or "unknown"


_DTYPE_ALIASES = {
    "float16": "fp16", "half": "fp16", "fp16": "fp16",
    "bfloat16": "bf16", "bf16": "bf16",
    "float32": "fp32", "fp32": "fp32",
}


def _normalize_dtype_name(dtype: Union[str, torch.dtype, None]) -> Optional[str]:
    if dtype is None:
        return None
    name = str(dtype).lower().replace("torch.", "")
    return _DTYPE_ALIASES.get(name, name)


# --------------------------------------------------------------------------
# Packaged policy cells
# --------------------------------------------------------------------------

def packaged_gate0_seed_only_batched_policy_registry() -> Dict[str, Any]:
    """Registry of the packaged seed-only cells (metadata only)."""

    payload = json.loads(_CELLS_FILE.read_text(encoding="utf-8"))
    return {
        "schema": payload.get("schema"),
        "default": payload.get("default", DEFAULT_GATE0_SEED_ONLY_BATCHED_POLICY),
        "policies": [dict(cell["registry"]) for cell in payload.get("cells", [])],
    }


def _packaged_cells() -> Dict[str, Dict[str, Any]]:
    payload = json.loads(_CELLS_FILE.read_text(encoding="utf-8"))
    by_name: Dict[str, Dict[str, Any]] = {}
    for cell in payload.get("cells", []):
        meta = cell["registry"]
        for name in (meta.get("name"), meta.get("policy_id"), *(meta.get("aliases") or [])):
            if name:
                by_name[str(name)] = cell
    return by_name


def list_packaged_gate0_seed_only_batched_policies(*, include_aliases: bool = False) -> List[str]:
    """Canonical cell names; with ``include_aliases`` also policy ids and aliases."""

    names: List[str] = []
    for meta in packaged_gate0_seed_only_batched_policy_registry()["policies"]:
        group = [meta.get("name")]
        if include_aliases:
            group += [meta.get("policy_id"), *(meta.get("aliases") or [])]
        for name in group:
            if name and str(name) not in names:
                names.append(str(name))
    return names


def find_packaged_gate0_seed_only_batched_policies(
    *,
    model_id: Optional[str] = None,
    layer_id: Optional[int] = None,
    dtype: Optional[str] = None,
    kv_len_bucket: Optional[int] = None,
    min_batch: Optional[int] = None,
    status: Optional[str] = "green",
) -> List[str]:
    """Metadata-only search of the packaged cells (reference decode.py:153-189)."""

    want_dtype = _normalize_dtype_name(dtype) if dtype is not None else None
    found: List[str] = []
    for meta in packaged_gate0_seed_only_batched_policy_registry()["policies"]:
        checks = (
            status is None or meta.get("status") == status,
            model_id is None or meta.get("model_id") == model_id,
            layer_id is None or int(meta.get("layer_id", -1)) == int(layer_id),
            want_dtype is None or _normalize_dtype_name(meta.get("dtype")) == want_dtype,
            kv_len_bucket is None or int(meta.get("kv_len_bucket", -1)) == int(kv_len_bucket),
            min_batch is None or int(meta.get("min_batch", 0)) <= int(min_batch),
        )
        name = meta.get("name")
        if all(checks) and name and str(name) not in found:
            found.append(str(name))
    return found


@dataclass(frozen=True)
class StreamAttnDecodePolicy:
    """Thresholds of the planned decode route (reference decode.py:253-293).

    Only ``safety_margin``, ``collect_telemetry_every``,
    ``allow_gate0_seed_only_batched`` and ``min_kv_len_for_gate0_seed_only`` act
    here; the other fields are kept so existing configurations still construct.
    """

    max_router_regret_pct: float = 0.05
    safety_margin: float = 1.10
    allow_mass: bool = True
    allow_value_bound: bool = True
    prefer_value_bound_if_within: float = 1.10
    collect_telemetry_every: int = 16
    min_kv_len_for_gate1: int = 4096
    max_active_fraction_mass: float = 0.35
    max_active_fraction_value_bound: float = 0.30
    min_confidence: float = 0.70
    require_metadata_for_value_bound: bool = True
    allow_gate0_fused_hybrid: bool = True
    min_kv_len_for_gate0: int = 16384
    allow_gate0_seed_only_batched: bool = True
    min_kv_len_for_gate0_seed_only: int = 16384

    def __post_init__(self) -> None:
        if self.max_router_regret_pct < 0.0:
            raise ValueError("max_router_regret_pct must be non-negative")
        if self.safety_margin < 1.0:
            raise ValueError("safety_margin must be >= 1")
        if self.prefer_value_bound_if_within < 1.0:
            raise ValueError("prefer_value_bound_if_within must be >= 1")
        if self.collect_telemetry_every < 0:
            raise ValueError("collect_telemetry_every must be non-negative")
        for name in ("min_kv_len_for_gate1", "min_kv_len_for_gate0", "min_kv_len_for_gate0_seed_only"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive")
        for name in ("max_active_fraction_mass", "max_active_fraction_value_bound", "min_confidence"):
            if not 0.0 <= getattr(self, name) <= 1.0:
                raise ValueError(f"{name} must be in [0, 1]")


def _truthy(*values: Any) -> Any:
    """First value that is truthy (``a or b or c`` chains of the policy format)."""

    for value in values:
        if value:
            return value
    return None


def _present(*values: Any) -> Any:
    """First value that is not None."""

    for value in values:
        if value is not None:
            return value
    return None


def _opt(kind, value):
    return None if value is None else kind(value)


_BLOCK_ORDERS = ("sequential", "recent_first", "sink_recent_first")


@dataclass(frozen=True)
class Gate0SeedOnlyBatchedPolicy:
    """One verified seed-only cell: where it applies and which seed set it reads.

    Field names, defaults and validation follow reference decode.py:319-388; the
    ``num_warps`` / ``num_stages`` fields are launch hints of the reference's
    Triton kernel and are ignored by the sm_100a kernel.
    """

    mode: str = "all_seed_only"
    model_id: str = "unknown"
    layer_id: int = -1
    policy_id: str = ""
    tensor_space: str = "post_rope"
    dtype: Optional[str] = None
    kv_len_bucket: Optional[int] = None
    min_batch: int = 4
    heads: Optional[int] = None
    kv_heads: Optional[int] = None
    dim: Optional[int] = None
    block_size: int = 32
    sink_blocks: int = 2
    recent_blocks: int = 2
    middle_seed_blocks: int = 8
    block_order: str = "recent_first"
    num_warps: int = 4
    num_stages: int = 2
    safety_gate: str = "distribution_aware"
    top1_must_match: bool = True
    min_topk_overlap: int = 4
    max_kl: Optional[float] = None
    max_logit_delta: Optional[float] = None
    max_logprob_delta: Optional[float] = None
    expected_seed_only_ms: Optional[float] = None
    expected_dense_ms: Optional[float] = None
    expected_speedup_vs_dense: Optional[float] = None
    expected_max_abs_error: Optional[float] = None
    fallback: str = "dense"

    def __post_init__(self) -> None:
        if self.mode != "all_seed_only":
            raise ValueError("Gate0SeedOnlyBatchedPolicy only supports all_seed_only mode")
        if self.tensor_space != "post_rope":
            raise ValueError("Gate0 seed-only policy currently requires post_rope tensors")
        if self.min_batch <= 0:
            raise ValueError("min_batch must be positive")
        if self.block_size <= 0:
            raise ValueError("block_size must be positive")
        if min(self.sink_blocks, self.recent_blocks, self.middle_seed_blocks) < 0:
            raise ValueError("seed block counts must be non-negative")
        if self.block_order not in _BLOCK_ORDERS:
            raise ValueError("block_order must be sequential, recent_first, or sink_recent_first")
        if self.num_warps <= 0 or self.num_stages <= 0:
            raise ValueError("num_warps and num_stages must be positive")
        if self.min_topk_overlap < 0:
            raise ValueError("min_topk_overlap must be non-negative")
        for name in ("max_kl", "max_logit_delta", "max_logprob_delta", "expected_max_abs_error"):
            value = getattr(self, name)
            if value is not None and value < 0.0:
                raise ValueError(f"{name} must be non-negative")
        for name in ("expected_seed_only_ms", "expected_dense_ms", "expected_speedup_vs_dense"):
            value = getattr(self, name)
            if value is not None and value <= 0.0:
                raise ValueError(f"{name} must be positive")

    @classmethod
    def from_entry(cls, entry: Dict[str, Any]) -> "Gate0SeedOnlyBatchedPolicy":
        """Parse one policy artifact entry (format of reference decode.py:390-512)."""

        runtime = dict(_truthy(entry.get("runtime"), entry.get("seed_config")) or {})
        safety = dict(entry.get("safety") or {})
        quality = dict(entry.get("quality") or {})
        timing = dict(_truthy(entry.get("timing"), quality) or {})
        shape = dict(entry.get("shape") or {})
        capture = dict(entry.get("capture") or {})
        seed_error = dict(quality.get("seed_vs_flashinfer_exact") or {})
        return cls(
            mode=str(_truthy(entry.get("mode"), runtime.get("mode"), "all_seed_only")),
            model_id=str(_truthy(entry.get("model_id"), entry.get("model"), "unknown")),
            layer_id=int(_present(entry.get("layer_id"), capture.get("layer_id"), -1)),
            policy_id=str(_truthy(entry.get("policy_id"), entry.get("id"), "")),
            tensor_space=str(_truthy(entry.get("tensor_space"), runtime.get("tensor_space"), "post_rope")),
            dtype=_normalize_dtype_name(_truthy(entry.get("dtype"), shape.get("dtype"), runtime.get("dtype"))),
            kv_len_bucket=_opt(int, _present(entry.get("kv_len_bucket"), shape.get("kv_len_bucket"),
                                             shape.get("kv_len"))),
            min_batch=int(_truthy(entry.get("min_batch"), runtime.get("min_batch"), shape.get("batch"), 4)),
            heads=_opt(int, _present(entry.get("heads"), shape.get("heads"), shape.get("q_heads"))),
            kv_heads=_opt(int, _present(entry.get("kv_heads"), shape.get("kv_heads"),
                                        shape.get("true_kv_heads"))),
            dim=_opt(int, _present(entry.get("dim"), shape.get("dim"))),
            block_size=int(_truthy(runtime.get("block_size"), 32)),
            sink_blocks=int(_truthy(runtime.get("sink_blocks"), 2)),
            recent_blocks=int(_truthy(runtime.get("recent_blocks"), 2)),
            middle_seed_blocks=int(_truthy(runtime.get("middle_seed_blocks"), 8)),
            block_order=str(_truthy(runtime.get("block_order"), "recent_first")),
            num_warps=int(_truthy(runtime.get("num_warps"), 4)),
            num_stages=int(_truthy(runtime.get("num_stages"), 2)),
            safety_gate=str(_truthy(safety.get("gate"), safety.get("safety_gate"), "distribution_aware")),
            top1_must_match=bool(safety.get("top1_must_match", True)),
            min_topk_overlap=int(_truthy(safety.get("min_top5_overlap"), safety.get("min_topk_overlap"), 4)),
            max_kl=_opt(float, safety.get("max_kl")),
            max_logit_delta=_opt(float, safety.get("max_logit_delta")),
            max_logprob_delta=_opt(float, safety.get("max_logprob_delta")),
            expected_seed_only_ms=_opt(float, _present(timing.get("seed_only_ms"),
                                                       timing.get("streamattn_seed_only_ms"),
                                                       timing.get("seed_direct_full_prealloc_ms"))),
            expected_dense_ms=_opt(float, _present(timing.get("dense_ms"), timing.get("flashinfer_tc_ms"),
                                                   timing.get("flashinfer_batch_tc_exact_ms"))),
            expected_speedup_vs_dense=_opt(float, _present(timing.get("speedup_vs_dense"), timing.get("speedup"),
                                                           timing.get("speedup_vs_flashinfer_batch"))),
            expected_max_abs_error=_opt(float, _present(timing.get("max_abs_error"),
                                                        seed_error.get("max_abs_error"))),
            fallback=str(_truthy(entry.get("fallback"), "dense")),
        )

    @classmethod
    def from_json(cls, path: Union[str, Path], *, entry_index: int = 0) -> "Gate0SeedOnlyBatchedPolicy":
        """Load a policy artifact file in the reference's JSON format."""

        payload = json.loads(Path(path).read_text(encoding="utf-8"))
        entries = _truthy(payload.get("stable_entries"), payload.get("entries"))
        return cls.from_entry(entries[entry_index] if entries else payload)

    @classmethod
    def from_packaged(cls, name: str = DEFAULT_GATE0_SEED_ONLY_BATCHED_POLICY, *,
                      entry_index: int = 0) -> "Gate0SeedOnlyBatchedPolicy":
        """Load a packaged cell by canonical name, policy id or alias."""

        cells = _packaged_cells()
        if name not in cells:
            known = ", ".join(sorted(cells))
            raise ValueError(f"unknown packaged Gate-0 seed-only policy {name!r}; known: {known}")
        if entry_index != 0:
            raise IndexError("packaged cells hold exactly one entry")
        known_fields = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in cells[name]["policy"].items() if k in known_fields})

    def mismatch_reasons(
        self,
        query: torch.Tensor,
        key: torch.Tensor,
        *,
        min_kv_len: int = 1,
        model_id: Optional[str] = None,
        layer_id: Optional[int] = None,
        backend_available: bool = True,
    ) -> List[str]:
        """Why this policy refuses the call (empty list = it applies).

        The reason names and their order are the reference's (decode.py:548-593): callers log
        and compare these lists.  Two tables: checks on the call's identity, then - only for
        4-D tensors - checks on its shape; a check is a (name, refuses?) pair.
        """

        identity = (
            ("model_mismatch", model_id is not None and model_id != self.model_id),
            ("layer_mismatch", layer_id is not None and int(layer_id) != self.layer_id),
            ("backend_unavailable", not backend_available),
            ("shape_mismatch", query.dim() != 4 or key.dim() != 4),
        )
        reasons = [name for name, refuses in identity if refuses]
        if reasons and reasons[-1] == "shape_mismatch":
            return reasons  # nothing below can be read off tensors of another rank
        batch, query_len, heads, dim = map(int, query.shape)
        key_batch, kv_len, kv_heads, key_dim = map(int, key.shape)
        dtype_wanted = _normalize_dtype_name(self.dtype)

        def pinned_differs(pinned, actual) -> bool:
            return pinned is not None and pinned != actual

        shape = (
            ("shape_mismatch", batch != key_batch or dim != key_dim),
            ("query_len_mismatch", query_len != 1),
            ("batch_below_min", batch < self.min_batch),
            ("kv_len_below_min", kv_len < min_kv_len),
            ("kv_len_bucket_mismatch",
             self.kv_len_bucket is not None and seq_bucket(kv_len) != seq_bucket(int(self.kv_len_bucket))),
            ("dtype_mismatch", pinned_differs(dtype_wanted, _normalize_dtype_name(query.dtype))),
            ("gqa_shape_mismatch", kv_heads <= 0 or heads % kv_heads != 0),
            ("heads_mismatch", pinned_differs(self.heads, heads)),
            ("kv_heads_mismatch", pinned_differs(self.kv_heads, kv_heads)),
            ("head_dim_mismatch", pinned_differs(self.dim, dim)),
        )
        return reasons + [name for name, refuses in shape if refuses]

    def matches_tensors(self, query: torch.Tensor, key: torch.Tensor, **kwargs) -> bool:
        return not self.mismatch_reasons(query, key, **kwargs)

    def seed_blocks(self, kv_len: int) -> List[int]:
        """Seed blocks this policy reads for a cache of ``kv_len`` tokens."""

        return policy_seed_blocks(
            seq_len=int(kv_len), block_size=self.block_size, sink_blocks=self.sink_blocks,
            recent_blocks=self.recent_blocks, middle_seed_blocks=self.middle_seed_blocks,
            block_order=self.block_order,
        )


def load_packaged_gate0_seed_only_batched_policy(
    name: str = DEFAULT_GATE0_SEED_ONLY_BATCHED_POLICY, *, entry_index: int = 0
) -> Gate0SeedOnlyBatchedPolicy:
    return Gate0SeedOnlyBatchedPolicy.from_packaged(name, entry_index=entry_index)


# --------------------------------------------------------------------------
# Telemetry records
# --------------------------------------------------------------------------

@dataclass(frozen=True)
class Gate0SeedOnlyBatchedStats:
    batch_size: int
    heads: int
    kv_heads: int
    kv_len: int
    block_size: int
    seed_blocks: int
    total_blocks: int

    @property
    def seed_fraction(self) -> float:
        return self.seed_blocks / self.total_blocks if self.total_blocks > 0 else 0.0


@dataclass(frozen=True)
class Gate0SeedOnlyBatchedRunInfo:
    policy: Gate0SeedOnlyBatchedPolicy
    stats: Optional[Gate0SeedOnlyBatchedStats]
    backend_used: str
    fallback_reason: Optional[str] = None


@dataclass(frozen=True)
class StreamAttnServingInfo:
    """Per-call telemetry, field for field as reference decode.py:650-673."""

    backend_used: str
    policy_id: Optional[str]
    fallback_reason: Optional[str]
    batch_size: int
    kv_len: int
    layer_id: Optional[int]
    model_id: Optional[str]
    dtype: str
    device: str
    plan_backend: str
    plan_reason: str
    seed_only_enabled: bool
    safety_policy_matched: bool
    runtime_counters: Dict[str, Dict[str, int]]
    stats: Optional[Dict[str, object]] = None

    def to_dict(self) -> Dict[str, object]:
        return asdict(self)


def _seed_stats(policy: Gate0SeedOnlyBatchedPolicy, query: torch.Tensor,
                key_cache: torch.Tensor) -> Gate0SeedOnlyBatchedStats:
    kv_len = int(key_cache.shape[1])
    total = -(-kv_len // policy.block_size)
    wanted = policy.sink_blocks + policy.recent_blocks + policy.middle_seed_blocks
    return Gate0SeedOnlyBatchedStats(
        batch_size=int(query.shape[0]), heads=int(query.shape[2]), kv_heads=int(key_cache.shape[2]),
        kv_len=kv_len, block_size=int(policy.block_size), seed_blocks=min(wanted, total), total_blocks=total,
    )


# --------------------------------------------------------------------------
# Backend availability and layout inference
# --------------------------------------------------------------------------

# (q_heads, kv_heads, head_dim) -> (batch, kv_len) cells the reference treats as
# head-major [B, Hkv, N, D] buffers purely from their shape
# (backends/sm90/transposed_gqa_exact.py:33-82 and :198-244).  Only the keys
# matter here: they keep layout inference identical for existing callers.
HEAD_MAJOR_CELLS = {
    (16, 2, 64): {(2, 16384), (4, 16384), (4, 32768), (4, 65536), (8, 16384), (8, 32768), (8, 65536)},
    (16, 4, 64): {(b, n) for b in (1, 2, 4, 8, 16) for n in (16384, 32768, 65536)} - {(1, 65536)},
    (32, 8, 128): {(4, 32768), (4, 65536), (8, 16384), (8, 65536), (16, 32768), (16, 65536)},
}


def infer_kv_layout(query: torch.Tensor, key_cache: torch.Tensor) -> str:
    """``"BHND"`` when the reference would read the cache as head-major, else ``"BNHD"``.

    The public contract is BNHD ``[B, N, Hkv, D]``.  The reference recognises its
    head-major fast-path buffers from the shape alone: reading the cache shape as
    ``(B, Hkv, N, D)`` must give a promoted (heads, batch, length) cell with
    bf16 contiguous tensors.  The same rule is applied here so that buffers laid
    out for the reference keep their meaning.
    """

    if query.dim() != 4 or key_cache.dim() != 4 or query.shape[1] != 1:
        return "BNHD"
    batch, _, q_heads, dim = (int(x) for x in query.shape)
    kv_batch, kv_heads, kv_len, kv_dim = (int(x) for x in key_cache.shape)
    cells = HEAD_MAJOR_CELLS.get((q_heads, kv_heads, dim))
    if (cells is None or (batch, kv_len) not in cells or batch != kv_batch or dim != kv_dim
            or query.dtype != torch.bfloat16 or key_cache.dtype != torch.bfloat16
            or not query.is_contiguous() or not key_cache.is_contiguous()):
        return "BNHD"
    return "BHND"


def _exact_native_supported(query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor) -> bool:
    """Whether the sm_100a exact kernels can serve these buffers."""

    tensors = (query, key_cache, value_cache)
    if not all(t.is_cuda for t in tensors):
        return False
    if any(t.dim() != 4 for t in tensors) or query.shape[1] != 1 or key_cache.shape != value_cache.shape:
        return False
    if query.shape[0] != key_cache.shape[0] or query.shape[3] != key_cache.shape[3]:
        return False
    if len({t.dtype for t in tensors}) != 1 or query.dtype not in native.SA_DTYPE:
        return False
    if not 0 < int(query.shape[3]) <= 256:
        return False
    layout = infer_kv_layout(query, key_cache)
    kv_heads = int(key_cache.shape[1] if layout == "BHND" else key_cache.shape[2])
    if kv_heads <= 0 or int(query.shape[2]) % kv_heads:
        return False
    return native.device_supported(query.device)


# --------------------------------------------------------------------------
# Fixed-buffer runners
# --------------------------------------------------------------------------

class _BoundRunner:
    """Shared bookkeeping of the direct runners: bound tensors and their identity."""

    def __init__(self, query, key_cache, value_cache, output, info) -> None:
        self.query = query
        self.key_cache = key_cache
        self.value_cache = value_cache
        self.output = output
        self.info = info
        self.query_shape = tuple(query.shape)
        self.key_shape = tuple(key_cache.shape)
        self.value_shape = tuple(value_cache.shape)
        self.query_stride = tuple(query.stride())
        self.key_stride = tuple(key_cache.stride())
        self.value_stride = tuple(value_cache.stride())
        self.query_data_ptr = int(query.data_ptr())
        self.key_data_ptr = int(key_cache.data_ptr())
        self.value_data_ptr = int(value_cache.data_ptr())


class StreamAttnSeedOnlyDirectRunner(_BoundRunner):
    """One seed-only launch into a reused output buffer (reference decode.py:704-782).

    The seed block list is fixed at construction from the policy and the cache
    length; ``run()`` neither allocates nor synchronises.
    """

    def __init__(self, *, policy: Gate0SeedOnlyBatchedPolicy, query: torch.Tensor,
                 key_cache: torch.Tensor, value_cache: torch.Tensor, output: torch.Tensor,
                 info: StreamAttnServingInfo, kernel: str = "auto") -> None:
        super().__init__(query, key_cache, value_cache, output, info)
        self.policy = policy
        kv_len, kv_heads = int(key_cache.shape[1]), int(key_cache.shape[2])
        self.seed_blocks = policy.seed_blocks(kv_len)
        batch, _, q_heads, dim = (int(x) for x in query.shape)
        # Grid of the launch: CTAs per (row, KV head) pair from the latency model of the kernel
        # (few seed tokens: one CTA per pair and no merge; many: the pair is split).
        from .seed_autotune import SeedKernelShape, autotune_seed_kernel_mode

        shape = SeedKernelShape(batch=batch, q_heads=q_heads, kv_heads=kv_heads, kv_len=kv_len, dim=dim,
                                block_size=policy.block_size, sink_blocks=len(self.seed_blocks),
                                recent_blocks=0, middle_seed_blocks=0, dtype_bytes=query.element_size())
        self.grid = autotune_seed_kernel_mode(shape, sm_count=native.sm_count(query.device))
        num_ctas = self.grid.recommended_num_ctas if query.is_cuda else 0
        self.workspace = native.new_workspace(query.device, batch, q_heads, kv_heads, dim, num_ctas)
        self._plan = native.seed_plan(query, key_cache, value_cache, output, self.workspace,
                                      block_size=policy.block_size, blocks=self.seed_blocks,
                                      kv_layout="BNHD", num_ctas=num_ctas, kernel=kernel)
        self.backend_variant = self._plan.kernel_name

    def run(self) -> torch.Tensor:
        self._plan.run()
        return self.output

    def run_with_info(self):
        return self.run(), self.info


class StreamAttnExactNativeDirectRunner(_BoundRunner):
    """Exact M=1 GQA decode bound to stable buffers (reference decode.py:785-878)."""

    def __init__(self, *, query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                 output: torch.Tensor, info: Optional[StreamAttnServingInfo],
                 kv_layout: Optional[str] = None, num_ctas: int = 0, kernel: str = "auto") -> None:
        if output.shape != query.shape or not output.is_contiguous():
            raise ValueError("exact-native output must be contiguous and match query shape")
        super().__init__(query, key_cache, value_cache, output, info)
        if not _exact_native_supported(query, key_cache, value_cache):
            raise ValueError("no exact-native runner supports these buffers")
        self.kv_layout = kv_layout or infer_kv_layout(query, key_cache)
        batch, _, q_heads, dim = (int(x) for x in query.shape)
        kv_heads = int(key_cache.shape[1] if self.kv_layout == "BHND" else key_cache.shape[2])
        self.workspace = native.new_workspace(query.device, batch, q_heads, kv_heads, dim, num_ctas)
        self._plan = native.exact_plan(query, key_cache, value_cache, output, self.workspace,
                                       kv_layout=self.kv_layout, num_ctas=num_ctas, kernel=kernel)
        self.backend_variant = self._plan.kernel_name

    def run(self) -> torch.Tensor:
        self._plan.run()
        return self.output

    def run_with_info(self):
        if self.info is None:
            raise RuntimeError("exact-native runner was planned without serving info")
        return self.run(), self.info


def stream_attn_exact_native_decode(query: torch.Tensor, key_cache: torch.Tensor,
                                    value_cache: torch.Tensor) -> torch.Tensor:
    """One-shot exact decode on the sm_100a kernels (reference decode.py:192-215).

    The reference falls back to a dense PyTorch path for CPU or unsupported
    buffers; this package has no such path and raises instead.
    """

    if not _exact_native_supported(query, key_cache, value_cache):
        native.require_cuda(query, key_cache, value_cache)
        raise ValueError("exact-native decode does not support these buffers")
    output = torch.empty_like(query)
    return StreamAttnExactNativeDirectRunner(
        query=query, key_cache=key_cache, value_cache=value_cache, output=output, info=None
    ).run()


# --------------------------------------------------------------------------
# Planned route: dense vs gate0_seed_only_batched
# --------------------------------------------------------------------------

@dataclass(frozen=True)
class DecodeCostKey:
    """Lookup key of the decode cost table (reference decode.py:881-933)."""

    device_class: str
    dtype: str
    query_len: int
    kv_bucket: int
    heads: int
    kv_heads: int
    dim: int
    attention_type: str
    block_size: int
    tile_size_q: int
    num_warps: int
    num_stages: int
    causal: bool = False

    @classmethod
    def from_tensors(cls, query: torch.Tensor, key: torch.Tensor, *, kv_heads: Optional[int] = None,
                     attention_type: str = "mha", block_size: int, tile_size_q: int, num_warps: int,
                     num_stages: int, causal: bool = False) -> "DecodeCostKey":
        if query.dim() != 4 or key.dim() != 4:
            raise ValueError("query and key must have shape [batch, seq, heads, dim]")
        if query.is_cuda:
            device_class = normalize_device_class(torch.cuda.get_device_name(query.device))
        else:
            device_class = normalize_device_class(query.device.type)
        return cls(
            device_class=device_class,
            dtype=str(query.dtype).replace("torch.", ""),
            query_len=int(query.shape[1]),
            kv_bucket=seq_bucket(int(key.shape[1])),
            heads=int(query.shape[2]),
            kv_heads=int(kv_heads if kv_heads is not None else key.shape[2]),
            dim=int(query.shape[3]),
            attention_type=attention_type,
            block_size=block_size,
            tile_size_q=tile_size_q,
            num_warps=num_warps,
            num_stages=num_stages,
            causal=causal,
        )


@dataclass(frozen=True)
class DecodeCostEntry:
    """Measured costs of one key.  Only ``dense_ms`` feeds the routes of this
    package; the remaining fields keep cost files written for the reference
    (decode.py:936-1059) loadable."""

    dense_ms: float
    qk_scan_ms: float = 1.0e-9
    gate1_mass_ms_at_calibration: float = 1.0e-9
    calibration_active_fraction: float = 1.0
    gate1_dense_equiv_ms: Optional[float] = None
    gate1_value_bound_ms_at_calibration: Optional[float] = None
    predicate_overhead_ms: float = 0.0
    metadata_update_ms: float = 0.0
    metadata_build_ms: Optional[float] = None
    measured_router_regret_pct: Optional[float] = None
    sample_count: int = 1
    last_updated: Optional[str] = None

    def __post_init__(self) -> None:
        if self.dense_ms <= 0.0:
            raise ValueError("dense_ms must be positive")
        if self.qk_scan_ms <= 0.0:
            raise ValueError("qk_scan_ms must be positive")
        if self.gate1_mass_ms_at_calibration <= 0.0:
            raise ValueError("gate1_mass_ms_at_calibration must be positive")
        if not 0.0 <= self.calibration_active_fraction <= 1.0:
            raise ValueError("calibration_active_fraction must be in [0, 1]")
        if self.sample_count < 0:
            raise ValueError("sample_count must be non-negative")


class DecodeCostModel:
    """Cost table with the reference's JSON round trip (decode.py:1062-1100)."""

    def __init__(self) -> None:
        self._entries: Dict[DecodeCostKey, DecodeCostEntry] = {}

    def update(self, key: DecodeCostKey, entry: DecodeCostEntry) -> None:
        self._entries[key] = entry

    def lookup(self, key: DecodeCostKey) -> Optional[DecodeCostEntry]:
        return self._entries.get(key)

    def to_dict(self) -> Dict[str, object]:
        return {"version": 1,
                "entries": [{"key": asdict(k), "entry": asdict(e)} for k, e in self._entries.items()]}

    @classmethod
    def from_dict(cls, payload: Dict[str, object]) -> "DecodeCostModel":
        model = cls()
        for item in payload.get("entries", []):
            model.update(DecodeCostKey(**dict(item["key"])), DecodeCostEntry(**dict(item["entry"])))
        return model

    def to_json(self, path: Union[str, Path]) -> None:
        Path(path).write_text(json.dumps(self.to_dict(), indent=2, sort_keys=True), encoding="utf-8")

    @classmethod
    def from_json(cls, path: Union[str, Path]) -> "DecodeCostModel":
        return cls.from_dict(json.loads(Path(path).read_text(encoding="utf-8")))


@dataclass
class StreamAttnDecodeWorkspace:
    """Reusable output buffer and step counter of the planned route
    (reference decode.py:1103-1241, without the Gate-1 scratch tensors)."""

    device: torch.device
    max_batch: int
    max_query_len: int
    max_kv_len: int
    max_heads: int
    head_dim: int
    block_size: int
    output: Optional[torch.Tensor] = None
    step_index: int = 0

    @classmethod
    def allocate(cls, *, device: Union[str, torch.device], max_batch: int, max_query_len: int,
                 max_kv_len: int, max_heads: int, head_dim: int, block_size: int,
                 dtype: torch.dtype = torch.float16) -> "StreamAttnDecodeWorkspace":
        device = torch.device(device)
        if device.type == "cuda" and device.index is None and torch.cuda.is_available():
            device = torch.device("cuda", torch.cuda.current_device())
        limits = dict(max_batch=max_batch, max_query_len=max_query_len, max_kv_len=max_kv_len,
                      max_heads=max_heads, head_dim=head_dim, block_size=block_size)
        for name, value in limits.items():
            if int(value) <= 0:
                raise ValueError(f"{name} must be positive")
        return cls(device=device, **{k: int(v) for k, v in limits.items()},
                   output=torch.empty((max_batch, max_query_len, max_heads, head_dim), device=device, dtype=dtype))

    def validate(self, query: Optional[torch.Tensor] = None, key: Optional[torch.Tensor] = None,
                 value: Optional[torch.Tensor] = None, *, batch: Optional[int] = None,
                 query_len: Optional[int] = None, kv_len: Optional[int] = None, heads: Optional[int] = None,
                 head_dim: Optional[int] = None, device: Optional[Union[str, torch.device]] = None) -> None:
        if query is not None:
            if query.dim() != 4:
                raise ValueError("query must have shape [batch, seq, heads, dim]")
            batch, query_len, heads, head_dim = (int(x) for x in query.shape)
            device = query.device
        for name, tensor in (("key", key), ("value", value)):
            if tensor is None:
                continue
            if tensor.dim() != 4:
                raise ValueError(f"{name} must have shape [batch, seq, heads, dim]")
            if batch is not None and tensor.shape[0] != batch:
                raise ValueError(f"query/{name} batch must match")
            if head_dim is not None and tensor.shape[3] != head_dim:
                raise ValueError(f"query/{name} head dim must match")
            if name == "value" and kv_len is not None and tensor.shape[1] != kv_len:
                raise ValueError("key/value sequence length must match")
            kv_len = int(tensor.shape[1])
            heads = max(heads or 0, int(tensor.shape[2]))
            device = tensor.device if device is None else device
        for name, actual, limit in (("batch", batch, self.max_batch), ("query_len", query_len, self.max_query_len),
                                    ("kv_len", kv_len, self.max_kv_len), ("heads", heads, self.max_heads)):
            if actual is not None and int(actual) > limit:
                raise ValueError(f"{name} {actual} exceeds workspace limit {limit}")
        if head_dim is not None and int(head_dim) != self.head_dim:
            raise ValueError(f"head_dim {head_dim} does not match workspace {self.head_dim}")
        if device is not None and torch.device(device) != self.device:
            raise ValueError(f"device {torch.device(device)} does not match workspace {self.device}")

    def reset_step(self) -> None:
        self.step_index = 0

    def advance_step(self) -> int:
        self.step_index += 1
        return self.step_index


@dataclass(frozen=True)
class StreamAttnDecodePlan:
    """Decision record of ``stream_attn_decode_plan`` (reference decode.py:1364-1390)."""

    backend: str
    reason: str
    query_len: int
    kv_len: int
    heads: int
    kv_heads: int
    dim: int
    attention_type: str
    block_size: int
    tile_size_q: int
    num_warps: int
    num_stages: int
    metadata_required: bool
    metadata_update_required: bool
    predicted_active_fraction: float
    predicted_ms: float
    dense_ms: float
    expected_regret_ms: float
    collect_telemetry: bool
    skip_predicate: Optional[str] = None
    active_threshold: Optional[float] = None
    projection_metadata_required: bool = False
    gate0_fused_hybrid_policy: Optional[object] = None
    gate0_seed_only_batched_policy: Optional[Gate0SeedOnlyBatchedPolicy] = None
    fallback_reason: Optional[str] = None


def _reject_research_routes(**kwargs) -> None:
    used = [name for name, value in kwargs.items() if value is not None]
    if used:
        raise NotImplementedError(
            "the Gate-1 / fused-hybrid routes are not part of streamattn_b200: " + ", ".join(used)
        )


def stream_attn_decode_plan(
    query: torch.Tensor,
    key: torch.Tensor,
    *,
    metadata=None,
    gate0_fused_hybrid_policy=None,
    gate0_seed_only_batched_policy: Optional[Gate0SeedOnlyBatchedPolicy] = None,
    gate0_projection_metadata=None,
    router=None,
    decode_cost_model: Optional[DecodeCostModel] = None,
    policy: Optional[StreamAttnDecodePolicy] = None,
    active_fraction_hint: Optional[float] = None,
    attention_type: str = "mha",
    kv_heads: Optional[int] = None,
    block_size: int = 64,
    tile_size_q: int = 16,
    num_warps: int = 4,
    num_stages: int = 3,
    error_budget: float = 1.0e-3,
    step_index: int = 0,
) -> StreamAttnDecodePlan:
    """Choose ``dense`` or ``gate0_seed_only_batched`` for one decode call.

    Same decision as reference decode.py:1410-1669 restricted to these two
    candidates: the seed-only route wins when the policy matches the tensors and
    its expected speed-up over dense is at least ``policy.safety_margin``.
    """

    _reject_research_routes(metadata=metadata, gate0_fused_hybrid_policy=gate0_fused_hybrid_policy,
                            gate0_projection_metadata=gate0_projection_metadata, router=router)
    if query.dim() != 4 or key.dim() != 4:
        raise ValueError("query and key must have shape [batch, seq, heads, dim]")
    if query.shape[0] != key.shape[0] or query.shape[3] != key.shape[3]:
        raise ValueError("query/key batch and dim must match")
    kv_heads = int(key.shape[2] if kv_heads is None else kv_heads)
    policy = policy or StreamAttnDecodePolicy()
    active = 1.0 if active_fraction_hint is None else min(1.0, max(0.0, float(active_fraction_hint)))
    cost = None
    if decode_cost_model is not None:
        cost = decode_cost_model.lookup(DecodeCostKey.from_tensors(
            query, key, kv_heads=kv_heads, attention_type=attention_type, block_size=block_size,
            tile_size_q=tile_size_q, num_warps=num_warps, num_stages=num_stages))
    collect = policy.collect_telemetry_every > 0 and step_index % policy.collect_telemetry_every == 0
    seed_policy = gate0_seed_only_batched_policy
    dense_ms = cost.dense_ms if cost is not None else 0.0
    if dense_ms <= 0.0 and seed_policy is not None:
        dense_ms = float(seed_policy.expected_dense_ms or 0.0)

    seed_ms: Optional[float] = None
    fallback_reason: Optional[str] = None
    if seed_policy is not None and policy.allow_gate0_seed_only_batched:
        mismatches = seed_policy.mismatch_reasons(query, key, min_kv_len=policy.min_kv_len_for_gate0_seed_only)
        seed_ms = seed_policy.expected_seed_only_ms
        if seed_ms is None and seed_policy.expected_speedup_vs_dense and dense_ms > 0.0:
            seed_ms = dense_ms / float(seed_policy.expected_speedup_vs_dense)
        if seed_ms is not None and dense_ms > 0.0:
            speedup: Optional[float] = dense_ms / seed_ms
        else:
            speedup = seed_policy.expected_speedup_vs_dense
        if mismatches:
            fallback_reason = mismatches[0]
        elif seed_ms is None or seed_ms <= 0.0:
            fallback_reason = "missing_seed_only_batched_timing"
        elif dense_ms <= 0.0:
            fallback_reason = "missing_dense_timing"
        elif speedup is None or speedup < policy.safety_margin:
            fallback_reason = "seed_only_batched_not_profitable"
        if fallback_reason is not None:
            seed_ms = None

    common = dict(
        query_len=int(query.shape[1]), kv_len=int(key.shape[1]), heads=int(query.shape[2]), kv_heads=kv_heads,
        dim=int(query.shape[3]), attention_type=attention_type, block_size=block_size, tile_size_q=tile_size_q,
        num_warps=num_warps, num_stages=num_stages, metadata_required=False, metadata_update_required=False,
        predicted_active_fraction=active, collect_telemetry=collect,
    )
    if seed_ms is not None and seed_ms <= dense_ms:
        return StreamAttnDecodePlan(
            backend=SEED_ONLY_BACKEND, reason="calibrated_gate0_seed_only_batched_policy",
            predicted_ms=float(seed_ms), dense_ms=dense_ms, expected_regret_ms=0.0,
            gate0_seed_only_batched_policy=seed_policy, **common)
    if cost is None:
        return StreamAttnDecodePlan(
            backend="dense", reason="missing_decode_cost", predicted_ms=0.0, dense_ms=0.0,
            expected_regret_ms=0.0, fallback_reason=fallback_reason, **common)
    return StreamAttnDecodePlan(
        backend="dense", reason="dense_fallback", predicted_ms=dense_ms, dense_ms=dense_ms,
        expected_regret_ms=0.0, fallback_reason=fallback_reason, **common)


def _dense(query, key, value, dense_fallback: Optional[DenseFallbackFn]) -> torch.Tensor:
    if dense_fallback is not None:
        return dense_fallback(query, key, value)
    return stream_attn_exact_native_decode(query, key, value)


def stream_attn_decode_run(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *,
    plan: StreamAttnDecodePlan,
    metadata=None,
    gate0_projection_metadata=None,
    gate0_workspace=None,
    output_workspace: Optional[torch.Tensor] = None,
    dense_fallback: Optional[DenseFallbackFn] = None,
    dense_fallback_backend: str = "dense",
    build_gate0_metadata_if_missing: bool = True,
    error_budget: float = 1.0e-3,
    return_info: bool = False,
):
    """Execute a plan of :func:`stream_attn_decode_plan` (reference decode.py:1672-1807).

    ``dense`` means exact attention: the injected ``dense_fallback`` if given,
    else the sm_100a exact kernel.
    """

    if plan.backend == "dense":
        output = _dense(query, key, value, dense_fallback)
        return (output, None) if return_info else output
    if plan.backend != SEED_ONLY_BACKEND:
        raise ValueError(f"unknown decode backend: {plan.backend}")
    seed_policy = plan.gate0_seed_only_batched_policy
    if seed_policy is None:
        raise ValueError("gate0_seed_only_batched plan is missing its policy")

    def fail_closed(reason: str):
        output = _dense(query, key, value, dense_fallback)
        info = Gate0SeedOnlyBatchedRunInfo(policy=seed_policy, stats=None,
                                           backend_used=dense_fallback_backend, fallback_reason=reason)
        return (output, info) if return_info else output

    if not all(t.is_cuda for t in (query, key, value)):
        return fail_closed("seed_only_batched_requires_cuda")
    try:
        reusable = (output_workspace is not None and output_workspace.shape == query.shape
                    and output_workspace.device == query.device and output_workspace.dtype == query.dtype
                    and output_workspace.is_contiguous())
        output = output_workspace if reusable else torch.empty_like(query)
        StreamAttnSeedOnlyDirectRunner(policy=seed_policy, query=query, key_cache=key, value_cache=value,
                                       output=output, info=None).run()
    except Exception as exc:
        if seed_policy.fallback != "dense":
            raise
        return fail_closed(f"seed_only_batched_backend_error:{type(exc).__name__}")
    if not return_info:
        return output
    info = Gate0SeedOnlyBatchedRunInfo(policy=seed_policy, stats=_seed_stats(seed_policy, query, key),
                                       backend_used=SEED_ONLY_BACKEND, fallback_reason=None)
    return output, info


class StreamAttnDecodeWrapper:
    """Stateful plan-then-run wrapper with routing counters (reference decode.py:1816-2083)."""

    def __init__(self, workspace: StreamAttnDecodeWorkspace, *, policy: Optional[StreamAttnDecodePolicy] = None,
                 decode_cost_model: Optional[DecodeCostModel] = None, router=None,
                 gate0_fused_hybrid_policy=None,
                 gate0_seed_only_batched_policy: Optional[Gate0SeedOnlyBatchedPolicy] = None,
                 gate0_projection_metadata=None, dense_fallback: Optional[DenseFallbackFn] = None,
                 dense_fallback_backend: str = "dense") -> None:
        _reject_research_routes(router=router, gate0_fused_hybrid_policy=gate0_fused_hybrid_policy,
                                gate0_projection_metadata=gate0_projection_metadata)
        self.workspace = workspace
        self.policy = policy or StreamAttnDecodePolicy()
        self.decode_cost_model = decode_cost_model or DecodeCostModel()
        self.gate0_seed_only_batched_policy = gate0_seed_only_batched_policy
        self.dense_fallback = dense_fallback
        self.dense_fallback_backend = dense_fallback_backend
        self.last_active_fraction: Optional[float] = None
        self.last_plan: Optional[StreamAttnDecodePlan] = None
        self.last_info = None
        self._static: Optional[Dict[str, object]] = None
        self.backend_counts: Dict[str, int] = {}
        self.fallback_reasons: Dict[str, int] = {}

    def plan(self, *, query_shape, kv_shape, attention_type: str = "mha", kv_heads: Optional[int] = None,
             block_size: Optional[int] = None, tile_size_q: int = 16, num_warps: int = 4, num_stages: int = 3,
             error_budget: float = 1.0e-3) -> "StreamAttnDecodeWrapper":
        query_shape = tuple(query_shape.shape if isinstance(query_shape, torch.Tensor) else query_shape)
        kv_shape = tuple(kv_shape.shape if isinstance(kv_shape, torch.Tensor) else kv_shape)
        if len(query_shape) != 4 or len(kv_shape) != 4:
            raise ValueError("query_shape and kv_shape must be [batch, seq, heads, dim]")
        if query_shape[0] != kv_shape[0] or query_shape[3] != kv_shape[3]:
            raise ValueError("query/KV batch and dim must match")
        self.workspace.validate(batch=int(query_shape[0]), query_len=int(query_shape[1]), kv_len=int(kv_shape[1]),
                                heads=max(int(query_shape[2]), int(kv_shape[2])), head_dim=int(query_shape[3]),
                                device=self.workspace.device)
        self._static = dict(
            query_shape=query_shape, kv_shape=kv_shape, attention_type=attention_type,
            kv_heads=int(kv_shape[2] if kv_heads is None else kv_heads),
            block_size=int(block_size or self.workspace.block_size), tile_size_q=int(tile_size_q),
            num_warps=int(num_warps), num_stages=int(num_stages), error_budget=float(error_budget),
        )
        self.last_plan = None
        self.last_info = None
        self.last_active_fraction = None
        self.reset_runtime_counters()
        self.workspace.reset_step()
        return self

    def observe_active_fraction(self, active_fraction: float) -> None:
        self.last_active_fraction = min(1.0, max(0.0, float(active_fraction)))

    def reset_runtime_counters(self) -> None:
        self.backend_counts.clear()
        self.fallback_reasons.clear()

    def runtime_counters(self) -> Dict[str, Dict[str, int]]:
        return {"backend_counts": dict(self.backend_counts), "fallback_reasons": dict(self.fallback_reasons)}

    def _require_static(self) -> Dict[str, object]:
        if self._static is None:
            raise RuntimeError("call plan(...) before run(...)")
        return self._static

    def _check_tensors(self, query, key_cache, value_cache=None) -> None:
        static = self._require_static()
        if tuple(query.shape) != tuple(static["query_shape"]):
            raise ValueError("query shape does not match planned query_shape")
        if tuple(key_cache.shape) != tuple(static["kv_shape"]):
            raise ValueError("key_cache shape does not match planned kv_shape")
        if value_cache is not None and tuple(value_cache.shape) != tuple(static["kv_shape"]):
            raise ValueError("value_cache shape does not match planned kv_shape")
        if query.device != self.workspace.device or key_cache.device != self.workspace.device:
            raise ValueError("query/key device does not match workspace device")
        if value_cache is not None and value_cache.device != self.workspace.device:
            raise ValueError("value device does not match workspace device")

    def plan_step(self, query, key_cache, *, metadata=None, active_fraction_hint: Optional[float] = None,
                  _validated: bool = False) -> StreamAttnDecodePlan:
        static = self._require_static()
        if not _validated:
            self._check_tensors(query, key_cache)
        hint = self.last_active_fraction if active_fraction_hint is None else active_fraction_hint
        if (self.policy.collect_telemetry_every == 0 and self.last_plan is not None and hint is not None
                and abs(self.last_plan.predicted_active_fraction - float(hint)) <= 1.0e-12):
            return self.last_plan
        self.last_plan = stream_attn_decode_plan(
            query, key_cache, metadata=metadata,
            gate0_seed_only_batched_policy=self.gate0_seed_only_batched_policy,
            decode_cost_model=self.decode_cost_model, policy=self.policy, active_fraction_hint=hint,
            attention_type=str(static["attention_type"]), kv_heads=int(static["kv_heads"]),
            block_size=int(static["block_size"]), tile_size_q=int(static["tile_size_q"]),
            num_warps=int(static["num_warps"]), num_stages=int(static["num_stages"]),
            error_budget=float(static["error_budget"]), step_index=self.workspace.step_index,
        )
        return self.last_plan

    def _record(self, plan: StreamAttnDecodePlan, info) -> None:
        backend = getattr(info, "backend_used", None)
        reason = getattr(info, "fallback_reason", None)
        if reason is None and plan.backend == "dense":
            reason = plan.fallback_reason
        if backend is None:
            injected = plan.backend == "dense" and self.dense_fallback is not None
            backend = self.dense_fallback_backend if injected else plan.backend
        self.backend_counts[str(backend)] = self.backend_counts.get(str(backend), 0) + 1
        if reason:
            self.fallback_reasons[str(reason)] = self.fallback_reasons.get(str(reason), 0) + 1

    def run(self, query, key_cache, value_cache, *, metadata=None, active_fraction_hint: Optional[float] = None,
            return_info: bool = False):
        static = self._require_static()
        self._check_tensors(query, key_cache, value_cache)
        plan = self.plan_step(query, key_cache, metadata=metadata, active_fraction_hint=active_fraction_hint,
                              _validated=True)
        wants_info = return_info or (plan.backend != "dense"
                                     and (plan.collect_telemetry or self.last_active_fraction is None))
        result = stream_attn_decode_run(
            query, key_cache, value_cache, plan=plan, output_workspace=self.workspace.output,
            dense_fallback=self.dense_fallback, dense_fallback_backend=self.dense_fallback_backend,
            error_budget=float(static["error_budget"]), return_info=wants_info,
        )
        output, info = result if wants_info else (result, None)
        self.last_info = info
        self._record(plan, info)
        stats = getattr(info, "stats", None)
        if stats is not None and hasattr(stats, "seed_fraction"):
            self.last_active_fraction = float(stats.seed_fraction)
        self.workspace.advance_step()
        return (output, info) if return_info else output


# --------------------------------------------------------------------------
# Fail-closed serving service
# --------------------------------------------------------------------------

class StreamAttnSeedOnlyDecodeService:
    """One verified seed-only policy with fail-closed exact fallback
    (reference decode.py:2086-2660)."""

    def __init__(self, *, policy: Optional[Gate0SeedOnlyBatchedPolicy] = None,
                 policy_name: str = DEFAULT_GATE0_SEED_ONLY_BATCHED_POLICY,
                 decode_policy: Optional[StreamAttnDecodePolicy] = None,
                 dense_fallback: Optional[DenseFallbackFn] = None,
                 dense_fallback_backend: str = STREAMATTN_EXACT_NATIVE_BACKEND,
                 model_id: Optional[str] = None, layer_id: Optional[int] = None,
                 use_planned_direct_seed_only_path: bool = True,
                 use_direct_seed_only_path: bool = False) -> None:
        self.policy = policy or load_packaged_gate0_seed_only_batched_policy(policy_name)
        self.decode_policy = decode_policy or StreamAttnDecodePolicy(collect_telemetry_every=0)
        self.dense_fallback = dense_fallback
        self.dense_fallback_backend = dense_fallback_backend
        self.model_id = model_id if model_id is not None else self.policy.model_id
        self.layer_id = layer_id if layer_id is not None else self.policy.layer_id
        self.use_planned_direct_seed_only_path = bool(use_planned_direct_seed_only_path)
        self.use_direct_seed_only_path = bool(use_direct_seed_only_path)
        self.workspace: Optional[StreamAttnDecodeWorkspace] = None
        self.wrapper: Optional[StreamAttnDecodeWrapper] = None
        self.output_workspace: Optional[torch.Tensor] = None
        self.direct_runner: Optional[StreamAttnSeedOnlyDirectRunner] = None
        self._direct_runner_key: Optional[tuple] = None
        self._planned_shape: Optional[tuple] = None

    @classmethod
    def from_packaged(cls, name: str = DEFAULT_GATE0_SEED_ONLY_BATCHED_POLICY,
                      **kwargs) -> "StreamAttnSeedOnlyDecodeService":
        return cls(policy=load_packaged_gate0_seed_only_batched_policy(name), **kwargs)

    # -- helpers ---------------------------------------------------------

    def _ids(self, model_id, layer_id):
        return (model_id if model_id is not None else self.model_id,
                layer_id if layer_id is not None else self.layer_id)

    @staticmethod
    def _check_ranks(query, key_cache, value_cache) -> None:
        if query.dim() != 4 or key_cache.dim() != 4 or value_cache.dim() != 4:
            raise ValueError("query, key_cache, and value_cache must be [batch, seq, heads, dim]")
        if key_cache.shape != value_cache.shape:
            raise ValueError("key_cache and value_cache shapes must match")
        if query.shape[0] != key_cache.shape[0] or query.shape[3] != key_cache.shape[3]:
            raise ValueError("query/KV batch and head_dim must match")

    def _policy_reasons(self, query, key_cache, model_id, layer_id) -> List[str]:
        return self.policy.mismatch_reasons(
            query, key_cache, min_kv_len=self.decode_policy.min_kv_len_for_gate0_seed_only,
            model_id=model_id, layer_id=layer_id)

    def _preflight_reasons(self, query, key_cache, *, model_id, layer_id, mode: str) -> List[str]:
        if normalize_stream_attn_mode(mode) == STREAMATTN_MODE_EXACT_NATIVE:
            return ["manual_dense" if mode == "dense" else "manual_exact_native"]
        reasons = self._policy_reasons(query, key_cache, model_id, layer_id)
        if reasons:
            return reasons
        if not (query.is_cuda and key_cache.is_cuda) or not native.device_supported(query.device):
            return ["backend_unavailable"]
        return []

    def _dense_output(self, query, key_cache, value_cache) -> torch.Tensor:
        return _dense(query, key_cache, value_cache, self.dense_fallback)

    def _allocate_output_workspace(self, query: torch.Tensor) -> torch.Tensor:
        ws = self.output_workspace
        if (ws is None or ws.shape != query.shape or ws.device != query.device or ws.dtype != query.dtype
                or not ws.is_contiguous()):
            self.output_workspace = torch.empty_like(query)
        return self.output_workspace

    def _serving_info(self, *, query, key_cache, model_id, layer_id, backend_used: str,
                      fallback_reason: Optional[str], plan_backend: str, plan_reason: str,
                      safety_policy_matched: bool, runtime_counters=None, stats=None) -> StreamAttnServingInfo:
        if runtime_counters is None:
            runtime_counters = {
                "backend_counts": {backend_used: 1},
                "fallback_reasons": {fallback_reason: 1} if fallback_reason is not None else {},
            }
        return StreamAttnServingInfo(
            backend_used=backend_used, policy_id=self.policy.policy_id, fallback_reason=fallback_reason,
            batch_size=int(query.shape[0]), kv_len=int(key_cache.shape[1]), layer_id=layer_id, model_id=model_id,
            dtype=_normalize_dtype_name(query.dtype) or str(query.dtype), device=str(query.device),
            plan_backend=plan_backend, plan_reason=plan_reason,
            seed_only_enabled=backend_used == SEED_ONLY_BACKEND, safety_policy_matched=safety_policy_matched,
            runtime_counters=runtime_counters, stats=asdict(stats) if stats is not None else None,
        )

    def _fallback_info(self, query, key_cache, model_id, layer_id, reason, matched) -> StreamAttnServingInfo:
        return self._serving_info(query=query, key_cache=key_cache, model_id=model_id, layer_id=layer_id,
                                  backend_used=self.dense_fallback_backend, fallback_reason=reason,
                                  plan_backend="dense", plan_reason=reason, safety_policy_matched=matched)

    # -- planning --------------------------------------------------------

    def plan_direct_seed_only(self, query, key_cache, value_cache, *, model_id: Optional[str] = None,
                              layer_id: Optional[int] = None, mode: str = "auto") -> StreamAttnSeedOnlyDirectRunner:
        """Validate once and bind a seed-only runner; any mismatch raises ValueError."""

        self._check_ranks(query, key_cache, value_cache)
        model_id, layer_id = self._ids(model_id, layer_id)
        reasons = self._preflight_reasons(query, key_cache, model_id=model_id, layer_id=layer_id, mode=mode)
        if reasons:
            raise ValueError(f"cannot plan direct seed-only route: {','.join(reasons)}")
        if not (query.is_contiguous() and key_cache.is_contiguous() and value_cache.is_contiguous()):
            raise ValueError("cannot plan direct seed-only route: layout_mismatch")
        info = self._serving_info(
            query=query, key_cache=key_cache, model_id=model_id, layer_id=layer_id,
            backend_used=SEED_ONLY_BACKEND, fallback_reason=None, plan_backend=SEED_ONLY_BACKEND,
            plan_reason="planned_direct_seed_only", safety_policy_matched=True,
            runtime_counters={"backend_counts": {SEED_ONLY_BACKEND: 1}, "fallback_reasons": {}},
            stats=_seed_stats(self.policy, query, key_cache),
        )
        return StreamAttnSeedOnlyDirectRunner(policy=self.policy, query=query, key_cache=key_cache,
                                              value_cache=value_cache,
                                              output=self._allocate_output_workspace(query), info=info)

    def plan_exact_native(self, query, key_cache, value_cache, *, model_id: Optional[str] = None,
                          layer_id: Optional[int] = None) -> StreamAttnExactNativeDirectRunner:
        """Bind an exact runner; raises ValueError when the sm_100a backend cannot serve the buffers."""

        if not _exact_native_supported(query, key_cache, value_cache):
            raise ValueError("cannot plan exact-native route: backend_unavailable")
        if not (query.is_contiguous() and key_cache.is_contiguous() and value_cache.is_contiguous()):
            raise ValueError("cannot plan exact-native route: layout_mismatch")
        model_id, layer_id = self._ids(model_id, layer_id)
        info = self._serving_info(
            query=query, key_cache=key_cache, model_id=model_id, layer_id=layer_id,
            backend_used=STREAMATTN_EXACT_NATIVE_BACKEND, fallback_reason=None,
            plan_backend=STREAMATTN_EXACT_NATIVE_BACKEND, plan_reason="planned_exact_native",
            safety_policy_matched=False,
        )
        return StreamAttnExactNativeDirectRunner(query=query, key_cache=key_cache, value_cache=value_cache,
                                                 output=self._allocate_output_workspace(query), info=info)

    def _runner_key(self, query, key_cache, value_cache, model_id, layer_id) -> tuple:
        def ident(t):
            return (tuple(t.shape), tuple(t.stride()), str(t.device), t.dtype, int(t.data_ptr()))
        return (self.policy.policy_id, model_id, layer_id, ident(query), ident(key_cache), ident(value_cache))

    def _direct_runner_matches(self, query, key_cache, value_cache, *, model_id, layer_id) -> bool:
        runner = self.direct_runner
        if runner is None:
            return False
        if query is not runner.query or key_cache is not runner.key_cache or value_cache is not runner.value_cache:
            return False
        return self._direct_runner_key == self._runner_key(query, key_cache, value_cache, model_id, layer_id)

    def _allocate_direct_runner(self, query, key_cache, value_cache, *, model_id, layer_id, mode):
        key = self._runner_key(query, key_cache, value_cache, model_id, layer_id)
        if self.direct_runner is None or self._direct_runner_key != key:
            self.direct_runner = self.plan_direct_seed_only(query, key_cache, value_cache, model_id=model_id,
                                                            layer_id=layer_id, mode=mode)
            self._direct_runner_key = key
        return self.direct_runner

    def _allocate_wrapper(self, query, key_cache, value_cache) -> StreamAttnDecodeWrapper:
        shape_key = (tuple(query.shape), tuple(key_cache.shape), tuple(value_cache.shape))
        if self.wrapper is None or self._planned_shape != shape_key:
            self.workspace = StreamAttnDecodeWorkspace.allocate(
                device=query.device, max_batch=query.shape[0], max_query_len=query.shape[1],
                max_kv_len=key_cache.shape[1], max_heads=max(query.shape[2], key_cache.shape[2]),
                head_dim=query.shape[3], block_size=self.policy.block_size, dtype=query.dtype)
            self.wrapper = StreamAttnDecodeWrapper(
                self.workspace, policy=self.decode_policy, gate0_seed_only_batched_policy=self.policy,
                dense_fallback=self.dense_fallback, dense_fallback_backend=self.dense_fallback_backend)
            self.wrapper.plan(query_shape=query.shape, kv_shape=key_cache.shape,
                              block_size=self.policy.block_size, tile_size_q=16,
                              num_warps=self.policy.num_warps, num_stages=self.policy.num_stages)
            self._planned_shape = shape_key
        return self.wrapper

    # -- execution -------------------------------------------------------

    def run(self, query, key_cache, value_cache, *, model_id: Optional[str] = None,
            layer_id: Optional[int] = None, mode: str = "auto",
            active_fraction_hint: Optional[float] = 1.0, return_info: bool = True):
        """One decode call through a public mode; any mismatch runs exact and says why."""

        model_id, layer_id = self._ids(model_id, layer_id)
        normalized = normalize_stream_attn_mode(mode)
        seed_modes = {STREAMATTN_MODE_VERIFIED_AUTO, STREAMATTN_MODE_SEED_ONLY_NATIVE}
        planned_direct = self.use_planned_direct_seed_only_path and not self.use_direct_seed_only_path
        if (normalized in seed_modes and planned_direct
                and self._direct_runner_matches(query, key_cache, value_cache, model_id=model_id, layer_id=layer_id)):
            runner = self.direct_runner
            return runner.run_with_info() if return_info else runner.run()

        self._check_ranks(query, key_cache, value_cache)
        policy_reasons = self._policy_reasons(query, key_cache, model_id, layer_id)
        reasons = self._preflight_reasons(query, key_cache, model_id=model_id, layer_id=layer_id, mode=mode)
        if reasons:
            output = self._dense_output(query, key_cache, value_cache)
            info = self._fallback_info(query, key_cache, model_id, layer_id, reasons[0], not policy_reasons)
            return (output, info) if return_info else output

        if planned_direct or self.use_direct_seed_only_path:
            try:
                runner = self._allocate_direct_runner(query, key_cache, value_cache, model_id=model_id,
                                                      layer_id=layer_id, mode=normalized)
                return runner.run_with_info() if return_info else runner.run()
            except Exception as exc:
                if self.policy.fallback != "dense":
                    raise
                reason = f"seed_only_batched_backend_error:{type(exc).__name__}"
                output = self._dense_output(query, key_cache, value_cache)
                if not return_info:
                    return output
                return output, self._fallback_info(query, key_cache, model_id, layer_id, reason, True)

        wrapper = self._allocate_wrapper(query, key_cache, value_cache)
        output, run_info = wrapper.run(query, key_cache, value_cache, active_fraction_hint=active_fraction_hint,
                                       return_info=True)
        plan = wrapper.last_plan
        backend = getattr(run_info, "backend_used", None) or plan.backend
        fallback_reason = getattr(run_info, "fallback_reason", None) or plan.fallback_reason
        info = self._serving_info(
            query=query, key_cache=key_cache, model_id=model_id, layer_id=layer_id, backend_used=str(backend),
            fallback_reason=fallback_reason, plan_backend=plan.backend, plan_reason=plan.reason,
            safety_policy_matched=True, runtime_counters=wrapper.runtime_counters(),
            stats=getattr(run_info, "stats", None),
        )
        return (output, info) if return_info else output


def stream_attn_seed_only_decode(query, key_cache, value_cache, *,
                                 policy: Optional[Gate0SeedOnlyBatchedPolicy] = None,
                                 policy_name: str = DEFAULT_GATE0_SEED_ONLY_BATCHED_POLICY,
                                 decode_policy: Optional[StreamAttnDecodePolicy] = None,
                                 dense_fallback: Optional[DenseFallbackFn] = None,
                                 dense_fallback_backend: str = STREAMATTN_EXACT_NATIVE_BACKEND,
                                 model_id: Optional[str] = None, layer_id: Optional[int] = None,
                                 use_planned_direct_seed_only_path: bool = True,
                                 use_direct_seed_only_path: bool = False, mode: str = "auto",
                                 active_fraction_hint: Optional[float] = 1.0, return_info: bool = True):
    """One-shot policy-aware decode (reference decode.py:2663-2703)."""

    service = StreamAttnSeedOnlyDecodeService(
        policy=policy, policy_name=policy_name, decode_policy=decode_policy, dense_fallback=dense_fallback,
        dense_fallback_backend=dense_fallback_backend, model_id=model_id, layer_id=layer_id,
        use_planned_direct_seed_only_path=use_planned_direct_seed_only_path,
        use_direct_seed_only_path=use_direct_seed_only_path,
    )
    return service.run(query, key_cache, value_cache, model_id=model_id, layer_id=layer_id, mode=mode,
                       active_fraction_hint=active_fraction_hint, return_info=return_info)
