"""Fixed-buffer decode engine: resolve a route once, then launch without replanning.

Public surface (names, arguments and defaults) follows the reference's
``stream_attention/engine.py:37-323``: ``StreamAttnEngine.plan(q, k, v, mode=...)``
returns a ``StreamAttnEnginePlan`` bound to the caller's buffers, ``.run()``
launches it, ``StreamAttnEngine.decode`` / ``stream_attn_decode`` do both.

Internally a call is handled in two steps.  ``_resolve_route`` turns (mode,
cache kind, policy check) into a small ``_Route`` record - which kernel family
serves the call and why - and ``_bind`` attaches the matching bound runner.
Routes:

========================  =====================================================
``exact_native``          exact GQA decode (contiguous or paged cache)
``seed_only_native``      seed-only decode; planning errors propagate
``verified_auto``         seed-only when the packaged policy verifies the call,
                          otherwise exact with the refusal reasons recorded
========================  =====================================================
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Union

import torch

from .decode import (
    STREAMATTN_EXACT_NATIVE_BACKEND,
    STREAMATTN_MODE_EXACT_NATIVE,
    STREAMATTN_MODE_SEED_ONLY_NATIVE,
    STREAMATTN_MODE_VERIFIED_AUTO,
    DenseFallbackFn,
    Gate0SeedOnlyBatchedPolicy,
    StreamAttnDecodePolicy,
    StreamAttnExactNativeDirectRunner,
    StreamAttnSeedOnlyDecodeService,
    StreamAttnSeedOnlyDirectRunner,
    StreamAttnServingInfo,
    normalize_stream_attn_mode,
)
from .paged import PagedExactDecodePlan, PagedExactDecodeRunner, PagedKVCache

_Runner = Union[StreamAttnSeedOnlyDirectRunner, StreamAttnExactNativeDirectRunner, PagedExactDecodeRunner]

_PAGED_REASON = {
    STREAMATTN_MODE_EXACT_NATIVE: "explicit_paged_exact_native",
    STREAMATTN_MODE_VERIFIED_AUTO: "paged_kv_exact_only",
}


@dataclass(frozen=True)
class _Route:
    """Outcome of route resolution: the kernel family, the recorded reason, the runner (if bound)."""

    backend: str
    reason: str
    runner: Optional[_Runner]


@dataclass(frozen=True)
class StreamAttnEnginePlan:
    """Result of :meth:`StreamAttnEngine.plan`: a route plus the buffers it was bound to."""

    mode: str
    backend: str
    reason: str
    model_id: Optional[str]
    layer_id: Optional[int]
    query: torch.Tensor
    key_cache: Union[torch.Tensor, PagedKVCache]
    value_cache: Optional[torch.Tensor]
    service: StreamAttnSeedOnlyDecodeService
    direct_runner: Optional[_Runner] = None

    @property
    def uses_fixed_buffers(self) -> bool:
        """True when a bound runner exists, i.e. ``run()`` is a single attribute hop to a launch."""

        return self.direct_runner is not None

    def run(self, *, return_info: bool = True):
        """Launch on the bound buffers; returns ``(output, info)`` or just ``output``."""

        if self.direct_runner is not None:
            call = self.direct_runner.run_with_info if return_info else self.direct_runner.run
            return call()
        # Nothing could be bound (the kernels do not take these buffers).  The service then
        # computes exact attention through the dense_fallback the caller injected, or raises:
        # this package has no CPU execution path of its own.
        if not isinstance(self.key_cache, torch.Tensor) or self.value_cache is None:
            raise RuntimeError("non-native plan is missing contiguous KV tensors")
        return self.service.run(self.query, self.key_cache, self.value_cache, model_id=self.model_id,
                                layer_id=self.layer_id, mode=STREAMATTN_MODE_EXACT_NATIVE,
                                return_info=return_info)


def _paged_serving_info(query: torch.Tensor, cache: PagedKVCache, plan: PagedExactDecodePlan,
                        reason: str) -> StreamAttnServingInfo:
    """Telemetry record of a paged exact plan (fields as the reference fills them, engine.py:119-160)."""

    stats: Dict[str, Any] = {"layout": cache.normalized_layout, "page_size": cache.page_size}
    stats["max_pages_per_request"] = cache.max_pages_per_request
    stats["splits"] = plan.splits
    stats["workspace_bytes"] = plan.workspace_bytes
    counters = {"backend_counts": {plan.backend: 1}, "fallback_reasons": {}}
    return StreamAttnServingInfo(
        backend_used=plan.backend, plan_backend=plan.backend, plan_reason=reason,
        policy_id=None, fallback_reason=None, model_id=None, layer_id=None,
        batch_size=int(query.shape[0]), kv_len=int(cache.sequence_lengths.max().item()),
        dtype=str(query.dtype).removeprefix("torch."), device=str(query.device),
        seed_only_enabled=False, safety_policy_matched=False,
        runtime_counters=counters, stats=stats)


class StreamAttnEngine:
    """Plans and runs the native decode modes over caller-owned buffers."""

    def __init__(self, *, policy: Optional[Gate0SeedOnlyBatchedPolicy] = None,
                 policy_name: str = "qwen25_05b_l8_32k_seed_only_batched",
                 decode_policy: Optional[StreamAttnDecodePolicy] = None,
                 dense_fallback: Optional[DenseFallbackFn] = None,
                 dense_fallback_backend: str = STREAMATTN_EXACT_NATIVE_BACKEND,
                 model_id: Optional[str] = None, layer_id: Optional[int] = None) -> None:
        self.service = StreamAttnSeedOnlyDecodeService(
            policy=policy, policy_name=policy_name, decode_policy=decode_policy, dense_fallback=dense_fallback,
            dense_fallback_backend=dense_fallback_backend, model_id=model_id, layer_id=layer_id,
            use_planned_direct_seed_only_path=True)

    # -- route resolution ------------------------------------------------------------------

    def _exact_route(self, reason: str, query, key_cache, value_cache, ids: Dict[str, Any]) -> _Route:
        """Exact decode; when the buffers cannot be bound the route stays, without a runner."""

        try:
            runner = self.service.plan_exact_native(query, key_cache, value_cache, **ids)
        except ValueError:
            runner = None
        return _Route(STREAMATTN_EXACT_NATIVE_BACKEND, reason, runner)

    def _paged_route(self, mode: str, query: torch.Tensor, cache: PagedKVCache) -> _Route:
        if mode not in _PAGED_REASON:
            raise ValueError("seed_only_native does not yet support paged KV; use exact_native or verified_auto")
        plan = PagedExactDecodePlan.build(query, cache)
        reason = _PAGED_REASON[mode]
        info = _paged_serving_info(query, cache, plan, reason)
        return _Route(plan.backend, reason, PagedExactDecodeRunner(plan=plan, info=info))

    def _resolve_route(self, mode: str, query, key_cache, value_cache, ids: Dict[str, Any]) -> _Route:
        if mode == STREAMATTN_MODE_EXACT_NATIVE:
            return self._exact_route("explicit_exact_native", query, key_cache, value_cache, ids)
        try:
            runner = self.service.plan_direct_seed_only(query, key_cache, value_cache, mode=mode, **ids)
        except ValueError as refusal:
            if mode == STREAMATTN_MODE_SEED_ONLY_NATIVE:
                raise  # the caller asked for seed-only and nothing else
            # verified_auto fails closed: exact decode, with the policy's refusal as the reason
            return self._exact_route(str(refusal), query, key_cache, value_cache, ids)
        return _Route(STREAMATTN_MODE_SEED_ONLY_NATIVE, "verified_policy_match", runner)

    # -- public API ------------------------------------------------------------------------

    def plan(self, query: torch.Tensor, key_cache: Union[torch.Tensor, PagedKVCache],
             value_cache: Optional[torch.Tensor] = None, *, mode: str = STREAMATTN_MODE_VERIFIED_AUTO,
             model_id: Optional[str] = None, layer_id: Optional[int] = None) -> StreamAttnEnginePlan:
        """Check the call once, choose its route and bind it to the given buffers."""

        mode = normalize_stream_attn_mode(mode)
        paged = isinstance(key_cache, PagedKVCache)
        if paged and value_cache is not None:
            raise ValueError("value_cache must be omitted when key_cache is PagedKVCache")
        if not paged and value_cache is None:
            raise ValueError("value_cache is required for contiguous KV decode")
        if paged:
            ids: Dict[str, Any] = {"model_id": None, "layer_id": None}
            route = self._paged_route(mode, query, key_cache)
        else:
            ids = {"model_id": self.service.model_id if model_id is None else model_id,
                   "layer_id": self.service.layer_id if layer_id is None else layer_id}
            route = self._resolve_route(mode, query, key_cache, value_cache, ids)
        return StreamAttnEnginePlan(mode=mode, backend=route.backend, reason=route.reason, query=query,
                                    key_cache=key_cache, value_cache=value_cache, service=self.service,
                                    direct_runner=route.runner, **ids)

    def decode(self, query, key_cache, value_cache=None, *, mode: str = STREAMATTN_MODE_VERIFIED_AUTO,
               model_id: Optional[str] = None, layer_id: Optional[int] = None, return_info: bool = True):
        """``plan(...)`` followed by one ``run()``; loops should keep the plan instead."""

        bound = self.plan(query, key_cache, value_cache, mode=mode, model_id=model_id, layer_id=layer_id)
        return bound.run(return_info=return_info)


def stream_attn_decode(query, key_cache, value_cache=None, *, mode: str = STREAMATTN_MODE_VERIFIED_AUTO,
                       engine: Optional[StreamAttnEngine] = None, return_info: bool = True, **engine_kwargs):
    """One-shot decode (exported as ``decode``): uses ``engine`` or builds one from ``engine_kwargs``."""

    if engine is None:
        engine = StreamAttnEngine(**engine_kwargs)
    return engine.decode(query, key_cache, value_cache, mode=mode, return_info=return_info)
