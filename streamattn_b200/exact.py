"""Bound exact-decode plan on the sm_100a kernels.

Counterpart of the reference's ``ExactDecodePlan``
(``stream_attention/backends/sm90/transposed_gqa_exact.py:264-430``): built once
over stable Q/K/V/output buffers, ``run()`` enqueues one launch and allocates
nothing.  Where the reference runs a producer kernel plus a merge kernel over a
fixed split count, this plan runs one launch whose CTAs take equal slices of a
flat tile list and merge their split states in the same launch; ``num_splits``
is kept as the knob "CTAs per (row, KV head)".
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from . import native
from .decode import infer_kv_layout

SM100_EXACT_BACKEND = "sm100_gqa_exact"


def choose_num_splits(*, batch: int, kv_heads: int, kv_len: int, target_producer_ctas: int = 256) -> int:
    """Smallest split count reaching the CTA target (reference transposed_gqa_exact.py:88-101)."""

    if batch <= 0 or kv_heads <= 0 or kv_len <= 0 or kv_len % 64:
        raise ValueError("batch/kv_heads must be positive and kv_len divisible by 64")
    pairs = batch * kv_heads
    needed = -(-target_producer_ctas // pairs)
    return max(1, min(kv_len // 64, needed))


@dataclass
class ExactDecodePlan:
    """Allocation-free exact GQA decode over bound buffers."""

    query: torch.Tensor
    key_cache: torch.Tensor
    value_cache: torch.Tensor
    output: torch.Tensor
    workspace: torch.Tensor
    num_splits: int
    kv_layout: str
    backend: str = SM100_EXACT_BACKEND
    _plan: native.NativePlan = field(default=None, repr=False)

    @classmethod
    def build(cls, query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor, *,
              output: Optional[torch.Tensor] = None, num_splits: Optional[int] = None,
              promoted_only: bool = True, kv_layout: Optional[str] = None,
              seq_lens: Optional[torch.Tensor] = None, kernel: str = "auto",
              dynamic_schedule: Optional[bool] = None,
              row_indices: Optional[torch.Tensor] = None) -> "ExactDecodePlan":
        """Bind a plan.

        ``query`` and ``output`` may be pinned host tensors (the kernel then reads
        the query and writes the result across PCIe itself, saving the two copies a
        host-driven decode step would otherwise enqueue).  ``kv_layout`` is ``"BHND"`` (head-major ``[B, Hkv, N, D]``, what the
        reference's plan takes) or ``"BNHD"``; by default head-major is assumed,
        as in the reference.  ``num_splits`` asks for that many CTAs per
        (row, KV head); ``None`` sizes the grid to the GPU.  ``promoted_only``
        is accepted for compatibility and has no effect: every supported shape
        is served.  ``dynamic_schedule=True`` lets the CTAs of a (row, KV head)
        pair claim tiles from a device counter (up to 3 % faster when HBM
        bound, in some runs slower: measure; results stay within tolerance but are no longer bit-identical
        from launch to launch); ``None`` follows ``STREAMATTN_B200_SCHEDULE``.
        ``row_indices`` (device int32/int64 tensor, read at run time) restricts the
        plan to those batch rows: the output rows of all other rows stay untouched
        (see :meth:`set_row_indices`).
        """

        del promoted_only
        native.require_cuda(key_cache, value_cache, host_io=(query, output))
        layout = kv_layout or "BHND"
        if query.dim() != 4 or key_cache.dim() != 4 or value_cache.dim() != 4:
            raise ValueError("unsupported exact decode buffers: rank")
        batch, _, q_heads, dim = (int(x) for x in query.shape)
        kv_heads = int(key_cache.shape[1] if layout == "BHND" else key_cache.shape[2])
        if kv_heads <= 0 or q_heads % kv_heads:
            raise ValueError("unsupported exact decode buffers: gqa")
        if output is None:
            output = torch.empty(query.shape, dtype=query.dtype, device=key_cache.device)
        if output.shape != query.shape or output.dtype != query.dtype:
            raise ValueError("output must match query shape and dtype")
        if not (output.is_cuda or output.is_pinned()) or not output.is_contiguous():
            raise ValueError("output must be a contiguous CUDA (or pinned host) tensor")
        if num_splits is not None and num_splits <= 0:
            raise ValueError("num_splits must be positive")
        num_ctas = 0 if num_splits is None else int(num_splits) * batch * kv_heads
        workspace = native.new_workspace(key_cache.device, batch, q_heads, kv_heads, dim, num_ctas)
        plan = native.exact_plan(query, key_cache, value_cache, output, workspace, kv_layout=layout,
                                 seq_lens=seq_lens, num_ctas=num_ctas, kernel=kernel, dynamic=dynamic_schedule)
        if row_indices is not None:
            plan.set_rows(row_indices)
        pairs = batch * kv_heads
        return cls(query=query, key_cache=key_cache, value_cache=value_cache, output=output,
                   workspace=workspace, num_splits=max(1, -(-plan.num_ctas // pairs)), kv_layout=layout,
                   _plan=plan)

    @property
    def workspace_bytes(self) -> int:
        return self.workspace.numel()

    @property
    def kernel_name(self) -> str:
        return self._plan.kernel_name

    @property
    def num_ctas(self) -> int:
        return self._plan.num_ctas

    @property
    def launches_per_run(self) -> int:
        return self._plan.launches

    def run(self) -> torch.Tensor:
        self._plan.run()
        return self.output

    def set_row_indices(self, row_indices: Optional[torch.Tensor]) -> None:
        """Compute only the listed batch rows from now on (``None``: every row again).

        Counterpart of the ``row_indices`` argument of the reference's row-refresh kernel
        (kernels/gate0_exact_refresh_triton.py:251-259): the tensor lives on the device and is
        read by each launch, so its contents may change between runs without touching the plan.
        """

        self._plan.set_rows(row_indices)

    # The reference exposes several launch orders of its two kernels; here they
    # are one launch, kept as aliases so existing call sites still work.
    run_two_call = run
    run_combined = run
    run_warp_merge = run

    def device_status(self) -> int:
        """Synchronise and return the kernels' status bits (0 = clean)."""

        return native.workspace_status(self.workspace)


def supports_exact_decode(query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor) -> bool:
    """Whether :class:`ExactDecodePlan` can bind these buffers (CUDA sm_100, matching shapes)."""

    from .decode import _exact_native_supported

    return _exact_native_supported(query, key_cache, value_cache)


def exact_decode_attention_rows_forward_out_bhnd(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                                                output: torch.Tensor, cache_position: torch.Tensor, *,
                                                row_indices=None, **_launch_hints) -> torch.Tensor:
    """Exact decode of selected batch rows over a BHND cache prefix, written in place.

    Same call as the reference's ``exact_decode_attention_rows_triton_forward_out_bhnd``
    (kernels/gate0_exact_refresh_triton.py:266-344): ``query`` is ``[B, Hq, 1, D]``, ``key`` /
    ``value`` are ``[B, Hkv, N, D]``, ``output`` is ``[B, 1, Hq, D]`` and only the rows in
    ``row_indices`` (a tensor, or any collection of ints; ``None`` = all rows) are overwritten.
    The prefix length of every row is ``min(cache_position[0] + 1, N)``, read on the device.
    Tile and warp hints of the Triton launcher are accepted and ignored.  A plan is built per
    call; steady-state loops should keep an :class:`ExactDecodePlan` with ``row_indices=``.
    """

    native.require_cuda(query, key, value, output, cache_position)
    if query.dim() != 4 or key.dim() != 4 or value.dim() != 4:
        raise ValueError("query must be [batch, heads, 1, dim], key/value must be [batch, kv_heads, seq, dim]")
    if query.shape[2] != 1:
        raise ValueError("exact refresh only supports query_len == 1")
    if tuple(output.shape) != (query.shape[0], 1, query.shape[1], query.shape[3]):
        raise ValueError("output must be [batch, 1, heads, dim]")
    if key.shape != value.shape:
        raise ValueError("key and value must have matching shape")
    if query.shape[0] != key.shape[0] or query.shape[3] != key.shape[3]:
        raise ValueError("query/key/value must have matching batch and dim")
    if query.shape[1] % key.shape[1] != 0:
        raise ValueError("query heads must be a multiple of KV heads")
    if not output.is_contiguous():
        raise ValueError("output must be contiguous")
    if cache_position.numel() < 1:
        raise ValueError("cache_position must contain at least one element")
    batch, heads, _, dim = (int(x) for x in query.shape)
    device = query.device
    if row_indices is None:
        rows = None
    elif isinstance(row_indices, torch.Tensor):
        rows = row_indices.to(device=device, dtype=torch.int64).contiguous().reshape(-1)
    else:
        rows = torch.tensor(sorted({int(r) for r in row_indices if 0 <= int(r) < batch}), dtype=torch.int64,
                            device=device)
    if rows is not None and rows.numel() == 0:
        return output
    lens = (cache_position.reshape(-1)[:1].to(torch.int64) + 1).expand(batch).contiguous()
    workspace = native.new_workspace(device, batch, heads, int(key.shape[1]), dim)
    plan = native.exact_plan(query.transpose(1, 2), key, value, output, workspace, kv_layout="BHND", seq_lens=lens)
    if rows is not None:
        plan.set_rows(rows)
    plan.run()
    return output


__all__ = ["ExactDecodePlan", "exact_decode_attention_rows_forward_out_bhnd", "SM100_EXACT_BACKEND", "choose_num_splits", "infer_kv_layout", "supports_exact_decode"]
