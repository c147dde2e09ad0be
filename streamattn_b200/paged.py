"""Paged-KV cache contract and exact paged decode plan on the sm_100a kernels.

Mirrors ``stream_attention/paged.py`` of the reference: the ``PagedKVCache``
contract and its validation messages (paged.py:54-182), the split rule
(:185-198) and a bound ``PagedExactDecodePlan`` (:259-538).  Differences: one
kernel family serves every page size / layout / ragged length combination
(no per-shape promoted table), the launch balances work by the rows' actual
token counts read on the device at run time, and there is no CPU reference
path in the product - building a plan on non-CUDA tensors raises.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from . import native

PAGED_EXACT_NATIVE_BACKEND = "streamattn_paged_exact_native"
PAGED_EXACT_SM100_BACKEND = "streamattn_paged_sm100_exact"
# Names of the reference's sm_90 backends.  One sm_100 kernel serves contiguous, fragmented and
# ragged page tables alike, so all of them name the backend a plan on this package reports.
PAGED_EXACT_SM90_BACKEND = PAGED_EXACT_SM100_BACKEND
PAGED_EXACT_SM90_FRAGMENTED_BACKEND = PAGED_EXACT_SM100_BACKEND
PAGED_EXACT_SM90_FRAGMENTED_RAGGED_BACKEND = PAGED_EXACT_SM100_BACKEND


@dataclass(frozen=True)
class PagedKVCache:
    """Physical KV pages plus the logical request-to-page mapping.

    NHD pages are ``[num_pages, page_size, kv_heads, head_dim]``, HND pages are
    ``[num_pages, kv_heads, page_size, head_dim]``.  ``page_table`` is
    ``[batch, max_pages_per_request]`` with -1 in inactive trailing slots;
    ``sequence_lengths`` is ``[batch]``.
    """

    key: torch.Tensor
    value: torch.Tensor
    page_table: torch.Tensor
    sequence_lengths: torch.Tensor
    layout: str = "NHD"

    @property
    def normalized_layout(self) -> str:
        return str(self.layout).upper()

    def _axis(self, nhd_axis: int, hnd_axis: int) -> int:
        if self.key.dim() != 4:
            return 0
        return int(self.key.shape[nhd_axis if self.normalized_layout == "NHD" else hnd_axis])

    @property
    def num_pages(self) -> int:
        return int(self.key.shape[0]) if self.key.dim() == 4 else 0

    @property
    def page_size(self) -> int:
        return self._axis(1, 2)

    @property
    def kv_heads(self) -> int:
        return self._axis(2, 1)

    @property
    def head_dim(self) -> int:
        return int(self.key.shape[3]) if self.key.dim() == 4 else 0

    @property
    def batch_size(self) -> int:
        return int(self.page_table.shape[0]) if self.page_table.dim() == 2 else 0

    @property
    def max_pages_per_request(self) -> int:
        return int(self.page_table.shape[1]) if self.page_table.dim() == 2 else 0

    @property
    def max_sequence_length(self) -> int:
        return self.max_pages_per_request * self.page_size

    def validate(self, query: torch.Tensor, *, validate_metadata: bool = True) -> None:
        """Shape / dtype / device / layout checks, then (optionally) the host-side
        check that every active page-table entry names a physical page."""

        def need(ok: bool, message: str) -> None:
            if not ok:
                raise ValueError(message)

        need(query.dim() == 4 and query.shape[1] == 1, "paged exact decode query must be [batch, 1, heads, dim]")
        need(self.key.dim() == 4 and self.value.dim() == 4, "paged key/value caches must be rank 4")
        need(self.key.shape == self.value.shape, "paged key/value cache shapes must match")
        need(self.normalized_layout in {"NHD", "HND"}, "paged KV layout must be NHD or HND")
        need(self.page_table.dim() == 2, "page_table must be [batch, max_pages_per_request]")
        need(self.sequence_lengths.dim() == 1, "sequence_lengths must be [batch]")
        need(self.batch_size == int(query.shape[0]), "query and page_table batch sizes must match")
        need(self.sequence_lengths.numel() == self.batch_size, "sequence_lengths size must match batch")
        need(min(self.num_pages, self.page_size, self.max_pages_per_request) > 0,
             "paged cache dimensions must be positive")
        need(self.page_size <= 256, "paged exact decode currently supports page_size <= 256")
        need(self.head_dim == int(query.shape[3]), "query and paged cache head dimensions must match")
        need(self.kv_heads > 0 and int(query.shape[2]) % self.kv_heads == 0,
             "query heads must be a multiple of KV heads")
        need(self.head_dim <= 256 and self.head_dim & (self.head_dim - 1) == 0,
             "head_dim must be a power of two no larger than 256")
        need(query.dtype == self.key.dtype == self.value.dtype, "query and paged key/value dtypes must match")
        need(torch.is_floating_point(query), "query and paged key/value tensors must be floating point")
        need(self.page_table.dtype in {torch.int32, torch.int64}, "page_table must use int32 or int64")
        need(self.sequence_lengths.dtype in {torch.int32, torch.int64}, "sequence_lengths must use int32 or int64")
        tensors = (query, self.key, self.value, self.page_table, self.sequence_lengths)
        # A pinned host query is allowed (the kernel reads it across PCIe); everything else shares a device.
        placed = tensors[1:] if (query.device.type == "cpu" and query.is_pinned()) else tensors
        need(len({str(t.device) for t in placed}) == 1, "query and paged cache metadata must share a device")
        need(all(t.is_contiguous() for t in tensors), "query and paged cache tensors must be contiguous")
        if not validate_metadata:
            return
        lengths = self.sequence_lengths.detach().to(device="cpu", dtype=torch.int64)
        need(not bool((lengths <= 0).any()), "sequence_lengths must be positive")
        need(not bool((lengths > self.max_sequence_length).any()), "sequence_lengths exceed page_table capacity")
        table = self.page_table.detach().to(device="cpu", dtype=torch.int64)
        active_pages = (lengths + self.page_size - 1) // self.page_size
        slot = torch.arange(self.max_pages_per_request).unsqueeze(0)
        active = slot < active_pages.unsqueeze(1)
        bad = active & ((table < 0) | (table >= self.num_pages))
        need(not bool(bad.any()), "active page_table entries must reference physical pages")


def choose_paged_exact_splits(*, batch: int, query_heads: int, max_pages_per_request: int,
                              target_ctas: int = 512, max_splits: int = 32) -> int:
    """Minimum split count exposing ``target_ctas`` CTAs (reference paged.py:185-198)."""

    if min(batch, query_heads, max_pages_per_request, target_ctas, max_splits) <= 0:
        raise ValueError("paged split inputs must be positive")
    work = batch * query_heads
    return max(1, min(max_pages_per_request, max_splits, -(-target_ctas // work)))


@dataclass
class PagedExactDecodePlan:
    """Allocation-free exact decode bound to paged KV buffers."""

    query: torch.Tensor
    cache: PagedKVCache
    output: torch.Tensor
    splits: int
    workspace: Optional[dict]
    backend: str
    trace: Optional[torch.Tensor] = None
    _plan: Any = field(default=None, repr=False)

    @classmethod
    def build(cls, query: torch.Tensor, cache: PagedKVCache, *, output: Optional[torch.Tensor] = None,
              splits: Optional[int] = None, validate_metadata: bool = True, record_page_walk: bool = False,
              kernel: str = "auto", dynamic_schedule: Optional[bool] = None,
              **_compat: Any) -> "PagedExactDecodePlan":
        """Validate once and bind a plan.

        ``query`` and ``output`` may be pinned host tensors, as for ``ExactDecodePlan``.  ``splits`` asks for that many CTAs per (row, KV head); ``None`` sizes the
        grid to the GPU.  ``record_page_walk`` adds an int32 ``trace`` tensor
        shaped like the page table in which every run records the physical page
        it loaded per visited logical page.  ``dynamic_schedule`` as in
        ``ExactDecodePlan.build`` (faster, not bit-reproducible).  Launch hints of the reference's
        Triton path (``tokens_per_tile`` and friends) are accepted and ignored.
        """

        cache.validate(query, validate_metadata=validate_metadata)
        if output is None:
            output = torch.empty(query.shape, dtype=query.dtype, device=cache.key.device)
        if output.shape != query.shape or output.dtype != query.dtype:
            raise ValueError("output must match query shape and dtype")
        on_cache_device = output.device == cache.key.device
        if not (on_cache_device or (output.device.type == "cpu" and output.is_pinned())) or not output.is_contiguous():
            raise ValueError("output must be contiguous and live on the cache device (or in pinned host memory)")
        if splits is not None and not 0 < int(splits) <= cache.max_pages_per_request:
            raise ValueError("splits must be in [1, max_pages_per_request]")
        native.require_cuda(cache.key, host_io=(query, output))
        batch, _, q_heads, dim = (int(x) for x in query.shape)
        num_ctas = 0 if splits is None else int(splits) * batch * cache.kv_heads
        workspace = native.new_workspace(cache.key.device, batch, q_heads, cache.kv_heads, dim, num_ctas)
        trace = torch.full_like(cache.page_table, -1, dtype=torch.int32) if record_page_walk else None
        plan = native.paged_plan(query, cache.key, cache.value, cache.page_table, cache.sequence_lengths,
                                 output, workspace, layout=cache.normalized_layout, trace=trace,
                                 num_ctas=num_ctas, kernel=kernel, dynamic=dynamic_schedule)
        pairs = batch * cache.kv_heads
        backend = PAGED_EXACT_SM100_BACKEND if plan.kernel == native.SA_KERNEL_STREAM else PAGED_EXACT_NATIVE_BACKEND
        return cls(query=query, cache=cache, output=output, splits=max(1, -(-plan.num_ctas // pairs)),
                   workspace={"split_states": workspace}, backend=backend, trace=trace, _plan=plan)

    @property
    def workspace_bytes(self) -> int:
        if self.workspace is None:
            return 0
        return sum(t.numel() * t.element_size() for t in self.workspace.values())

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
        """Execute on the bound buffers; page contents, the page table and the
        lengths are read on the device at run time, so in-place updates are seen."""

        self._plan.run()
        return self.output

    def device_status(self) -> int:
        """Synchronise and return the kernels' status bits (0 = clean)."""

        return native.workspace_status(self.workspace["split_states"])


@dataclass
class PagedExactDecodeRunner:
    """Engine-facing runner: a paged plan plus its precomputed telemetry."""

    plan: PagedExactDecodePlan
    info: Any

    def run(self) -> torch.Tensor:
        return self.plan.run()

    def run_with_info(self):
        return self.run(), self.info


def stream_attn_paged_exact_decode(query: torch.Tensor, cache: PagedKVCache, *,
                                   output: Optional[torch.Tensor] = None,
                                   splits: Optional[int] = None) -> torch.Tensor:
    """Plan and execute one exact paged-KV decode call."""

    return PagedExactDecodePlan.build(query, cache, output=output, splits=splits).run()


def paged_exact_reference(query: torch.Tensor, cache: PagedKVCache, *,
                          output: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Page-by-page exact attention in plain tensor operations, for CHECKING results.

    Same contract as the reference's ``paged_exact_reference`` (paged.py:201-256): walks each
    request's page table in order, never gathers the pages into a contiguous cache, keeps a
    running (max, denominator, numerator) per query head in float32.  It runs wherever the
    tensors live and is slow by construction (a Python loop over pages).  Nothing in this
    package calls it: decode always goes through the sm_100a kernels and raises on tensors
    they cannot take.
    """

    cache.validate(query)
    if output is None:
        output = torch.empty_like(query)
    if output.shape != query.shape or output.dtype != query.dtype:
        raise ValueError("output must match query shape and dtype")
    if output.device != query.device or not output.is_contiguous():
        raise ValueError("output must be contiguous and share the query device")
    batch, _, heads, dim = (int(x) for x in query.shape)
    page, kv_heads = cache.page_size, cache.kv_heads
    group = heads // kv_heads
    hnd = cache.normalized_layout == "HND"
    scale = float(dim) ** -0.5
    lengths = [int(n) for n in cache.sequence_lengths.tolist()]
    table = cache.page_table.tolist()
    for b, n in enumerate(lengths):
        q = query[b, 0].float().view(kv_heads, group, dim)                      # [Hkv, G, D]
        top = torch.full((kv_heads, group), -float("inf"), dtype=torch.float32, device=query.device)
        den = torch.zeros_like(top)
        num = torch.zeros(kv_heads, group, dim, dtype=torch.float32, device=query.device)
        for slot in range(-(-n // page)):
            valid = min(page, n - slot * page)
            k_page, v_page = cache.key[table[b][slot]], cache.value[table[b][slot]]
            if hnd:                                                              # -> [Hkv, valid, D]
                k_page, v_page = k_page[:, :valid], v_page[:, :valid]
            else:
                k_page, v_page = k_page[:valid].transpose(0, 1), v_page[:valid].transpose(0, 1)
            scores = torch.einsum("hgd,htd->hgt", q, k_page.float()) * scale
            new_top = torch.maximum(top, scores.amax(dim=-1))
            keep = torch.exp(top - new_top)
            weights = torch.exp(scores - new_top[..., None])
            num = num * keep[..., None] + torch.einsum("hgt,htd->hgd", weights, v_page.float())
            den = den * keep + weights.sum(dim=-1)
            top = new_top
        output[b, 0].copy_((num / den[..., None]).view(heads, dim).to(output.dtype))
    return output
