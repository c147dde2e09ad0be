"""KV-cache update: the step that precedes every decode call.

The model adapter of the reference writes the current token's K/V into the cache (and rotates
q/K with the rotary embedding) before it asks for attention:
``_apply_qwen_rope`` + ``copy_`` in benchmarks/profile_seed_only_fused_rope_parity.py:24-30,97-102,
the append kernel in benchmarks/profile_kv_cache_update_floor.py:46-75 and the RoPE+append prologue
of kernels/gate0_seed_only_triton.py:731-770.  Here that step is one launch of ``append_kv_kernel``
(csrc/sa_append.cu) for contiguous and paged caches, with a host-side page allocator for the
paged case.  Everything stays on the device: positions are read from a device tensor and the
per-row lengths can be advanced in place, so a decode loop (append, decode, append, ...) needs no
host synchronisation and can be captured in a CUDA graph.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from . import native
from .paged import PagedKVCache


def _rows(t: torch.Tensor, heads_axis: int, name: str) -> Tuple[int, int, int, int, int]:
    """(batch, heads, dim, stride_b, stride_h) of a 4-D tensor with one token: [B,1,H,D] or [B,H,1,D]."""

    if t.dim() != 4 or t.stride(3) != 1:
        raise ValueError(f"{name} must be a 4-D tensor with a contiguous last dimension")
    token_axis = 3 - heads_axis
    if int(t.shape[token_axis]) != 1:
        raise ValueError(f"{name} must hold exactly one token")
    return int(t.shape[0]), int(t.shape[heads_axis]), int(t.shape[3]), int(t.stride(0)), int(t.stride(heads_axis))


def _heads_axis(layout: str) -> int:
    layout = layout.upper()
    if layout not in ("BHND", "BNHD"):
        raise ValueError("layout must be BHND or BNHD")
    return 1 if layout == "BHND" else 2


def _rope_args(cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], batch: int, dim: int, dtype: torch.dtype):
    if (cos is None) != (sin is None):
        raise ValueError("cos and sin must be given together")
    if cos is None:
        return None, None, 0
    for name, t in (("cos", cos), ("sin", sin)):
        if t.dtype != dtype:
            raise ValueError(f"{name} must have the cache dtype")
        if t.dim() == 3 and int(t.shape[1]) == 1:
            pass
        elif t.dim() != 2:
            raise ValueError(f"{name} must be [batch_or_1, dim] or [batch_or_1, 1, dim]")
        if int(t.shape[-1]) != dim or t.stride(-1) != 1 or int(t.shape[0]) not in (1, batch):
            raise ValueError(f"{name} must be [batch_or_1, (1,) dim] with a contiguous last dimension")
    if cos.shape[0] != sin.shape[0] or cos.stride(0) != sin.stride(0):
        raise ValueError("cos and sin must share shape and strides")
    return cos, sin, (0 if int(cos.shape[0]) == 1 else int(cos.stride(0)))


def _query_args(query, query_out, q_layout, batch, dim, dtype):
    if query is None:
        if query_out is not None:
            raise ValueError("query_out needs query")
        return None, None, 0, (0, 0, 0, 0)
    axis = _heads_axis(q_layout)
    qb, qh, qd, qi_sb, qi_sh = _rows(query, axis, "query")
    if query_out is None:
        query_out = torch.empty_like(query)
    ob, oh, od, qo_sb, qo_sh = _rows(query_out, axis, "query_out")
    if (qb, qd) != (batch, dim) or (ob, oh, od) != (qb, qh, qd) or query.dtype != dtype or query_out.dtype != dtype:
        raise ValueError("query / query_out must match the batch, head_dim and dtype of the cache")
    if query_out.data_ptr() == query.data_ptr():
        raise ValueError("query_out must not alias query")
    return query, query_out, qh, (qi_sb, qi_sh, qo_sb, qo_sh)


def _positions(positions: torch.Tensor, batch: int, lengths_out: Optional[torch.Tensor]):
    if positions.dtype not in native.SA_INDEX or positions.dim() != 1 or not positions.is_contiguous():
        raise ValueError("positions must be a contiguous 1-D int32/int64 tensor")
    if int(positions.numel()) not in (1, batch):
        raise ValueError("positions must hold one entry or one per batch row")
    if lengths_out is not None:
        if lengths_out.dtype != positions.dtype or lengths_out.shape != (batch,) or not lengths_out.is_contiguous():
            raise ValueError("lengths_out must be a contiguous [batch] tensor of the positions dtype")
    return native.SA_INDEX[positions.dtype], int(positions.numel())


def append_kv(key_cache: torch.Tensor, value_cache: torch.Tensor, key_new: torch.Tensor, value_new: torch.Tensor,
              positions: torch.Tensor, *, kv_layout: str = "BHND", new_layout: Optional[str] = None,
              cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
              query: Optional[torch.Tensor] = None, query_out: Optional[torch.Tensor] = None,
              query_layout: str = "BNHD", lengths_out: Optional[torch.Tensor] = None,
              status: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Write the current token's K/V rows into a contiguous cache (one launch, no host sync).

    ``key_cache``/``value_cache`` are ``[B, Hkv, N, D]`` (``kv_layout="BHND"``) or ``[B, N, Hkv, D]``;
    ``key_new``/``value_new`` hold one token in ``new_layout`` (default: the cache layout), i.e.
    ``[B, Hkv, 1, D]`` or ``[B, 1, Hkv, D]``.  ``positions`` (device int32/int64, one entry or one per
    row) is the token index written; ``lengths_out`` receives ``position + 1`` and may be the
    per-row ``positions`` tensor itself.  With ``cos``/``sin`` (``[B or 1, (1,) D]``, cache dtype) K is
    rotated first - ``x * cos + rotate_half(x) * sin`` with torch's rounding - and so is ``query``
    (layout ``query_layout``: ``[B, 1, Hq, D]`` or ``[B, Hq, 1, D]``) into ``query_out``, which is
    returned.  ``status`` (device int32 scalar) collects ``SA_DEV_BAD_POSITION`` for rows whose
    position is outside the cache; such rows are skipped.
    """

    return AppendKVPlan.build(key_cache, value_cache, key_new, value_new, positions, kv_layout=kv_layout,
                              new_layout=new_layout, cos=cos, sin=sin, query=query, query_out=query_out,
                              query_layout=query_layout, lengths_out=lengths_out, status=status).run()


def paged_append_kv(cache: PagedKVCache, key_new: torch.Tensor, value_new: torch.Tensor, *,
                    positions: Optional[torch.Tensor] = None, advance_lengths: bool = True,
                    new_layout: str = "BNHD", cos: Optional[torch.Tensor] = None,
                    sin: Optional[torch.Tensor] = None, query: Optional[torch.Tensor] = None,
                    query_out: Optional[torch.Tensor] = None, query_layout: str = "BNHD",
                    status: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Write the current token's K/V rows into a paged cache.

    By default the row of request ``b`` goes to token index ``cache.sequence_lengths[b]`` and that
    length is advanced in place on the device (``advance_lengths``), so a plan bound to the cache
    sees the new token on its next run.  The page that holds the position must already be in
    ``cache.page_table`` (see :class:`PagedKVWriter`); a missing or out-of-range page is reported
    through ``status`` (``SA_DEV_BAD_PAGE``) and the row is skipped.
    """

    return AppendKVPlan.build_paged(cache, key_new, value_new, positions=positions, advance_lengths=advance_lengths,
                                    new_layout=new_layout, cos=cos, sin=sin, query=query, query_out=query_out,
                                    query_layout=query_layout, status=status).run()


class AppendKVPlan:
    """A validated, bound cache update: ``run()`` is one native call (no checks, no allocation).

    The tensors are bound by address, like the decode plans: refill ``key_new`` / ``value_new`` /
    ``query`` / ``cos`` / ``sin`` in place between runs; positions and lengths are read on the
    device at run time.
    """

    def __init__(self, fn_name: str, args: tuple, device: torch.device, keep: tuple, query_out) -> None:
        self._fn = getattr(native.load(), fn_name)
        self._args = args
        self._device = device
        self._device_index = device.index if device.index is not None else torch.cuda.current_device()
        self._keep = keep
        self.query_out = query_out

    def run(self) -> Optional[torch.Tensor]:
        if torch.cuda.current_device() != self._device_index:
            with torch.cuda.device(self._device_index):
                rc = self._fn(*self._args, native._current_raw_stream(self._device_index))
        else:
            rc = self._fn(*self._args, native._current_raw_stream(self._device_index))
        if rc:
            native.check(rc)
        return self.query_out

    @classmethod
    def build(cls, key_cache: torch.Tensor, value_cache: torch.Tensor, key_new: torch.Tensor,
              value_new: torch.Tensor, positions: torch.Tensor, *, kv_layout: str = "BHND",
              new_layout: Optional[str] = None, cos: Optional[torch.Tensor] = None,
              sin: Optional[torch.Tensor] = None, query: Optional[torch.Tensor] = None,
              query_out: Optional[torch.Tensor] = None, query_layout: str = "BNHD",
              lengths_out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> "AppendKVPlan":
        """Arguments as :func:`append_kv`."""

        device = native.require_cuda(key_cache, value_cache, key_new, value_new, positions, cos, sin, query,
                                     query_out, lengths_out, status)
        dtype = key_cache.dtype
        if dtype not in native.SA_DTYPE or any(t.dtype != dtype for t in (value_cache, key_new, value_new)):
            raise ValueError("caches and new rows must share a dtype of bf16, fp16 or fp32")
        kv_heads, kv_len, sb, sn, sh = native._kv_geometry(key_cache, value_cache, kv_layout)
        batch, dim = int(key_cache.shape[0]), int(key_cache.shape[3])
        nb, nh, nd, new_sb, new_sh = _rows(key_new, _heads_axis(new_layout or kv_layout), "key_new")
        if (nb, nh, nd) != (batch, kv_heads, dim) or value_new.shape != key_new.shape \
                or value_new.stride() != key_new.stride():
            raise ValueError("key_new / value_new must be one token of the cache's batch, KV heads and head_dim")
        pos_dtype, num_positions = _positions(positions, batch, lengths_out)
        cos, sin, rope_sb = _rope_args(cos, sin, batch, dim, dtype)
        query, query_out, q_heads, qs = _query_args(query, query_out, query_layout, batch, dim, dtype)
        args = (native._ptr(key_new), native._ptr(value_new), native._ptr(key_cache), native._ptr(value_cache),
                native._ptr(positions), pos_dtype, num_positions, native._ptr(lengths_out),
                native._ptr(cos), native._ptr(sin), rope_sb,
                native._ptr(query), native._ptr(query_out), q_heads, *qs,
                batch, kv_heads, dim, kv_len, new_sb, new_sh, sb, sn, sh,
                native.SA_DTYPE[dtype], native._ptr(status))
        keep = (key_cache, value_cache, key_new, value_new, positions, lengths_out, cos, sin, query, query_out, status)
        return cls("sa_append_kv", args, device, keep, query_out)

    @classmethod
    def build_paged(cls, cache: PagedKVCache, key_new: torch.Tensor, value_new: torch.Tensor, *,
                    positions: Optional[torch.Tensor] = None, advance_lengths: bool = True,
                    new_layout: str = "BNHD", cos: Optional[torch.Tensor] = None,
                    sin: Optional[torch.Tensor] = None, query: Optional[torch.Tensor] = None,
                    query_out: Optional[torch.Tensor] = None, query_layout: str = "BNHD",
                    status: Optional[torch.Tensor] = None) -> "AppendKVPlan":
        """Arguments as :func:`paged_append_kv`."""

        return cls(*_paged_call(cache, key_new, value_new, positions, advance_lengths, new_layout, cos, sin, query,
                                query_out, query_layout, status))


def _paged_call(cache, key_new, value_new, positions, advance_lengths, new_layout, cos, sin, query, query_out,
                query_layout, status):
    if positions is None:
        positions = cache.sequence_lengths
    lengths_out = cache.sequence_lengths if advance_lengths else None
    device = native.require_cuda(cache.key, cache.value, cache.page_table, key_new, value_new, positions, cos, sin,
                                 query, query_out, lengths_out, status)
    dtype = cache.key.dtype
    if dtype not in native.SA_DTYPE or any(t.dtype != dtype for t in (cache.value, key_new, value_new)):
        raise ValueError("caches and new rows must share a dtype of bf16, fp16 or fp32")
    layout = cache.normalized_layout
    if not (cache.key.is_contiguous() and cache.value.is_contiguous() and cache.page_table.is_contiguous()):
        raise ValueError("paged cache tensors must be contiguous")
    num_pages = int(cache.key.shape[0])
    if layout == "NHD":
        page_size, kv_heads = int(cache.key.shape[1]), int(cache.key.shape[2])
    else:
        kv_heads, page_size = int(cache.key.shape[1]), int(cache.key.shape[2])
    batch, max_pages = int(cache.page_table.shape[0]), int(cache.page_table.shape[1])
    dim = int(cache.key.shape[3])
    nb, nh, nd, new_sb, new_sh = _rows(key_new, _heads_axis(new_layout), "key_new")
    if (nb, nh, nd) != (batch, kv_heads, dim) or value_new.shape != key_new.shape or value_new.stride() != key_new.stride():
        raise ValueError("key_new / value_new must be one token of the cache's batch, KV heads and head_dim")
    if lengths_out is not None and lengths_out.dtype != positions.dtype:
        raise ValueError("positions must have the dtype of cache.sequence_lengths when lengths are advanced")
    pos_dtype, num_positions = _positions(positions, batch, lengths_out)
    cos, sin, rope_sb = _rope_args(cos, sin, batch, dim, dtype)
    query, query_out, q_heads, qs = _query_args(query, query_out, query_layout, batch, dim, dtype)
    args = (native._ptr(key_new), native._ptr(value_new), native._ptr(cache.key), native._ptr(cache.value),
            native._ptr(cache.page_table), native.SA_INDEX[cache.page_table.dtype],
            native._ptr(positions), pos_dtype, num_positions, native._ptr(lengths_out),
            native._ptr(cos), native._ptr(sin), rope_sb,
            native._ptr(query), native._ptr(query_out), q_heads, *qs,
            batch, kv_heads, dim, page_size, max_pages, num_pages, native.SA_LAYOUT[layout], new_sb, new_sh,
            native.SA_DTYPE[dtype], native._ptr(status))
    keep = (cache, key_new, value_new, positions, lengths_out, cos, sin, query, query_out, status)
    return "sa_paged_append_kv", args, device, keep, query_out


class PagePool:
    """Free-list allocator over the physical pages of a paged cache (host side, no device work)."""

    def __init__(self, num_pages: int, reserved: Sequence[int] = ()) -> None:
        if num_pages <= 0:
            raise ValueError("num_pages must be positive")
        taken = set(int(p) for p in reserved)
        if any(p < 0 or p >= num_pages for p in taken):
            raise ValueError("reserved page id out of range")
        self.num_pages = int(num_pages)
        # Lowest ids are handed out first, so an empty pool fills the cache front to back.
        self._free: List[int] = [p for p in range(num_pages - 1, -1, -1) if p not in taken]
        self._used = taken

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def allocate(self, count: int) -> List[int]:
        if count < 0:
            raise ValueError("count must be >= 0")
        if count > len(self._free):
            raise RuntimeError(f"out of KV pages: {count} requested, {len(self._free)} free")
        pages = [self._free.pop() for _ in range(count)]
        self._used.update(pages)
        return pages

    def release(self, pages: Sequence[int]) -> None:
        for p in pages:
            p = int(p)
            if p not in self._used:
                raise ValueError(f"page {p} is not allocated")
            self._used.remove(p)
            self._free.append(p)


@dataclass
class PagedKVWriter:
    """Grows the requests of a :class:`PagedKVCache` token by token.

    Holds host mirrors of the lengths and of the pages each request owns, assigns a fresh page
    from the pool whenever a request's next token starts a new page (one small device write into
    ``cache.page_table``), and launches the append.  The device never waits for the host: page
    assignment for step ``t + 1`` can be enqueued while step ``t`` is still running.
    """

    cache: PagedKVCache
    pool: PagePool
    lengths: List[int]
    pages: List[List[int]] = field(default_factory=list)

    @classmethod
    def attach(cls, cache: PagedKVCache, pool: Optional[PagePool] = None) -> "PagedKVWriter":
        """Adopt a cache as it is (reads lengths and page table back once)."""

        lengths = [int(x) for x in cache.sequence_lengths.tolist()]
        table = cache.page_table.tolist()
        page_size = cache.page_size
        pages = [[int(p) for p in row[: -(-n // page_size)]] for row, n in zip(table, lengths)]
        if pool is None:
            pool = PagePool(int(cache.key.shape[0]), reserved=[p for row in pages for p in row])
        return cls(cache=cache, pool=pool, lengths=lengths, pages=pages)

    def reserve(self, tokens: int = 1) -> int:
        """Make sure every request has pages for ``tokens`` more tokens; returns pages assigned.

        All-or-nothing: every row's need is worked out and checked against the table capacity and
        the pool first, and only then are pages taken and the device table written, so a refused
        call leaves the pool, the host mirrors and the device table exactly as they were.
        """

        page_size = self.cache.page_size
        max_pages = int(self.cache.page_table.shape[1])
        wanted: List[Tuple[int, int, int]] = []  # (row, pages it has, pages it needs)
        for b, n in enumerate(self.lengths):
            need = -(-(n + tokens) // page_size)
            if need > max_pages:
                raise ValueError("sequence lengths exceed page_table capacity")
            if need > len(self.pages[b]):
                wanted.append((b, len(self.pages[b]), need))
        total = sum(need - have for _, have, need in wanted)
        if total > self.pool.free_pages:
            raise RuntimeError(f"out of KV pages: {total} requested, {self.pool.free_pages} free")
        if total == 0:
            return 0
        fresh = self.pool.allocate(total)
        rows: List[int] = []
        slots: List[int] = []
        taken = 0
        for b, have, need in wanted:
            mine = fresh[taken:taken + need - have]
            taken += need - have
            rows.extend([b] * len(mine))
            slots.extend(range(have, need))
            self.pages[b].extend(mine)
        table = self.cache.page_table
        index = (torch.tensor(rows, device=table.device), torch.tensor(slots, device=table.device))
        table.index_put_(index, torch.tensor(fresh, dtype=table.dtype, device=table.device))
        return total

    def append(self, key_new: torch.Tensor, value_new: torch.Tensor, **kwargs) -> Optional[torch.Tensor]:
        """Append one token to every request (assigning pages first); lengths advance on the device."""

        self.reserve(1)
        out = paged_append_kv(self.cache, key_new, value_new, advance_lengths=True, **kwargs)
        self.lengths = [n + 1 for n in self.lengths]
        return out

    def release(self, row: int) -> None:
        """Give the pages of request ``row`` back to the pool.

        The row becomes an empty request on the host AND on the device: its table row is filled
        with -1 and its entry of ``cache.sequence_lengths`` is set to 0 on the current stream, so
        the next append writes position 0 of a fresh page and a decode in between reads nothing.
        """

        self.pool.release(self.pages[row])
        self.pages[row] = []
        self.lengths[row] = 0
        self.cache.page_table[row].fill_(-1)
        self.cache.sequence_lengths[row].fill_(0)


__all__ = ["append_kv", "paged_append_kv", "AppendKVPlan", "PagePool", "PagedKVWriter"]
