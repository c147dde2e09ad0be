"""ctypes front-end of the C oracle (``sa_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Every function takes torch CPU tensors of any float dtype, upcasts them
exactly to float32 and calls the C code, which accumulates in double.  The
reference line ranges each C function follows are listed in ``sa_oracle.c``.
"""

from __future__ import annotations

import ctypes
import subprocess
import threading
from pathlib import Path
from typing import Optional, Sequence, Tuple

import torch

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "liboracle.so"
_LOCK = threading.Lock()
_LIB: Optional[ctypes.CDLL] = None

_f32p = ctypes.POINTER(ctypes.c_float)
_i64p = ctypes.POINTER(ctypes.c_int64)
_i64 = ctypes.c_int64
_int = ctypes.c_int


def build(force: bool = False) -> Path:
    """Compile ``liboracle.so`` with the Makefile beside this file."""

    with _LOCK:
        src = _HERE / "sa_oracle.c"
        stale = _LIB_PATH.exists() and _LIB_PATH.stat().st_mtime < src.stat().st_mtime
        if force or stale or not _LIB_PATH.exists():
            if _LIB_PATH.exists():
                _LIB_PATH.unlink()
            subprocess.run(["make", "-C", str(_HERE), "liboracle.so"], check=True,
                           capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        build()
        handle = ctypes.CDLL(str(_LIB_PATH))
        handle.oracle_exact_decode.argtypes = [
            _f32p, _f32p, _f32p, _f32p, _f32p, _i64p,
            _int, _int, _int, _int, _i64,
            _i64, _i64, _i64, _i64, _i64, _i64, _i64,
        ]
        handle.oracle_paged_decode.argtypes = [
            _f32p, _f32p, _f32p, _i64p, _i64p, _f32p, _i64p,
            _int, _int, _int, _int, _int, _int, _i64, _i64, _i64, _i64,
        ]
        handle.oracle_seed_blocks.argtypes = [_i64, _int, _int, _int, _int, _int, _i64p, _int]
        handle.oracle_seed_tokens_from_blocks.argtypes = [_i64, _int, _i64p, _int, _i64p, _i64]
        handle.oracle_seed_tokens_from_blocks.restype = _i64
        handle.oracle_seed_decode.argtypes = [
            _f32p, _f32p, _f32p, _f32p, _i64p, _i64,
            _int, _int, _int, _int, _i64, _i64, _i64, _i64, _i64,
        ]
        handle.oracle_merge_states.argtypes = [_f32p, _int, _i64, _int, _int, _f32p]
        _LIB = handle
    return _LIB


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(device="cpu", dtype=torch.float32)


def _ptr(t: Optional[torch.Tensor], ctype):
    if t is None:
        return ctypes.cast(None, ctype)
    return ctypes.cast(t.data_ptr(), ctype)


BLOCK_ORDER_IDS = {"sequential": 0, "recent_first": 1, "sink_recent_first": 2}


def _kv_strides(k: torch.Tensor, kv_layout: str) -> Tuple[int, int, int, int, int]:
    """Return (kv_heads, kv_len, stride_b, stride_n, stride_h) for a KV tensor."""

    if kv_layout == "BNHD":
        return int(k.shape[2]), int(k.shape[1]), k.stride(0), k.stride(1), k.stride(2)
    if kv_layout == "BHND":
        return int(k.shape[1]), int(k.shape[2]), k.stride(0), k.stride(2), k.stride(1)
    raise ValueError("kv_layout must be BNHD or BHND")


def exact_decode(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *,
    kv_layout: str = "BNHD",
    lengths: Optional[torch.Tensor] = None,
    token_range: Optional[Tuple[int, int]] = None,
    return_state: bool = False,
):
    """softmax(q K^T / sqrt(D)) V for q[B,1,Hq,D]; returns float32 [B,1,Hq,D].

    ``token_range`` restricts attention to tokens [lo, hi) (one context shard);
    ``return_state`` additionally returns (o, m, l) as [B,Hq,D+2] float32.
    """

    q = _f32(query).contiguous()
    k = _f32(key)
    v = _f32(value)
    if k.stride() != v.stride():
        v = v.contiguous()
        k = k.contiguous()
    if k.stride(3) != 1:
        k = k.contiguous()
        v = v.contiguous()
    batch, _, q_heads, dim = map(int, q.shape)
    kv_heads, kv_len, sb, sn, sh = _kv_strides(k, kv_layout)
    out = torch.empty(batch, 1, q_heads, dim, dtype=torch.float32)
    state = torch.empty(batch, q_heads, dim + 2, dtype=torch.float32) if return_state else None
    lens = lengths.detach().to("cpu", torch.int64).contiguous() if lengths is not None else None
    lo, hi = token_range if token_range is not None else (-1, -1)
    rc = lib().oracle_exact_decode(
        _ptr(q, _f32p), _ptr(k, _f32p), _ptr(v, _f32p), _ptr(out, _f32p),
        _ptr(state, _f32p), _ptr(lens, _i64p),
        batch, q_heads, kv_heads, dim, kv_len,
        q.stride(0), q.stride(2), sb, sn, sh, lo, hi,
    )
    if rc:
        raise ValueError(f"oracle_exact_decode failed with code {rc}")
    return (out, state) if return_state else out


def paged_decode(
    query: torch.Tensor,
    key_pages: torch.Tensor,
    value_pages: torch.Tensor,
    page_table: torch.Tensor,
    lengths: torch.Tensor,
    *,
    layout: str = "NHD",
    return_traversal: bool = False,
):
    """Paged exact decode; raises ValueError on an invalid active page entry."""

    q = _f32(query).contiguous()
    k = _f32(key_pages).contiguous()
    v = _f32(value_pages).contiguous()
    batch, _, q_heads, dim = map(int, q.shape)
    layout = layout.upper()
    num_pages = int(k.shape[0])
    if layout == "NHD":
        page_size, kv_heads = int(k.shape[1]), int(k.shape[2])
        sp, st, sh = k.stride(0), k.stride(1), k.stride(2)
    elif layout == "HND":
        kv_heads, page_size = int(k.shape[1]), int(k.shape[2])
        sp, st, sh = k.stride(0), k.stride(2), k.stride(1)
    else:
        raise ValueError("layout must be NHD or HND")
    table = page_table.detach().to("cpu", torch.int64).contiguous()
    lens = lengths.detach().to("cpu", torch.int64).contiguous()
    max_pages = int(table.shape[1])
    out = torch.empty(batch, 1, q_heads, dim, dtype=torch.float32)
    trav = torch.full((batch, max_pages), -1, dtype=torch.int64)
    rc = lib().oracle_paged_decode(
        _ptr(q, _f32p), _ptr(k, _f32p), _ptr(v, _f32p), _ptr(table, _i64p), _ptr(lens, _i64p),
        _ptr(out, _f32p), _ptr(trav, _i64p),
        batch, q_heads, kv_heads, dim, page_size, max_pages, num_pages, sp, st, sh,
    )
    if rc:
        raise ValueError(f"oracle_paged_decode rejected the page table (code {rc})")
    return (out, trav) if return_traversal else out


def seed_blocks(
    *,
    seq_len: int,
    block_size: int,
    sink_blocks: int,
    recent_blocks: int,
    middle_seed_blocks: int,
    block_order: str,
) -> list:
    cap = max(1, sink_blocks + recent_blocks + middle_seed_blocks)
    buf = (ctypes.c_int64 * cap)()
    n = lib().oracle_seed_blocks(
        seq_len, block_size, sink_blocks, recent_blocks, middle_seed_blocks,
        BLOCK_ORDER_IDS[block_order], buf, cap,
    )
    if n < 0:
        raise ValueError("oracle_seed_blocks failed")
    return [int(buf[i]) for i in range(n)]


def seed_tokens_from_blocks(*, seq_len: int, block_size: int, blocks: Sequence[int]) -> torch.Tensor:
    nb = len(blocks)
    cap = max(1, nb * block_size)
    blk = (ctypes.c_int64 * max(1, nb))(*[int(b) for b in blocks])
    out = torch.empty(cap, dtype=torch.int64)
    n = lib().oracle_seed_tokens_from_blocks(seq_len, block_size, blk, nb, _ptr(out, _i64p), cap)
    if n < 0:
        raise ValueError("oracle_seed_tokens_from_blocks failed")
    return out[:n].clone()


def seed_indices(**kwargs) -> torch.Tensor:
    blocks = seed_blocks(**kwargs)
    return seed_tokens_from_blocks(
        seq_len=kwargs["seq_len"], block_size=kwargs["block_size"], blocks=blocks
    )


def seed_decode(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    tokens: torch.Tensor,
    *,
    kv_layout: str = "BNHD",
) -> torch.Tensor:
    q = _f32(query).contiguous()
    k = _f32(key)
    v = _f32(value)
    if k.stride() != v.stride() or k.stride(3) != 1:
        k = k.contiguous()
        v = v.contiguous()
    batch, _, q_heads, dim = map(int, q.shape)
    kv_heads, _kv_len, sb, sn, sh = _kv_strides(k, kv_layout)
    toks = tokens.detach().to("cpu", torch.int64).contiguous()
    out = torch.empty(batch, 1, q_heads, dim, dtype=torch.float32)
    rc = lib().oracle_seed_decode(
        _ptr(q, _f32p), _ptr(k, _f32p), _ptr(v, _f32p), _ptr(out, _f32p),
        _ptr(toks, _i64p), int(toks.numel()),
        batch, q_heads, kv_heads, dim, q.stride(0), q.stride(2), sb, sn, sh,
    )
    if rc:
        raise ValueError(f"oracle_seed_decode failed with code {rc}")
    return out


def merge_states(states: torch.Tensor, *, log2_domain: bool) -> torch.Tensor:
    """states [parts, rows, D+2] -> merged normalised output [rows, D] float32."""

    s = _f32(states).contiguous()
    parts, rows, width = map(int, s.shape)
    dim = width - 2
    out = torch.empty(rows, dim, dtype=torch.float32)
    lib().oracle_merge_states(_ptr(s, _f32p), parts, rows, dim, int(bool(log2_domain)), _ptr(out, _f32p))
    return out
