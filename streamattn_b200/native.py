"""ctypes binding of ``libstreamattn_b200.so`` (the C ABI in ``include/streamattn_b200.h``).

There is no fallback: if the library cannot be loaded (or built with nvcc) every
entry point raises.  Tensors are passed as raw device pointers plus the current
CUDA stream handle of their device.
"""

from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional, Sequence

import torch

from . import build as _build

SA_OK = 0
SA_ERR_INVALID = 1
SA_ERR_UNSUPPORTED = 2
SA_ERR_CUDA = 3
SA_ERR_DEVICE = 4

SA_DTYPE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
SA_INDEX = {torch.int32: 0, torch.int64: 1}
SA_LAYOUT = {"NHD": 0, "HND": 1}
SA_BLOCK_ORDER = {"sequential": 0, "recent_first": 1, "sink_recent_first": 2}
SA_OUT_FINAL = 0
SA_OUT_STATE = 1
SA_KERNEL_AUTO = 0
SA_KERNEL_STREAM = 1
SA_KERNEL_GENERIC = 2
SA_KERNEL = {"auto": SA_KERNEL_AUTO, "stream": SA_KERNEL_STREAM, "generic": SA_KERNEL_GENERIC}
SA_KERNEL_FLAG_DYNAMIC = 0x100
SA_KERNEL_NAMES = {SA_KERNEL_STREAM: "sm100_tma_mma_stream", SA_KERNEL_GENERIC: "sm100_generic_simt"}
SA_DEV_PIPELINE_TIMEOUT = 1
SA_DEV_BAD_PAGE = 2
SA_DEV_BAD_POSITION = 4
SA_MAX_SEED_BLOCKS = 256

_vp = ctypes.c_void_p
_i = ctypes.c_int
_i64 = ctypes.c_int64
_sz = ctypes.c_size_t
_i32p = ctypes.POINTER(ctypes.c_int32)
_i64p = ctypes.POINTER(ctypes.c_int64)

_EXACT_ARGS = [_vp, _vp, _vp, _vp, _vp, _sz, _vp, _i, _i, _i, _i, _i, _i64,
               _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _i]
_PAGED_ARGS = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _i, _i, _i, _i, _i, _i, _i64,
               _i, _i, _i, _i, _i, _i, _i]
_SEED_COMMON = [_vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64, _i]

_SIGNATURES = {
    "sa_version": ([], _i),
    "sa_last_error": ([], ctypes.c_char_p),
    "sa_device_supported": ([_i], _i),
    "sa_device_sm_count": ([_i], _i),
    "sa_workspace_bytes": ([_i, _i, _i, _i, _i], _sz),
    "sa_workspace_status": ([_vp, _vp], _i),
    "sa_exact_decode": (_EXACT_ARGS + [_vp], _i),
    "sa_exact_decode_static": ([_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i64,
                                _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _i, _vp], _i),
    "sa_static_status": ([_vp], _i),
    "sa_paged_decode": (_PAGED_ARGS + [_vp], _i),
    "sa_seed_blocks": ([_i64, _i, _i, _i, _i, _i, _i32p, _i], _i),
    "sa_seed_token_indices": ([_i64, _i, _i32p, _i, _i64p, _i64], _i64),
    "sa_seed_decode": (_SEED_COMMON + [_i, _i, _i, _i, _i, _i, _i, _vp], _i),
    "sa_seed_decode_blocks": (_SEED_COMMON + [_i, _i32p, _i, _i, _i, _vp], _i),
    "sa_merge_states": ([_vp, _i, _i64, _i, _vp, _i, _vp], _i),
    "sa_block_scores": ([_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _vp], _i),
    "sa_seed_list_length": ([_i64, _i, _i, _i, _i], _i),
    "sa_select_seed_blocks": ([_vp, _vp, _i, _i, _i, _i64, _i, _i, _i, _i, _i, _vp], _i),
    "sa_seed_plan_create_device": (_SEED_COMMON + [_i, _vp, _i, _i, _i, _i], _vp),
    "sa_cp_exchange_bytes": ([_i, _i64, _i], _sz),
    "sa_cp_exchange_merge": ([_vp, ctypes.POINTER(ctypes.c_uint64), _i, _i, ctypes.c_uint32, _i64, _i, _vp, _i, _vp], _i),
    "sa_cp_exchange_status": ([_vp, _i, _i64, _i, _vp], _i),
    "sa_cp_fused_bytes": ([_i, _i, _i, _i, _i], _sz),
    "sa_cp_fused_plan_create": ([_vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64,
                                 _i, _i, ctypes.POINTER(ctypes.c_uint64), _i, _i], _vp),
    "sa_exact_plan_create": (_EXACT_ARGS, _vp),
    "sa_paged_plan_create": (_PAGED_ARGS, _vp),
    "sa_seed_plan_create": (_SEED_COMMON + [_i, _i32p, _i, _i, _i], _vp),
    "sa_plan_run": ([_vp, _vp], _i),
    "sa_plan_kernel": ([_vp], _i),
    "sa_plan_num_ctas": ([_vp], _i),
    "sa_plan_launches": ([_vp], _i),
    "sa_plan_destroy": ([_vp], None),
    "sa_plan_set_rows": ([_vp, _vp, _i, _i], _i),
    "sa_set_wait_limit_ns": ([ctypes.c_uint64], _i),
    "sa_plan_set_wait_limit_ns": ([_vp, ctypes.c_uint64], _i),
    "sa_o_proj": ([_vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i, _i, _vp], _i),
    # k_new v_new k_cache v_cache | positions pos_dtype num_positions lens_out | cos sin rope_stride_b |
    # q_in q_out q_heads 4 q strides | batch kv_heads head_dim kv_len | 2 new strides | 3 kv strides | dtype status stream
    "sa_append_kv": ([_vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _i64, _vp, _vp, _i, _i64, _i64, _i64, _i64,
                      _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64, _i, _vp, _vp], _i),
    # ... k_pages v_pages page_table table_dtype | positions ... | batch kv_heads head_dim page_size max_pages
    # num_pages layout | 2 new strides | dtype status stream
    "sa_paged_append_kv": ([_vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _vp, _vp, _vp, _i64, _vp, _vp, _i, _i64, _i64,
                            _i64, _i64, _i, _i, _i, _i, _i, _i64, _i, _i64, _i64, _i, _vp, _vp], _i),
}

_LOCK = threading.Lock()
_LIB: Optional[ctypes.CDLL] = None


def exported_symbols() -> Sequence[str]:
    """Names this binding expects the library to export."""

    return tuple(_SIGNATURES)


def load() -> ctypes.CDLL:
    """Load (building first if needed) the native library; raises if impossible."""

    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = _build.LIB_PATH
        if _build.is_stale():
            if path.is_file() and _build.find_nvcc() is None:
                pass  # a prebuilt library without a compiler: use it as shipped
            else:
                path = _build.build()
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as exc:
            raise RuntimeError(
                f"cannot load {path}: {exc}; streamattn_b200 has no CPU or interpreted fallback"
            ) from exc
        for name, (argtypes, restype) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _LIB = lib
        return lib


def last_error() -> str:
    msg = load().sa_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc: int) -> None:
    """Map a C status code to the exception types of the reference API."""

    if rc == SA_OK:
        return
    msg = last_error()
    if rc in (SA_ERR_INVALID, SA_ERR_UNSUPPORTED):
        raise ValueError(msg or f"streamattn_b200 native error {rc}")
    raise RuntimeError(msg or f"streamattn_b200 native error {rc}")


def require_cuda(*tensors: torch.Tensor, host_io: Sequence[torch.Tensor] = ()) -> torch.device:
    """All tensors must live on one CUDA device; there is no CPU execution path.

    Tensors listed in ``host_io`` (the query and the output of a plan) may instead be pinned
    host tensors: pinned memory is addressable from the GPU, so the kernels read the query and
    write the result across PCIe themselves and no separate copy is enqueued.
    """

    devices = {t.device for t in tensors if t is not None}
    for t in host_io:
        if t is None:
            continue
        if t.device.type == "cpu" and t.is_pinned():
            continue
        devices.add(t.device)
    if len(devices) != 1:
        raise ValueError("all tensors of a decode call must share one device")
    device = next(iter(devices))
    if device.type != "cuda":
        raise RuntimeError(
            "streamattn_b200 executes only on CUDA (sm_100) tensors; it has no CPU fallback "
            f"(got device {device})"
        )
    return device


def device_supported(device: torch.device) -> bool:
    index = device.index if device.index is not None else torch.cuda.current_device()
    return bool(load().sa_device_supported(int(index)))


def sm_count(device: torch.device) -> int:
    """Streaming multiprocessors of ``device`` (148 on a B200)."""

    index = device.index if device.index is not None else torch.cuda.current_device()
    return int(load().sa_device_sm_count(int(index))) or 148


_current_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
if _current_raw_stream is None:  # older torch: go through the Stream object
    def _current_raw_stream(index: int) -> int:
        return int(torch.cuda.current_stream(index).cuda_stream)


def stream_handle(device: torch.device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    return int(_current_raw_stream(index))


def workspace_bytes(batch: int, q_heads: int, kv_heads: int, head_dim: int, num_ctas: int = 0) -> int:
    n = int(load().sa_workspace_bytes(batch, q_heads, kv_heads, head_dim, num_ctas))
    if n == 0:
        raise ValueError(last_error())
    return n


def new_workspace(device: torch.device, batch: int, q_heads: int, kv_heads: int, head_dim: int,
                  num_ctas: int = 0) -> torch.Tensor:
    """Zero-filled workspace (the library needs zeros once, then keeps it consistent)."""

    return torch.zeros(workspace_bytes(batch, q_heads, kv_heads, head_dim, num_ctas),
                       dtype=torch.uint8, device=device)


def workspace_status(workspace: torch.Tensor) -> int:
    """Synchronise and return (then clear) the status bits of the kernels that used ``workspace``.

    After ``SA_DEV_PIPELINE_TIMEOUT`` a launch may have left split states behind; the workspace
    is zero-filled again here so that the next run starts from the state the kernels expect.
    """

    with torch.cuda.device(workspace.device):
        rc = int(load().sa_workspace_status(workspace.data_ptr(), stream_handle(workspace.device)))
    if rc < 0:
        raise RuntimeError(last_error())
    if rc & SA_DEV_PIPELINE_TIMEOUT:
        workspace.zero_()
    return rc


def static_status(device: torch.device) -> int:
    """Status bits collected by :func:`exact_decode_static` calls on ``device`` (then cleared)."""

    with torch.cuda.device(device):
        rc = int(load().sa_static_status(stream_handle(device)))
    if rc < 0:
        raise RuntimeError(last_error())
    return rc


def set_wait_limit_ns(limit_ns: int) -> None:
    """Process-wide default limit of the kernels' bounded waits (plans created later, one-shot calls)."""

    check(load().sa_set_wait_limit_ns(int(limit_ns)))


def seed_blocks(kv_len: int, block_size: int, sink_blocks: int, recent_blocks: int,
                middle_seed_blocks: int, block_order: str) -> list:
    if block_order not in SA_BLOCK_ORDER:
        raise ValueError("block_order must be sequential, recent_first, or sink_recent_first")
    cap = max(1, sink_blocks + recent_blocks + middle_seed_blocks)
    buf = (ctypes.c_int32 * cap)()
    n = load().sa_seed_blocks(kv_len, block_size, sink_blocks, recent_blocks, middle_seed_blocks,
                              SA_BLOCK_ORDER[block_order], buf, cap)
    if n < 0:
        raise ValueError(last_error())
    return [int(buf[i]) for i in range(n)]


def seed_token_indices(kv_len: int, block_size: int, blocks: Sequence[int]) -> torch.Tensor:
    nb = len(blocks)
    arr = (ctypes.c_int32 * max(1, nb))(*[int(b) for b in blocks])
    cap = max(1, nb * block_size)
    out = torch.empty(cap, dtype=torch.int64)
    n = load().sa_seed_token_indices(kv_len, block_size, arr, nb,
                                     ctypes.cast(out.data_ptr(), _i64p), cap)
    if n < 0:
        raise ValueError(last_error())
    return out[:n].clone()


class NativePlan:
    """Owner of one ``sa_plan_t``; ``run()`` enqueues on the device's current stream."""

    def __init__(self, handle: int, device: torch.device, keepalive: tuple) -> None:
        if not handle:
            msg = last_error()
            raise ValueError(msg or "native plan creation failed")
        self._handle = ctypes.c_void_p(handle)
        self._device = device
        self._device_index = device.index if device.index is not None else torch.cuda.current_device()
        self._keepalive = keepalive
        lib = load()
        self._run = lib.sa_plan_run
        self.kernel = int(lib.sa_plan_kernel(self._handle))
        self.kernel_name = SA_KERNEL_NAMES.get(self.kernel, "unknown")
        self.num_ctas = int(lib.sa_plan_num_ctas(self._handle))
        self.launches = int(lib.sa_plan_launches(self._handle))

    def run(self) -> None:
        # Raw handle of the device's current stream; the library selects the plan's device itself.
        rc = self._run(self._handle, _current_raw_stream(self._device_index))
        if rc:
            check(rc)

    def set_rows(self, rows: Optional[torch.Tensor]) -> None:
        """Compute only the batch rows listed in the device tensor ``rows`` (``None``: every row)."""

        if rows is None:
            check(load().sa_plan_set_rows(self._handle, None, 0, 0))
            self._rows = None
            return
        if rows.device != self._device or rows.dtype not in SA_INDEX or rows.dim() != 1 or not rows.is_contiguous():
            raise ValueError("rows must be a contiguous 1-D int32/int64 tensor on the plan's device")
        if rows.numel() == 0:  # an empty tensor has no storage: any valid device address will do
            rows = torch.zeros(1, dtype=rows.dtype, device=rows.device)[:0]
            pointer = rows.untyped_storage().data_ptr()
        else:
            pointer = rows.data_ptr()
        check(load().sa_plan_set_rows(self._handle, pointer, SA_INDEX[rows.dtype], int(rows.numel())))
        self._rows = rows  # keep the list alive: the kernel reads it at run time

    def set_wait_limit_ns(self, limit_ns: int) -> None:
        check(load().sa_plan_set_wait_limit_ns(self._handle, int(limit_ns)))

    def __del__(self) -> None:
        handle, self._handle = getattr(self, "_handle", None), None
        if handle and _LIB is not None:
            _LIB.sa_plan_destroy(handle)


def _q_strides(query: torch.Tensor) -> tuple:
    """query is [B,1,Hq,D] with D contiguous; returns (stride_b, stride_h) in elements."""

    if query.dim() != 4 or query.shape[1] != 1:
        raise ValueError("decode query must be [batch, 1, heads, dim]")
    if query.stride(3) != 1 and query.shape[3] > 1:
        raise ValueError("query head_dim must be contiguous")
    return int(query.stride(0)), int(query.stride(2))


def _kv_geometry(key: torch.Tensor, value: torch.Tensor, kv_layout: str) -> tuple:
    """Returns (kv_heads, kv_len, stride_b, stride_n, stride_h) for BNHD / BHND caches."""

    if key.shape != value.shape or key.stride() != value.stride():
        raise ValueError("key_cache and value_cache must have identical shape and strides")
    if key.stride(3) != 1 and key.shape[3] > 1:
        raise ValueError("cache head_dim must be contiguous")
    if kv_layout == "BNHD":
        return int(key.shape[2]), int(key.shape[1]), int(key.stride(0)), int(key.stride(1)), int(key.stride(2))
    if kv_layout == "BHND":
        return int(key.shape[1]), int(key.shape[2]), int(key.stride(0)), int(key.stride(2)), int(key.stride(1))
    raise ValueError("kv_layout must be BNHD or BHND")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else int(t.data_ptr())


def dynamic_default() -> bool:
    """Whether plans use the dynamic tile schedule when the caller does not say.

    ``STREAMATTN_B200_SCHEDULE=dynamic`` turns it on: up to 3 % faster on HBM-bound calls (in some runs slower),
    results within tolerance but no longer bit-identical from one launch to the next.
    """

    return os.environ.get("STREAMATTN_B200_SCHEDULE", "static").strip().lower() == "dynamic"


def _kernel_code(kernel: str, dynamic: Optional[bool]) -> int:
    if kernel not in SA_KERNEL:
        raise ValueError(f"kernel must be one of {sorted(SA_KERNEL)}")
    if dynamic is None:
        dynamic = dynamic_default()
    return SA_KERNEL[kernel] | (SA_KERNEL_FLAG_DYNAMIC if dynamic else 0)


def exact_plan(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, output: torch.Tensor,
               workspace: torch.Tensor, *, kv_layout: str = "BNHD",
               seq_lens: Optional[torch.Tensor] = None, out_state: bool = False,
               num_ctas: int = 0, kernel: str = "auto", dynamic: Optional[bool] = None) -> NativePlan:
    device = require_cuda(key, value, workspace, seq_lens, host_io=(query, output))
    if query.dtype not in SA_DTYPE or key.dtype != query.dtype or value.dtype != query.dtype:
        raise ValueError("query/key/value must share a dtype of bf16, fp16 or fp32")
    q_sb, q_sh = _q_strides(query)
    kv_heads, kv_len, sb, sn, sh = _kv_geometry(key, value, kv_layout)
    batch, _, q_heads, dim = map(int, query.shape)
    if int(key.shape[0]) != batch or int(key.shape[3]) != dim:
        raise ValueError("query/KV batch and head_dim must match")
    _check_output(output, query, out_state)
    lens_dtype = SA_INDEX[seq_lens.dtype] if seq_lens is not None else 0
    with torch.cuda.device(device):
        handle = load().sa_exact_plan_create(
            _ptr(query), _ptr(key), _ptr(value), _ptr(output), _ptr(workspace), workspace.numel(),
            _ptr(seq_lens), lens_dtype, batch, q_heads, kv_heads, dim, kv_len,
            q_sb, q_sh, sb, sn, sh, SA_DTYPE[query.dtype],
            SA_OUT_STATE if out_state else SA_OUT_FINAL, int(num_ctas), _kernel_code(kernel, dynamic),
        )
    return NativePlan(handle, device, (query, key, value, output, workspace, seq_lens))


def _check_output(output: torch.Tensor, query: torch.Tensor, out_state: bool) -> None:
    batch, _, q_heads, dim = map(int, query.shape)
    if not output.is_contiguous():
        raise ValueError("output must be contiguous")
    if out_state:
        if output.dtype != torch.float32 or tuple(output.shape) != (batch, q_heads, dim + 2):
            raise ValueError("state output must be float32 [batch, heads, dim + 2]")
    elif output.shape != query.shape or output.dtype != query.dtype:
        raise ValueError("output must match query shape and dtype")


def exact_decode_static(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, output: torch.Tensor, *,
                        kv_layout: str = "BNHD", seq_lens: Optional[torch.Tensor] = None,
                        out_state: bool = False, num_ctas: int = 0, kernel: str = "auto") -> torch.Tensor:
    """Exact decode with the library's built-in scratch (``sa_exact_decode_static``).

    For callers that cannot allocate a workspace (all device memory already
    owned by another allocator, or allocation not allowed on the calling path).
    Nothing is allocated here or in the library.  Shapes whose split states
    exceed the 2 MiB built-in array raise ``ValueError``.  Calls on one device
    share that array: issue them on one stream, never concurrently.  The first
    call on a device should happen outside any CUDA stream capture.
    """

    device = require_cuda(query, key, value, output, seq_lens)
    if query.dtype not in SA_DTYPE or key.dtype != query.dtype or value.dtype != query.dtype:
        raise ValueError("query/key/value must share a dtype of bf16, fp16 or fp32")
    q_sb, q_sh = _q_strides(query)
    kv_heads, kv_len, sb, sn, sh = _kv_geometry(key, value, kv_layout)
    batch, _, q_heads, dim = map(int, query.shape)
    if int(key.shape[0]) != batch or int(key.shape[3]) != dim:
        raise ValueError("query/KV batch and head_dim must match")
    _check_output(output, query, out_state)
    lens_dtype = SA_INDEX[seq_lens.dtype] if seq_lens is not None else 0
    with torch.cuda.device(device):
        rc = load().sa_exact_decode_static(
            _ptr(query), _ptr(key), _ptr(value), _ptr(output), _ptr(seq_lens), lens_dtype,
            batch, q_heads, kv_heads, dim, kv_len, q_sb, q_sh, sb, sn, sh, SA_DTYPE[query.dtype],
            SA_OUT_STATE if out_state else SA_OUT_FINAL, int(num_ctas), SA_KERNEL[kernel], stream_handle(device),
        )
    check(rc)
    return output


def paged_plan(query: torch.Tensor, key_pages: torch.Tensor, value_pages: torch.Tensor,
               page_table: torch.Tensor, seq_lens: torch.Tensor, output: torch.Tensor,
               workspace: torch.Tensor, *, layout: str, trace: Optional[torch.Tensor] = None,
               out_state: bool = False, num_ctas: int = 0, kernel: str = "auto",
               dynamic: Optional[bool] = None) -> NativePlan:
    device = require_cuda(key_pages, value_pages, page_table, seq_lens, workspace, trace, host_io=(query, output))
    layout = layout.upper()
    if layout not in SA_LAYOUT:
        raise ValueError("paged KV layout must be NHD or HND")
    if query.dtype not in SA_DTYPE or key_pages.dtype != query.dtype or value_pages.dtype != query.dtype:
        raise ValueError("query and paged key/value dtypes must match (bf16, fp16 or fp32)")
    tensors = (query, key_pages, value_pages, page_table, seq_lens)
    if not all(t.is_contiguous() for t in tensors):
        raise ValueError("query and paged cache tensors must be contiguous")
    batch, _, q_heads, dim = map(int, query.shape)
    num_pages = int(key_pages.shape[0])
    if layout == "NHD":
        page_size, kv_heads = int(key_pages.shape[1]), int(key_pages.shape[2])
    else:
        kv_heads, page_size = int(key_pages.shape[1]), int(key_pages.shape[2])
    if trace is not None and (trace.dtype != torch.int32 or trace.shape != page_table.shape
                              or not trace.is_contiguous()):
        raise ValueError("trace must be a contiguous int32 tensor shaped like page_table")
    _check_output(output, query, out_state)
    with torch.cuda.device(device):
        handle = load().sa_paged_plan_create(
            _ptr(query), _ptr(key_pages), _ptr(value_pages), _ptr(page_table), _ptr(seq_lens),
            _ptr(output), _ptr(workspace), workspace.numel(), _ptr(trace),
            batch, q_heads, kv_heads, dim, page_size, int(page_table.shape[1]), num_pages,
            SA_LAYOUT[layout], SA_DTYPE[query.dtype], SA_INDEX[page_table.dtype], SA_INDEX[seq_lens.dtype],
            SA_OUT_STATE if out_state else SA_OUT_FINAL, int(num_ctas), _kernel_code(kernel, dynamic),
        )
    return NativePlan(handle, device,
                      (query, key_pages, value_pages, page_table, seq_lens, output, workspace, trace))


def seed_plan(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, output: torch.Tensor,
              workspace: torch.Tensor, *, block_size: int, blocks: Sequence[int],
              kv_layout: str = "BNHD", num_ctas: int = 0, kernel: str = "auto") -> NativePlan:
    device = require_cuda(key, value, workspace, host_io=(query, output))
    if query.dtype not in SA_DTYPE or key.dtype != query.dtype or value.dtype != query.dtype:
        raise ValueError("query/key/value must share a dtype of bf16, fp16 or fp32")
    q_sb, q_sh = _q_strides(query)
    kv_heads, kv_len, sb, sn, sh = _kv_geometry(key, value, kv_layout)
    batch, _, q_heads, dim = map(int, query.shape)
    if int(key.shape[0]) != batch or int(key.shape[3]) != dim:
        raise ValueError("query/KV batch and head_dim must match")
    _check_output(output, query, False)
    nb = len(blocks)
    arr = (ctypes.c_int32 * max(1, nb))(*[int(b) for b in blocks])
    with torch.cuda.device(device):
        handle = load().sa_seed_plan_create(
            _ptr(query), _ptr(key), _ptr(value), _ptr(output), _ptr(workspace), workspace.numel(),
            batch, q_heads, kv_heads, dim, kv_len, q_sb, q_sh, sb, sn, sh, SA_DTYPE[query.dtype],
            int(block_size), arr, nb, int(num_ctas), SA_KERNEL[kernel],
        )
    return NativePlan(handle, device, (query, key, value, output, workspace))


SA_SELECTOR = {"qk_block_max": 0, "block_mean_proxy": 1}


def block_scores(query: torch.Tensor, key: torch.Tensor, *, block_size: int, selector: str,
                 kv_layout: str = "BNHD", seq_lens: Optional[torch.Tensor] = None,
                 scores: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``scores[B, Hq, ceil(N / block_size)]`` (float32) of every cache block against the query."""

    device = require_cuda(query, key, seq_lens, scores)
    if selector not in SA_SELECTOR:
        raise ValueError(f"selector must be one of {sorted(SA_SELECTOR)}")
    if query.dtype not in (torch.bfloat16, torch.float16) or key.dtype != query.dtype:
        raise ValueError("query/key must share a dtype of bf16 or fp16")
    q_sb, q_sh = _q_strides(query)
    kv_heads, kv_len, sb, sn, sh = _kv_geometry(key, key, kv_layout)
    batch, _, q_heads, dim = map(int, query.shape)
    num_blocks = -(-kv_len // int(block_size))
    if scores is None:
        scores = torch.empty(batch, q_heads, num_blocks, dtype=torch.float32, device=device)
    if tuple(scores.shape) != (batch, q_heads, num_blocks) or scores.dtype != torch.float32 or not scores.is_contiguous():
        raise ValueError("scores must be a contiguous float32 [batch, q_heads, blocks] tensor")
    lens_dtype = SA_INDEX[seq_lens.dtype] if seq_lens is not None else 0
    with torch.cuda.device(device):
        rc = load().sa_block_scores(_ptr(query), _ptr(key), _ptr(scores), _ptr(seq_lens), lens_dtype, batch, q_heads,
                                    kv_heads, dim, kv_len, q_sb, q_sh, sb, sn, sh, SA_DTYPE[query.dtype],
                                    int(block_size), SA_SELECTOR[selector], stream_handle(device))
    check(rc)
    return scores


def seed_list_length(kv_len: int, block_size: int, sink_blocks: int, recent_blocks: int,
                     middle_seed_blocks: int) -> int:
    n = int(load().sa_seed_list_length(int(kv_len), int(block_size), int(sink_blocks), int(recent_blocks),
                                       int(middle_seed_blocks)))
    if n < 0:
        raise ValueError(last_error())
    return n


def select_seed_blocks(scores: torch.Tensor, *, kv_heads: int, kv_len: int, block_size: int, sink_blocks: int,
                       recent_blocks: int, middle_seed_blocks: int, block_order: str,
                       blocks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per (row, KV head) block lists ``[B, Hkv, L]`` (int32, ascending) from block scores."""

    device = require_cuda(scores, blocks)
    if block_order not in SA_BLOCK_ORDER:
        raise ValueError("block_order must be sequential, recent_first, or sink_recent_first")
    if scores.dtype != torch.float32 or scores.dim() != 3 or not scores.is_contiguous():
        raise ValueError("scores must be a contiguous float32 [batch, q_heads, blocks] tensor")
    batch, q_heads, num_blocks = map(int, scores.shape)
    if num_blocks != -(-int(kv_len) // int(block_size)):
        raise ValueError("scores do not cover ceil(kv_len / block_size) blocks")
    length = seed_list_length(kv_len, block_size, sink_blocks, recent_blocks, middle_seed_blocks)
    if blocks is None:
        blocks = torch.empty(batch, int(kv_heads), length, dtype=torch.int32, device=device)
    if tuple(blocks.shape) != (batch, int(kv_heads), length) or blocks.dtype != torch.int32 or not blocks.is_contiguous():
        raise ValueError("blocks must be a contiguous int32 [batch, kv_heads, list length] tensor")
    with torch.cuda.device(device):
        rc = load().sa_select_seed_blocks(_ptr(scores), _ptr(blocks), batch, q_heads, int(kv_heads), int(kv_len),
                                          int(block_size), int(sink_blocks), int(recent_blocks),
                                          int(middle_seed_blocks), SA_BLOCK_ORDER[block_order], stream_handle(device))
    check(rc)
    return blocks


def seed_plan_device_blocks(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, output: torch.Tensor,
                            workspace: torch.Tensor, blocks: torch.Tensor, *, block_size: int,
                            includes_last_block: bool = True, kv_layout: str = "BNHD", num_ctas: int = 0,
                            kernel: str = "auto") -> NativePlan:
    """Seed-only plan whose per-pair block lists ``[B, Hkv, L]`` (int32) are read on the device at run time."""

    device = require_cuda(key, value, workspace, blocks, host_io=(query, output))
    if query.dtype not in SA_DTYPE or key.dtype != query.dtype or value.dtype != query.dtype:
        raise ValueError("query/key/value must share a dtype of bf16, fp16 or fp32")
    q_sb, q_sh = _q_strides(query)
    kv_heads, kv_len, sb, sn, sh = _kv_geometry(key, value, kv_layout)
    batch, _, q_heads, dim = map(int, query.shape)
    if int(key.shape[0]) != batch or int(key.shape[3]) != dim:
        raise ValueError("query/KV batch and head_dim must match")
    _check_output(output, query, False)
    if blocks.dtype != torch.int32 or blocks.dim() != 3 or tuple(blocks.shape[:2]) != (batch, kv_heads) \
            or not blocks.is_contiguous():
        raise ValueError("blocks must be a contiguous int32 [batch, kv_heads, list length] tensor")
    with torch.cuda.device(device):
        handle = load().sa_seed_plan_create_device(
            _ptr(query), _ptr(key), _ptr(value), _ptr(output), _ptr(workspace), workspace.numel(),
            batch, q_heads, kv_heads, dim, kv_len, q_sb, q_sh, sb, sn, sh, SA_DTYPE[query.dtype],
            int(block_size), _ptr(blocks), int(blocks.shape[2]), int(bool(includes_last_block)), int(num_ctas),
            SA_KERNEL[kernel],
        )
    return NativePlan(handle, device, (query, key, value, output, workspace, blocks))


def merge_states(states: torch.Tensor, output: torch.Tensor) -> torch.Tensor:
    """states [parts, rows, D+2] float32 -> output [rows, D] (any supported dtype)."""

    device = require_cuda(states, host_io=(output,))
    if states.dtype != torch.float32 or states.dim() != 3 or not states.is_contiguous():
        raise ValueError("states must be a contiguous float32 [parts, rows, dim + 2] tensor")
    parts, rows, width = map(int, states.shape)
    dim = width - 2
    if output.dtype not in SA_DTYPE or output.numel() != rows * dim or not output.is_contiguous():
        raise ValueError("output must be contiguous with rows * dim elements")
    with torch.cuda.device(device):
        rc = load().sa_merge_states(states.data_ptr(), parts, rows, dim, output.data_ptr(),
                                    SA_DTYPE[output.dtype], stream_handle(device))
    check(rc)
    return output


def cp_exchange_bytes(world_size: int, rows: int, head_dim: int) -> int:
    n = int(load().sa_cp_exchange_bytes(world_size, rows, head_dim))
    if n == 0:
        raise ValueError(last_error())
    return n


class PeerExchange:
    """Bound ``sa_cp_exchange_merge`` call: peer addresses fixed, step counter kept here."""

    def __init__(self, local_state: torch.Tensor, peer_buffer_ptrs: Sequence[int], rank: int,
                 output: torch.Tensor) -> None:
        device = require_cuda(local_state, host_io=(output,))
        if local_state.dtype != torch.float32 or local_state.dim() != 3 or not local_state.is_contiguous():
            raise ValueError("local_state must be a contiguous float32 [batch, heads, dim + 2] tensor")
        self.world = len(peer_buffer_ptrs)
        self.rank = int(rank)
        self.rows = int(local_state.shape[0] * local_state.shape[1])
        self.dim = int(local_state.shape[2]) - 2
        if output.numel() != self.rows * self.dim or not output.is_contiguous() or output.dtype not in SA_DTYPE:
            raise ValueError("output must be contiguous with rows * dim elements")
        self._ptrs = (ctypes.c_uint64 * self.world)(*[int(x) for x in peer_buffer_ptrs])
        self._local_buffer = int(peer_buffer_ptrs[self.rank])
        self._state = local_state
        self._out = output
        self._device_index = device.index if device.index is not None else torch.cuda.current_device()
        self._fn = load().sa_cp_exchange_merge
        self._dtype = SA_DTYPE[output.dtype]
        self.step = 0

    def run(self) -> None:
        self.step += 1
        rc = self._fn(self._state.data_ptr(), self._ptrs, self.world, self.rank, self.step, self.rows, self.dim,
                      self._out.data_ptr(), self._dtype, _current_raw_stream(self._device_index))
        if rc:
            check(rc)

    def status(self) -> int:
        rc = int(load().sa_cp_exchange_status(self._local_buffer, self.world, self.rows, self.dim,
                                              _current_raw_stream(self._device_index)))
        if rc < 0:
            raise RuntimeError(last_error())
        return rc


def cp_fused_bytes(world_size: int, batch: int, q_heads: int, kv_heads: int, head_dim: int) -> int:
    n = int(load().sa_cp_fused_bytes(world_size, batch, q_heads, kv_heads, head_dim))
    if n == 0:
        raise ValueError(last_error())
    return n


def cp_fused_plan(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, output: torch.Tensor,
                  workspace: torch.Tensor, peer_buffer_ptrs: Sequence[int], rank: int, *,
                  kv_layout: str = "BHND", num_ctas: int = 0) -> NativePlan:
    """One-launch context-parallel step: shard decode + peer exchange + cross-rank merge.

    ``query`` and ``output`` may be pinned host tensors, as in :func:`exact_plan`.
    """

    device = require_cuda(key, value, workspace, host_io=(query, output))
    if query.dtype not in SA_DTYPE or key.dtype != query.dtype or value.dtype != query.dtype:
        raise ValueError("query/key/value must share a dtype of bf16 or fp16")
    q_sb, q_sh = _q_strides(query)
    kv_heads, kv_len, sb, sn, sh = _kv_geometry(key, value, kv_layout)
    batch, _, q_heads, dim = map(int, query.shape)
    _check_output(output, query, False)
    world = len(peer_buffer_ptrs)
    ptrs = (ctypes.c_uint64 * world)(*[int(x) for x in peer_buffer_ptrs])
    with torch.cuda.device(device):
        handle = load().sa_cp_fused_plan_create(
            _ptr(query), _ptr(key), _ptr(value), _ptr(output), _ptr(workspace), workspace.numel(),
            batch, q_heads, kv_heads, dim, kv_len, q_sb, q_sh, sb, sn, sh, SA_DTYPE[query.dtype],
            int(num_ctas), ptrs, world, int(rank),
        )
    return NativePlan(handle, device, (query, key, value, output, workspace))
