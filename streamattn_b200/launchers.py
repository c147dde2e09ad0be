"""Reference-named kernel launchers on the sm_100a kernels.

The reference exposes its Triton kernels through launcher functions that model adapters and
benchmark scripts call directly.  The same names and argument meanings are kept here; every
launcher validates like the reference, builds a one-shot plan and runs it on the current
stream.  Launch hints that only make sense for Triton (``num_warps``, ``num_stages``, tile
sizes, a split-K ``workspace`` dict) are accepted and ignored - steady-state callers should
hold a plan (``ExactDecodePlan``, ``PagedExactDecodePlan``, the engine) instead.

================================================  ============================================
launcher                                          reference
================================================  ============================================
``paged_exact_decode_triton_forward_out``         kernels/paged_exact_triton.py:193-306
``make_paged_exact_workspace``                    kernels/paged_exact_triton.py:309-331
``exact_decode_attention_rows_triton_forward_     kernels/gate0_exact_refresh_triton.py:266-344
out_bhnd``
``gate0_seed_only_attention_triton_forward_out``  kernels/gate0_seed_only_triton.py:1458-1537
``..._forward_out_prechecked``                    kernels/gate0_seed_only_triton.py:2322-2378
``..._forward_out_dynamic_n[_bhnd]``              kernels/gate0_seed_only_triton.py:1540-1720
``qwen_o_proj_triton_forward``                    kernels/qwen_o_proj_triton.py:77-145
================================================  ============================================
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from . import native
from .exact import exact_decode_attention_rows_forward_out_bhnd
from .o_proj import qwen_o_proj_forward
from .paged import PagedExactDecodePlan, PagedKVCache

# The reference modules carry this flag; nothing here needs Triton.
TRITON_AVAILABLE = False


def make_paged_exact_workspace(*, batch: int, heads: int, splits: int, dim: int,
                               device: torch.device) -> Dict[str, torch.Tensor]:
    """Workspace record of the reference's Triton path.

    The sm_100a kernels keep their split states in a private workspace that the plan allocates,
    so this record only carries that buffer; its key names the reference's tensors replace.
    """

    if min(batch, heads, splits, dim) <= 0:
        raise ValueError("workspace dimensions must be positive")
    return {"sm100_workspace": native.new_workspace(torch.device(device), batch, heads, 1, dim, 0)}


def paged_exact_decode_triton_forward_out(query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                                          page_table: torch.Tensor, sequence_lengths: torch.Tensor,
                                          output: torch.Tensor, *, layout: str, splits: int,
                                          workspace: Optional[Dict[str, torch.Tensor]] = None,
                                          **_launch_hints) -> torch.Tensor:
    """Exact M=1 decode directly over a paged KV cache, into ``output``."""

    tensors = (query, key_cache, value_cache, page_table, sequence_lengths, output)
    if not all(t.is_cuda for t in tensors):
        raise RuntimeError("paged exact decode requires CUDA tensors")
    if splits <= 0:
        raise ValueError("splits must be positive")
    del workspace
    cache = PagedKVCache(key=key_cache, value=value_cache, page_table=page_table,
                         sequence_lengths=sequence_lengths, layout=layout)
    splits = min(int(splits), cache.max_pages_per_request)
    PagedExactDecodePlan.build(query, cache, output=output, splits=splits, validate_metadata=False).run()
    return output


def exact_decode_attention_rows_triton_forward_out_bhnd(query, key, value, output, cache_position, *,
                                                        row_indices=None, **_launch_hints) -> torch.Tensor:
    """Exact decode of selected batch rows over a BHND cache prefix (see :mod:`streamattn_b200.exact`)."""

    return exact_decode_attention_rows_forward_out_bhnd(query, key, value, output, cache_position,
                                                        row_indices=row_indices)


def _seed_checks(query, key, value, output, block_size, sink_blocks, recent_blocks, middle_seed_blocks, what):
    if not all(t.is_cuda for t in (query, key, value, output)):
        raise RuntimeError(f"{what} requires CUDA tensors")
    if query.dim() != 4 or key.dim() != 4 or value.dim() != 4:
        raise ValueError("query, key, and value must be [batch, seq, heads, dim]")
    if query.shape[1] != 1:
        raise ValueError("seed-only Gate-0 only supports query_len == 1")
    if output.shape != query.shape:
        raise ValueError("output must have the same shape as query")
    if not output.is_contiguous():
        raise ValueError("output must be contiguous")
    if key.shape != value.shape:
        raise ValueError("key and value must have the same shape")
    if block_size <= 0:
        raise ValueError("block_size must be positive")
    if sink_blocks < 0 or recent_blocks < 0 or middle_seed_blocks < 0:
        raise ValueError("seed block counts must be non-negative")


def _seed_launch(query, key, value, output, kv_layout, block_size, sink_blocks, recent_blocks, middle_seed_blocks,
                 block_order):
    kv_len = int(key.shape[1] if kv_layout == "BNHD" else key.shape[2])
    kv_heads = int(key.shape[2] if kv_layout == "BNHD" else key.shape[1])
    if query.shape[0] != key.shape[0] or query.shape[3] != key.shape[3]:
        raise ValueError("query/key/value must have matching batch and dim")
    if query.shape[2] % kv_heads != 0:
        raise ValueError("query heads must be a multiple of KV heads")
    blocks = native.seed_blocks(kv_len, int(block_size), int(sink_blocks), int(recent_blocks),
                                int(middle_seed_blocks), block_order)
    batch, _, q_heads, dim = (int(x) for x in query.shape)
    workspace = native.new_workspace(query.device, batch, q_heads, kv_heads, dim)
    native.seed_plan(query, key, value, output, workspace, block_size=int(block_size), blocks=blocks,
                     kv_layout=kv_layout).run()
    return output


def gate0_seed_only_attention_triton_forward_out(query, key, value, output, *, block_size: int = 32,
                                                 sink_blocks: int = 2, recent_blocks: int = 2,
                                                 middle_seed_blocks: int = 8, block_order: str = "recent_first",
                                                 **_launch_hints) -> torch.Tensor:
    """Seed-only decode (``key``/``value`` ``[B, N, Hkv, D]``) into a caller-provided output."""

    _seed_checks(query, key, value, output, block_size, sink_blocks, recent_blocks, middle_seed_blocks,
                 "gate0_seed_only_attention_triton_forward_out")
    return _seed_launch(query, key, value, output, "BNHD", block_size, sink_blocks, recent_blocks,
                        middle_seed_blocks, block_order)


# The reference has a variant that skips the argument checks and one that keeps the cache length
# a run-time scalar to avoid Triton recompilation; neither distinction exists here.
gate0_seed_only_attention_triton_forward_out_prechecked = gate0_seed_only_attention_triton_forward_out
gate0_seed_only_attention_triton_forward_out_dynamic_n = gate0_seed_only_attention_triton_forward_out


def gate0_seed_only_attention_triton_forward_out_dynamic_n_bhnd(query, key, value, output, *, block_size: int = 32,
                                                                sink_blocks: int = 2, recent_blocks: int = 2,
                                                                middle_seed_blocks: int = 8,
                                                                block_order: str = "recent_first",
                                                                **_launch_hints) -> torch.Tensor:
    """Seed-only decode against the head-major cache layout ``[B, Hkv, N, D]`` (no transpose)."""

    _seed_checks(query, key, value, output, block_size, sink_blocks, recent_blocks, middle_seed_blocks,
                 "gate0_seed_only_attention_triton_forward_out_dynamic_n_bhnd")
    return _seed_launch(query, key, value, output, "BHND", block_size, sink_blocks, recent_blocks,
                        middle_seed_blocks, block_order)


def qwen_o_proj_triton_forward(attn_output, weight, bias=None, **_launch_hints) -> torch.Tensor:
    """``F.linear`` for ``[batch, 1, hidden]`` decode tensors (see :mod:`streamattn_b200.o_proj`)."""

    return qwen_o_proj_forward(attn_output, weight, bias)


__all__ = [name for name in dir() if not name.startswith("_") and name not in
           ("Dict", "Optional", "torch", "native", "annotations")]
