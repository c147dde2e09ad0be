"""Seed block / token set definition of seed-only decode.

The integer rule lives in the native library (``sa_seed_blocks`` and
``sa_seed_token_indices``), which the kernel launch itself uses, so the index
set a caller inspects here is the one the GPU reads.  The rule restates the
reference's ``policy_seed_blocks`` / ``seed_indices`` /
``seed_token_indices_from_blocks`` (``stream_attention/seed_selectors.py:77-173``),
which equal the in-kernel block rule of
``stream_attention/kernels/gate0_seed_only_triton.py:64-79``.
"""

from __future__ import annotations

from typing import List, Sequence

import torch

from . import native


def policy_seed_blocks(*, seq_len: int, block_size: int, sink_blocks: int, recent_blocks: int,
                       middle_seed_blocks: int, block_order: str, include_middle: bool = True) -> List[int]:
    """Seed blocks in the reference's order: sink, recent, then middle blocks.

    ``nb = ceil(seq_len / block_size)``; sink = ``[0, sink)``, recent =
    ``[nb - recent, nb)``, middle = ``sink + i`` (sequential) or
    ``nb - recent - 1 - i`` (recent_first / sink_recent_first); blocks outside
    ``[0, nb)`` and duplicates are dropped.
    """

    return native.seed_blocks(int(seq_len), int(block_size), int(sink_blocks), int(recent_blocks),
                              int(middle_seed_blocks) if include_middle else 0, block_order)


def seed_token_indices_from_blocks(*, seq_len: int, block_size: int, blocks: Sequence[int],
                                   device: torch.device = torch.device("cpu")) -> torch.Tensor:
    """Sorted unique token indices covered by ``blocks`` (clipped to ``seq_len``)."""

    return native.seed_token_indices(int(seq_len), int(block_size), list(blocks)).to(device)


def seed_indices(*, seq_len: int, block_size: int, sink_blocks: int, recent_blocks: int,
                 middle_seed_blocks: int, block_order: str) -> torch.Tensor:
    """Token index set of a seed policy (int64, ascending)."""

    blocks = policy_seed_blocks(seq_len=seq_len, block_size=block_size, sink_blocks=sink_blocks,
                                recent_blocks=recent_blocks, middle_seed_blocks=middle_seed_blocks,
                                block_order=block_order)
    return seed_token_indices_from_blocks(seq_len=seq_len, block_size=block_size, blocks=blocks)
