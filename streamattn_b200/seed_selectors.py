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

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

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


# ---------------------------------------------------------------------------------------------
# Run-time selection of the middle seed blocks (reference seed_selectors.py:17-73, 274-396)
# ---------------------------------------------------------------------------------------------

DEFAULT_SELECTOR_PROFILES = ("fixed_policy",)
# Profiles that need nothing but q and K and therefore run on the device.  The reference also
# lists support-key proxies (its diagnostics) and oracles that need labels; they are not provided.
SELECTOR_PROFILES = frozenset({"fixed_policy", "qk_block_max", "block_mean_proxy"})


def parse_selector_profiles(text: str) -> List[str]:
    """Comma / semicolon separated profile names; empty text means the default profile."""

    profiles = [part.strip() for part in text.replace(";", ",").split(",") if part.strip()]
    if not profiles:
        profiles = list(DEFAULT_SELECTOR_PROFILES)
    unknown = sorted(set(profiles) - SELECTOR_PROFILES)
    if unknown:
        raise ValueError(f"unknown selector profiles: {unknown}; supported={sorted(SELECTOR_PROFILES)}")
    return profiles


@dataclass(frozen=True)
class SeedBlockSelection:
    selector: str
    selected_blocks: List[int]
    middle_blocks: List[int]
    base_blocks: List[int]
    fixed_blocks: List[int]
    cost: Dict[str, float]


def selector_cost_estimate(selector: str, *, seq_len: int, block_size: int) -> Dict[str, float]:
    """Bytes-per-key ratio of a selector's scoring pass (1.0 = it reads every key once)."""

    blocks = max(1, -(-int(seq_len) // int(block_size)))
    reads_all_keys = selector in ("qk_block_max", "block_mean_proxy")
    return {"num_blocks": float(blocks), "key_read_ratio": 1.0 if reads_all_keys else 0.0}


def select_seed_blocks_by_profile(*, q: torch.Tensor, k: torch.Tensor, policy, selector: str) -> SeedBlockSelection:
    """Seed blocks of ONE (row, head): ``q`` is ``[D]``, ``k`` is ``[N, D]`` (reference signature).

    ``fixed_policy`` is the policy's own rule.  The scoring profiles run the block-score and
    selection kernels on the device (CUDA tensors required) and read the short result back; a
    decode loop should use :class:`DynamicSeedDecodePlan`, which keeps the list on the device.
    """

    if selector not in SELECTOR_PROFILES:
        raise ValueError(f"unknown selector profile: {selector}")
    seq_len, block_size = int(k.shape[0]), int(policy.block_size)
    rule = dict(seq_len=seq_len, block_size=block_size, sink_blocks=int(policy.sink_blocks),
                recent_blocks=int(policy.recent_blocks), middle_seed_blocks=int(policy.middle_seed_blocks),
                block_order=str(policy.block_order))
    base_blocks = policy_seed_blocks(**rule, include_middle=False)
    fixed_blocks = policy_seed_blocks(**rule, include_middle=True)
    if selector == "fixed_policy":
        selected = list(fixed_blocks)
    else:
        native.require_cuda(q, k)
        query = q.reshape(1, 1, 1, -1)
        key = k.unsqueeze(0).unsqueeze(2)                                   # [1, N, 1, D]
        scores = native.block_scores(query, key, block_size=block_size, selector=selector)
        chosen = native.select_seed_blocks(scores, kv_heads=1, kv_len=seq_len, block_size=block_size,
                                           sink_blocks=rule["sink_blocks"], recent_blocks=rule["recent_blocks"],
                                           middle_seed_blocks=rule["middle_seed_blocks"],
                                           block_order=rule["block_order"])
        picked = sorted(set(chosen.view(-1).tolist()))
        base = set(base_blocks)
        # base blocks first (policy order), then the scored blocks, best first
        ranked = scores.view(-1).tolist()
        middle = sorted((b for b in picked if b not in base), key=lambda b: (-ranked[b], b))
        selected = list(base_blocks) + middle
    base = set(base_blocks)
    return SeedBlockSelection(selector=selector, selected_blocks=[int(b) for b in selected],
                              middle_blocks=[int(b) for b in selected if b not in base],
                              base_blocks=[int(b) for b in base_blocks], fixed_blocks=[int(b) for b in fixed_blocks],
                              cost=selector_cost_estimate(selector, seq_len=seq_len, block_size=block_size))


class DynamicSeedDecodePlan:
    """Seed-only decode whose middle blocks are re-selected on the device at every step.

    Three launches per ``run()`` on the current stream, no host synchronisation and no
    allocation: block scores of the K cache against the bound query, per (row, KV head) selection
    (sink and recent blocks kept, the best ``middle_seed_blocks`` others added), and the seed-only
    decode reading each pair's list from device memory.  ``policy`` supplies ``block_size``,
    ``sink_blocks``, ``recent_blocks``, ``middle_seed_blocks`` and ``block_order``; it needs at
    least one recent block (every list then ends with the cache's last block).
    """

    def __init__(self, query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor, policy, *,
                 selector: str = "qk_block_max", kv_layout: str = "BNHD", output: Optional[torch.Tensor] = None,
                 num_ctas: int = 0) -> None:
        if selector not in native.SA_SELECTOR:
            raise ValueError(f"selector must be one of {sorted(native.SA_SELECTOR)}")
        if int(policy.recent_blocks) < 1:
            raise ValueError("run-time seed selection needs a policy with at least one recent block")
        device = native.require_cuda(query, key_cache, value_cache)
        batch, _, q_heads, dim = (int(x) for x in query.shape)
        kv_heads, kv_len, *_ = native._kv_geometry(key_cache, value_cache, kv_layout)
        self.query, self.key_cache, self.value_cache = query, key_cache, value_cache
        self.policy, self.selector, self.kv_layout = policy, selector, kv_layout
        self.output = torch.empty_like(query) if output is None else output
        self._rule = dict(kv_heads=kv_heads, kv_len=kv_len, block_size=int(policy.block_size),
                          sink_blocks=int(policy.sink_blocks), recent_blocks=int(policy.recent_blocks),
                          middle_seed_blocks=int(policy.middle_seed_blocks), block_order=str(policy.block_order))
        blocks_total = -(-kv_len // int(policy.block_size))
        length = native.seed_list_length(kv_len, policy.block_size, policy.sink_blocks, policy.recent_blocks,
                                         policy.middle_seed_blocks)
        self.scores = torch.empty(batch, q_heads, blocks_total, dtype=torch.float32, device=device)
        self.blocks = torch.zeros(batch, kv_heads, length, dtype=torch.int32, device=device)
        self.workspace = native.new_workspace(device, batch, q_heads, kv_heads, dim, num_ctas)
        self._plan = native.seed_plan_device_blocks(query, key_cache, value_cache, self.output, self.workspace,
                                                    self.blocks, block_size=int(policy.block_size),
                                                    includes_last_block=True, kv_layout=kv_layout, num_ctas=num_ctas)
        self.launches_per_run = 2 + self._plan.launches

    def select(self) -> torch.Tensor:
        """Score and select only; returns the device block lists ``[B, Hkv, L]``."""

        native.block_scores(self.query, self.key_cache, block_size=self._rule["block_size"], selector=self.selector,
                            kv_layout=self.kv_layout, scores=self.scores)
        return native.select_seed_blocks(self.scores, blocks=self.blocks, **self._rule)

    def run(self) -> torch.Tensor:
        self.select()
        self._plan.run()
        return self.output

    def device_status(self) -> int:
        return native.workspace_status(self.workspace)
