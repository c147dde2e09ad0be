"""Context-parallel plumbing on CPU: world_size-2 gloo ranks.

The product's sharding rule and state all-gather run for real (over gloo);
the per-shard states and the final merge come from the CPU oracle, standing
in for the kernels, so the test needs no GPU.
"""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results) -> None:
    for path in (str(ROOT), str(ROOT / "tests" / "golden")):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import cases
        from oracle import cpu_oracle
        from streamattn_b200.context_parallel import gather_states, shard_bounds, shard_requests

        case = cases.EXACT_CASES["g4_d128_n257"]
        q, k, v = cases.exact_inputs(case)
        lo, hi = shard_bounds(case.kv_len, world, rank)
        _, local = cpu_oracle.exact_decode(q, k, v, token_range=(lo, hi), return_state=True)
        gathered = gather_states(local)
        assert tuple(gathered.shape) == (world, case.batch, case.q_heads, case.dim + 2)
        assert torch.equal(gathered[rank], local)
        merged = cpu_oracle.merge_states(gathered.view(world, -1, case.dim + 2), log2_domain=False)
        want = cpu_oracle.exact_decode(q, k, v)
        torch.testing.assert_close(merged.view_as(want), want, atol=2e-6, rtol=1e-5)
        rlo, rhi = shard_requests(7, world, rank)
        results[rank] = (lo, hi, rlo, rhi)
    finally:
        dist.destroy_process_group()


def test_shard_gather_merge_world2():
    world = 2
    manager = mp.get_context("spawn").Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert results[0][:2] == (0, 128) and results[1][:2] == (128, 257)
    assert results[0][2:] == (0, 3) and results[1][2:] == (3, 7)


def test_shard_bounds_cover_the_sequence():
    from streamattn_b200.context_parallel import shard_bounds

    for n in (1, 7, 1000, 1048576):
        for world in (1, 2, 3, 8):
            pieces = [shard_bounds(n, world, r) for r in range(world)]
            assert pieces[0][0] == 0 and pieces[-1][1] == n
            assert all(pieces[i][1] == pieces[i + 1][0] for i in range(world - 1))
