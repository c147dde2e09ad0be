"""Context-parallel decode on GPUs: the fused peer-store exchange and the NCCL path.

With one GPU the exchange kernel is exercised at world size 1 (its own buffer is the only
peer); with two or more GPUs real ranks are spawned (NCCL rendezvous on 127.0.0.1, symmetric memory
for the peer exchange, plain peer stores only).
"""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
from oracle import cpu_oracle

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _close(got, want):
    diff = (got.float().cpu() - want.float()).abs()
    assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3, (float(diff.max()), float(diff.mean()))


def _worker(rank: int, world: int, port: int, exchange: str, results) -> None:
    for path in (str(ROOT), str(ROOT / "tests" / "golden")):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import cases as _cases
        from oracle import cpu_oracle as _oracle
        from streamattn_b200.context_parallel import ContextParallelExactDecode, shard_bounds

        case = _cases.EXACT_CASES["g4_d128_n257"]
        q, k, v = (t.bfloat16() for t in _cases.exact_inputs(case))
        want = _oracle.exact_decode(q, k, v)
        lo, hi = shard_bounds(case.kv_len, world, rank)
        kh = k[:, lo:hi].permute(0, 2, 1, 3).contiguous().to(dev)
        vh = v[:, lo:hi].permute(0, 2, 1, 3).contiguous().to(dev)
        cp = ContextParallelExactDecode(q.to(dev), kh, vh, kv_layout="BHND", exchange=exchange)
        errs = []
        for step in range(4):  # several steps: both parities of the double buffer, flags re-armed
            out = cp.run()
            torch.cuda.synchronize(dev)
            errs.append(float((out.float().cpu() - want).abs().max()))
        results[rank] = (cp.exchange, cp.device_status(), max(errs))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["fused", "peer", "nccl"])
def test_context_parallel_two_ranks(exchange):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    results = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), exchange, results), nprocs=world, join=True)
    for rank in range(world):
        used, status, err = results[rank]
        assert used == exchange and status == 0 and err <= 2e-2, (rank, results[rank])


def test_peer_exchange_kernel_world_size_one():
    """One rank is its own only peer: the kernel raises its flag before it waits for it, so
    nothing here waits on another launch (kernels that wait on each other must never share a GPU)."""

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; refusing to skip")
    dev = torch.device("cuda:0")
    case = cases.EXACT_CASES["g4_d128_n257"]
    q, k, v = (t.bfloat16() for t in cases.exact_inputs(case))
    want = cpu_oracle.exact_decode(q, k, v)

    # World size 1 through the public class (process group of one rank).
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(_free_port())
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    try:
        from streamattn_b200.context_parallel import ContextParallelExactDecode

        kh = k.permute(0, 2, 1, 3).contiguous().to(dev)
        vh = v.permute(0, 2, 1, 3).contiguous().to(dev)
        for exchange, launches in (("peer", 2), ("fused", 1)):
            cp = ContextParallelExactDecode(q.to(dev), kh, vh, exchange=exchange)
            assert cp.exchange == exchange and cp.launches_per_run == launches
            for _ in range(3):
                _close(cp.run(), want)
            assert cp.device_status() == 0
    finally:
        dist.destroy_process_group()
