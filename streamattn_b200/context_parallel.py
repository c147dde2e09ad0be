"""Multi-GPU decode: context-parallel exact decode and request sharding.

The reference has no multi-GPU decode path.  Softmax attention over a token
partition is exactly mergeable from per-shard ``(m, l, o)`` states, so a long
KV sequence can be split across the GPUs of one box:

* rank r owns tokens ``[r*N/G, (r+1)*N/G)`` of every (row, KV head);
* each rank runs the exact kernel on its shard and emits the split state
  ``[B, Hq, D+2]`` (float32) instead of a normalised output;
* the G states are brought into each rank's own memory and merged exactly, on
  every rank.  Three exchanges are provided: ``"fused"`` - the whole step is ONE launch: the
  CTA that completes a (row, KV head) pair stores its state rows to every rank, raises the
  pair's flag, waits (bounded) for the other ranks' flags and merges; ``"peer"`` - one extra kernel that stores
  the state into every rank's symmetric-memory buffer with plain peer stores
  over NVLink, raises a flag, waits (bounded) for all ranks' flags and merges;
  and ``"nccl"`` - ``all_gather_into_tensor`` followed by the merge kernel.

The exchange is ``B*Hq*(D+2)*4`` bytes per rank (16.6 KB for one row of 32
heads of 128), so it is latency- not bandwidth-bound.  Batch-parallel shapes
shard by request and need no collective (:func:`shard_requests`).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import native


def shard_bounds(kv_len: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Token range ``[lo, hi)`` of ``rank`` when ``kv_len`` tokens are split evenly."""

    if kv_len < 0 or world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("bad shard arguments")
    return kv_len * rank // world_size, kv_len * (rank + 1) // world_size


def shard_requests(batch: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Row range ``[lo, hi)`` of ``rank`` for batch-parallel decode (no collective)."""

    return shard_bounds(batch, world_size, rank)


def gather_states(local_state: torch.Tensor, gathered: Optional[torch.Tensor] = None,
                  group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gather the per-rank split states into ``[world, B, Hq, D+2]`` on every rank."""

    world = dist.get_world_size(group)
    if gathered is None:
        gathered = local_state.new_empty((world, *local_state.shape))
    if tuple(gathered.shape) != (world, *local_state.shape) or not gathered.is_contiguous():
        raise ValueError("gathered must be a contiguous [world, *local_state.shape] tensor")
    # Concatenation form (world*B leading rows): accepted by both the NCCL and the gloo backend.
    flat = gathered.view(world * local_state.shape[0], *local_state.shape[1:])
    dist.all_gather_into_tensor(flat, local_state.contiguous(), group=group)
    return gathered


def _peer_exchange_buffers(nbytes: int, device: torch.device, group: Optional[dist.ProcessGroup]):
    """Allocate this rank's exchange buffer in symmetric memory; returns (buffer, peer addresses)."""

    if dist.get_world_size(group) == 1:
        buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        return buf, [int(buf.data_ptr())]
    import torch.distributed._symmetric_memory as symm_mem

    buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
    handle = symm_mem.rendezvous(buf, group if group is not None else dist.group.WORLD)
    buf.zero_()
    torch.cuda.synchronize(device)
    dist.barrier(group)  # nobody may store into a buffer that is not yet cleared
    ptrs = [int(x) for x in handle.buffer_ptrs]
    return (buf, handle), ptrs


class ContextParallelExactDecode:
    """Exact decode over a KV sequence sharded across the ranks of a process group.

    Bound once to this rank's shard; ``run()`` launches the local kernel and the
    exchange + merge on the current stream and allocates nothing.  ``query`` and
    ``output`` may be pinned host tensors: the kernels then read the query and
    write the merged result across PCIe themselves, so a host-driven step is one
    launch and one wait with no separate copies.
    ``key_shard`` / ``value_shard`` hold this rank's tokens only, in ``kv_layout``
    (``"BHND"`` head-major by default).  ``shard_lens`` optionally gives per-row
    valid token counts inside the shard (ragged rows).  ``exchange`` selects how
    the per-rank states meet: ``"fused"`` (decode + exchange + merge in one launch, up
    to 8 ranks), ``"peer"`` (a separate peer-store exchange + merge kernel), ``"nccl"``
    (all-gather then merge) or ``"auto"`` (the first of these that can be set up on
    every rank; all ranks take the same decision).
    """

    def __init__(self, query: torch.Tensor, key_shard: torch.Tensor, value_shard: torch.Tensor, *,
                 kv_layout: str = "BHND", group: Optional[dist.ProcessGroup] = None,
                 output: Optional[torch.Tensor] = None, shard_lens: Optional[torch.Tensor] = None,
                 num_ctas: int = 0, kernel: str = "auto", exchange: str = "auto") -> None:
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised for context-parallel decode")
        if exchange not in ("auto", "fused", "peer", "nccl"):
            raise ValueError("exchange must be auto, fused, peer or nccl")
        device = native.require_cuda(key_shard, value_shard, host_io=(query, output))
        self.group = group
        self.world_size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.query = query
        batch, _, q_heads, dim = (int(x) for x in query.shape)
        kv_heads = int(key_shard.shape[1] if kv_layout == "BHND" else key_shard.shape[2])
        self.output = torch.empty(query.shape, dtype=query.dtype, device=device) if output is None else output
        self.local_state = torch.empty(batch, q_heads, dim + 2, dtype=torch.float32, device=device)
        self.workspace = native.new_workspace(device, batch, q_heads, kv_heads, dim, num_ctas)
        self._plan = native.exact_plan(query, key_shard, value_shard, self.local_state, self.workspace,
                                       kv_layout=kv_layout, seq_lens=shard_lens, out_state=True,
                                       num_ctas=num_ctas, kernel=kernel)
        self._rows = batch * q_heads
        self._dim = dim
        self._peer: Optional[native.PeerExchange] = None
        self._fused: Optional[native.NativePlan] = None
        self._keepalive = None
        self.exchange_fallback_reason: Optional[str] = None

        def agree(ok: bool) -> bool:
            """All ranks must use the same exchange: a mode is taken only if it works everywhere."""

            if self.world_size == 1:
                return ok
            flag = torch.tensor([1 if ok else 0], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
            return bool(int(flag.item()))

        def attempt(mode: str, build) -> bool:
            ok = True
            try:
                build()
            except Exception as exc:  # symmetric memory unavailable, shape not covered, ...
                if exchange == mode:
                    raise
                ok = False
                self.exchange_fallback_reason = f"{mode}: {type(exc).__name__}: {exc}"
            if not agree(ok):
                self._fused = self._peer = self._keepalive = None
                return False
            return True

        def build_fused() -> None:
            if shard_lens is not None:
                raise ValueError("the fused exchange needs a uniform shard length")
            nbytes = native.cp_fused_bytes(self.world_size, batch, q_heads, kv_heads, dim)
            keep, ptrs = _peer_exchange_buffers(nbytes, device, group)
            self._fused = native.cp_fused_plan(query, key_shard, value_shard, self.output, self.workspace, ptrs,
                                               self.rank, kv_layout=kv_layout, num_ctas=num_ctas)
            self._keepalive = keep

        def build_peer() -> None:
            nbytes = native.cp_exchange_bytes(self.world_size, self._rows, dim)
            keep, ptrs = _peer_exchange_buffers(nbytes, device, group)
            self._peer = native.PeerExchange(self.local_state, ptrs, self.rank, self.output)
            self._keepalive = keep

        self.exchange = "nccl"
        if exchange in ("auto", "fused") and self.world_size <= 8 and kernel != "generic" and attempt("fused", build_fused):
            self.exchange = "fused"
        elif exchange in ("auto", "peer") and self.world_size <= 16 and attempt("peer", build_peer):
            self.exchange = "peer"
        if self.exchange == "nccl":
            self.gathered = torch.empty(self.world_size, batch, q_heads, dim + 2, dtype=torch.float32,
                                        device=device)
        # The exchange kernels wait for their peers for at most the wait limit (2 s by default).
        # Run the shard kernel once here - it loads the kernel image, the slow part of a first
        # launch - and line the ranks up, so that the first exchanged step starts everywhere at
        # about the same time.  Results of run() are valid only while device_status() stays 0.
        self._plan.run()
        torch.cuda.synchronize(device)
        if self.world_size > 1:
            dist.barrier(group)

    @property
    def kernel_name(self) -> str:
        return self._plan.kernel_name

    @property
    def exchange_bytes_per_rank(self) -> int:
        return self.local_state.numel() * 4

    @property
    def launches_per_run(self) -> int:
        """Kernels of this package per run (the NCCL collective is not counted)."""

        return 1 if self._fused is not None else self._plan.launches + 1

    def device_status(self) -> int:
        """Synchronise and return the status bits of the local kernel and the exchange (0 = clean)."""

        status = native.workspace_status(self.workspace)
        if self._peer is not None:
            status |= self._peer.status()
        return status

    def run_local(self) -> torch.Tensor:
        """Only the local shard kernel; returns this rank's state."""

        self._plan.run()
        return self.local_state

    def run(self) -> torch.Tensor:
        if self._fused is not None:
            self._fused.run()
            return self.output
        self._plan.run()
        if self._peer is not None:
            self._peer.run()
            return self.output
        if self.world_size == 1:
            states = self.local_state.view(1, self._rows, self._dim + 2)
        else:
            gather_states(self.local_state, self.gathered, self.group)
            states = self.gathered.view(self.world_size, self._rows, self._dim + 2)
        native.merge_states(states, self.output)
        return self.output
