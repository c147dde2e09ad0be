"""Row-subset decode and the bounded device-side waits, through the C ABI.

Row subset: only the listed batch rows are computed and written, every other output row keeps
its bytes (reference: ``row_indices`` of ``exact_decode_attention_rows_triton_forward_out_bhnd``,
kernels/gate0_exact_refresh_triton.py:251-344).

Bounded waits: a kernel that waits for words that never arrive must return by itself and
report ``SA_DEV_PIPELINE_TIMEOUT``.  The wait is made to run out on ONE GPU by declaring a world
of two ranks whose second buffer is a local allocation that no kernel ever writes rank 1's words
into; nothing faults, traps or hangs, and no second kernel is involved.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

import cases
from oracle import cpu_oracle
from streamattn_b200 import native

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; refusing to skip")
    return torch.device("cuda:0")


def _close(got, want):
    diff = (got.float().cpu() - want.float()).abs()
    assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3, (float(diff.max()), float(diff.mean()))


@pytest.mark.parametrize("dtype,kernel", [(torch.bfloat16, "stream"), (torch.float16, "stream"),
                                          (torch.float32, "generic"), (torch.bfloat16, "generic")])
@pytest.mark.parametrize("rows", [[1, 3], [0], [2, 2, 5, -1, 99], []])
def test_row_subset_writes_only_the_listed_rows(dev, dtype, kernel, rows):
    g = torch.Generator().manual_seed(11)
    batch, q_heads, kv_heads, dim, kv_len = 6, 8, 2, 64, 700
    q = torch.randn(batch, 1, q_heads, dim, generator=g).to(dtype)
    k = torch.randn(batch, kv_heads, kv_len, dim, generator=g).to(dtype)
    v = torch.randn(batch, kv_heads, kv_len, dim, generator=g).to(dtype)
    lens = torch.tensor([700, 13, 0, 512, 64, 699], dtype=torch.int32)
    want = cpu_oracle.exact_decode(q, k, v, kv_layout="BHND", lengths=lens.long())
    marker = 7.0
    out = torch.full((batch, 1, q_heads, dim), marker, dtype=dtype, device=dev)
    ws = native.new_workspace(dev, batch, q_heads, kv_heads, dim)
    plan = native.exact_plan(q.to(dev), k.to(dev), v.to(dev), out, ws, kv_layout="BHND", seq_lens=lens.to(dev),
                             kernel=kernel)
    plan.set_rows(torch.tensor(rows, dtype=torch.int64, device=dev))
    for _ in range(2):  # the second run proves counters and split states were left clean
        plan.run()
    torch.cuda.synchronize()
    selected = sorted({r for r in rows if 0 <= r < batch})
    for b in range(batch):
        if b in selected:
            _close(out[b], want[b])
        else:
            assert torch.all(out[b] == marker), f"row {b} was not selected and must stay untouched"
    assert native.workspace_status(ws) == 0
    # Back to every row with the same plan.
    plan.set_rows(None)
    plan.run()
    _close(out, want)


def test_row_subset_on_a_paged_plan_int32_rows(dev):
    pc = cases.PAGED_CASES["p16_g8_d64"]
    q, kp, vp, table, lengths = cases.paged_inputs(pc, layout="HND")
    q, kp, vp = (t.bfloat16() for t in (q, kp, vp))
    want = cpu_oracle.paged_decode(q, kp, vp, table, lengths, layout="HND")
    want = want[0] if isinstance(want, tuple) else want
    batch = int(q.shape[0])
    out = torch.full(q.shape, 3.0, dtype=torch.bfloat16, device=dev)
    ws = native.new_workspace(dev, batch, int(q.shape[2]), int(kp.shape[1]), int(q.shape[3]))
    plan = native.paged_plan(q.to(dev), kp.to(dev), vp.to(dev), table.to(dev), lengths.to(dev), out, ws, layout="HND")
    keep = batch - 1
    plan.set_rows(torch.tensor([keep], dtype=torch.int32, device=dev))
    plan.run()
    torch.cuda.synchronize()
    _close(out[keep], want[keep])
    assert all(torch.all(out[b] == 3.0) for b in range(batch) if b != keep)


def test_rows_function_mirrors_the_reference_call(dev):
    from streamattn_b200.exact import exact_decode_attention_rows_forward_out_bhnd

    g = torch.Generator().manual_seed(5)
    batch, heads, kv_heads, dim, n = 4, 8, 2, 64, 300
    q = torch.randn(batch, heads, 1, dim, generator=g).bfloat16()
    k = torch.randn(batch, kv_heads, n, dim, generator=g).bfloat16()
    v = torch.randn(batch, kv_heads, n, dim, generator=g).bfloat16()
    position = torch.tensor([199], dtype=torch.int64)  # prefix length 200
    want = cpu_oracle.exact_decode(q.transpose(1, 2), k, v, kv_layout="BHND",
                                   lengths=torch.full((batch,), 200, dtype=torch.int64))
    out = torch.zeros(batch, 1, heads, dim, dtype=torch.bfloat16, device=dev)
    got = exact_decode_attention_rows_forward_out_bhnd(q.to(dev), k.to(dev), v.to(dev), out, position.to(dev),
                                                       row_indices={3, 1, 17})
    assert got is out
    torch.cuda.synchronize()
    _close(out[1], want[1])
    _close(out[3], want[3])
    assert float(out[0].abs().max()) == 0.0 and float(out[2].abs().max()) == 0.0
    with pytest.raises(ValueError, match="output must be"):
        exact_decode_attention_rows_forward_out_bhnd(q.to(dev), k.to(dev), v.to(dev), out[:, :, :4], position.to(dev))


def _shard_inputs(dev):
    case = cases.EXACT_CASES["g4_d128_n257"]
    q, k, v = (t.bfloat16() for t in cases.exact_inputs(case))
    want = cpu_oracle.exact_decode(q, k, v)
    kh = k.permute(0, 2, 1, 3).contiguous().to(dev)
    vh = v.permute(0, 2, 1, 3).contiguous().to(dev)
    return case, q.to(dev), kh, vh, want


def test_fused_exchange_wait_runs_out_and_reports(dev):
    """World of two on one GPU where rank 1 never sends: the kernel gives up after 2 ms, sets the
    status bit and returns; the context stays usable and a world-of-one plan then runs clean."""

    case, q, kh, vh, want = _shard_inputs(dev)
    batch, q_heads, kv_heads, dim = case.batch, case.q_heads, case.kv_heads, case.dim
    out = torch.zeros_like(q)
    ws = native.new_workspace(dev, batch, q_heads, kv_heads, dim)
    nbytes = native.cp_fused_bytes(2, batch, q_heads, kv_heads, dim)
    mine = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    silent_peer = torch.zeros(nbytes, dtype=torch.uint8, device=dev)  # nobody writes rank 1's rows into `mine`
    plan = native.cp_fused_plan(q, kh, vh, out, ws, [mine.data_ptr(), silent_peer.data_ptr()], 0)
    plan.set_wait_limit_ns(2_000_000)
    plan.run()
    torch.cuda.synchronize()  # returns: the wait is bounded
    status = native.workspace_status(ws)
    assert status & native.SA_DEV_PIPELINE_TIMEOUT
    # rank 0's own rows did arrive in both buffers (it stores to every rank, itself included)
    assert int(mine.view(torch.int64).ne(0).sum()) > 0 and int(silent_peer.view(torch.int64).ne(0).sum()) > 0

    # The context is intact: a world of one on fresh buffers is clean and correct.
    out1 = torch.zeros_like(q)
    ws1 = native.new_workspace(dev, batch, q_heads, kv_heads, dim)
    solo = torch.zeros(native.cp_fused_bytes(1, batch, q_heads, kv_heads, dim), dtype=torch.uint8, device=dev)
    plan1 = native.cp_fused_plan(q, kh, vh, out1, ws1, [solo.data_ptr()], 0)
    for _ in range(3):
        plan1.run()
    _close(out1, want)
    assert native.workspace_status(ws1) == 0
    # ... and so is the workspace that saw the time-out, after workspace_status() re-zeroed it.
    plain = native.exact_plan(q, kh, vh, out, ws, kv_layout="BHND")
    plain.run()
    _close(out, want)
    assert native.workspace_status(ws) == 0


def test_exchange_kernel_wait_runs_out_and_reports(dev):
    """The separate exchange + merge kernel, same construction: rank 1's flag is never raised."""

    case, q, kh, vh, want = _shard_inputs(dev)
    rows, dim = case.batch * case.q_heads, case.dim
    state = torch.zeros(case.batch, case.q_heads, dim + 2, dtype=torch.float32, device=dev)
    ws = native.new_workspace(dev, case.batch, case.q_heads, case.kv_heads, dim)
    native.exact_plan(q, kh, vh, state, ws, kv_layout="BHND", out_state=True).run()
    out = torch.zeros_like(q)
    nbytes = native.cp_exchange_bytes(2, rows, dim)
    mine = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    silent_peer = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    native.set_wait_limit_ns(2_000_000)
    try:
        ex = native.PeerExchange(state, [mine.data_ptr(), silent_peer.data_ptr()], 0, out)
        ex.run()
        torch.cuda.synchronize()
        assert ex.status() & native.SA_DEV_PIPELINE_TIMEOUT
        assert ex.status() == 0  # read-and-clear
    finally:
        native.set_wait_limit_ns(2_000_000_000)
    solo = torch.zeros(native.cp_exchange_bytes(1, rows, dim), dtype=torch.uint8, device=dev)
    ex1 = native.PeerExchange(state, [solo.data_ptr()], 0, out)
    ex1.run()
    _close(out, want)
    assert ex1.status() == 0


def test_wait_limit_arguments_are_checked(dev):
    lib = native.load()
    assert lib.sa_set_wait_limit_ns(ctypes.c_uint64(0)) == native.SA_ERR_INVALID
    assert lib.sa_plan_set_wait_limit_ns(None, ctypes.c_uint64(5)) == native.SA_ERR_INVALID
    assert lib.sa_plan_set_rows(None, None, 0, 0) == native.SA_ERR_INVALID


@pytest.mark.parametrize("world", [4, 8])
def test_fused_exchange_data_path_of_many_ranks_on_one_gpu(dev, world):
    """The 4- and 8-rank exchange (addresses, strides, merge over all ranks) checked on ONE GPU
    without two kernels ever waiting on each other: the ranks' launches run one after the other,
    each with a 0.3 ms wait limit.  All but the last give up their wait (and say so); the last
    one finds every rank's words of the step already in its buffer and must produce the exact
    result.  The launch order rotates, so different ranks come last in different steps."""

    case = cases.EXACT_CASES["g4_d128_n257"]
    q, k, v = (t.bfloat16() for t in cases.exact_inputs(case))
    want = cpu_oracle.exact_decode(q, k, v)
    batch, q_heads, kv_heads, dim = case.batch, case.q_heads, case.kv_heads, case.dim
    qd = q.to(dev)
    nbytes = native.cp_fused_bytes(world, batch, q_heads, kv_heads, dim)
    buffers = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(world)]
    ptrs = [b.data_ptr() for b in buffers]
    plans, outs, spaces = [], [], []
    for r in range(world):
        lo, hi = case.kv_len * r // world, case.kv_len * (r + 1) // world
        kh = k[:, lo:hi].permute(0, 2, 1, 3).contiguous().to(dev)
        vh = v[:, lo:hi].permute(0, 2, 1, 3).contiguous().to(dev)
        out = torch.zeros_like(qd)
        ws = native.new_workspace(dev, batch, q_heads, kv_heads, dim)
        plan = native.cp_fused_plan(qd, kh, vh, out, ws, ptrs, r)
        plan.set_wait_limit_ns(300_000)
        plans.append(plan)
        outs.append(out)
        spaces.append(ws)
    for step in range(3):
        order = [(step * 3 + i) % world for i in range(world)]
        for r in order:
            plans[r].run()
            torch.cuda.synchronize()
        last = order[-1]
        _close(outs[last], want)
        for r in order:
            status = native.workspace_status(spaces[r])
            assert (status == 0) == (r == last), (step, r, status)
