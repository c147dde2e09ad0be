"""GPU parity: the sm_100a kernels, called through the C ABI, against the CPU oracle.

Inputs are seeded on the CPU, rounded to the tested dtype, and handed to both
sides, so the oracle (double accumulation) sees the same bits as the kernel.
Tolerances: bf16/fp16 outputs within max-abs 2e-2 and mean-abs 2e-3 of the
fp32/fp64 reference (the bound the drop-in contract states); fp32 outputs
within 2e-5.  Index work (page walk, seed sets) is compared bit-exactly.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

import cases
import streamattn_b200 as sa
from oracle import cpu_oracle
from streamattn_b200 import native

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
MEAN_ABS = 2e-3
F32_ATOL = 2e-5


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; refusing to skip")
    device = torch.device("cuda:0")
    assert native.device_supported(device), "the kernels are built for sm_100a only"
    return device


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: torch.dtype) -> None:
    diff = (got.detach().float().cpu() - want.float().cpu()).abs()
    assert torch.isfinite(got.float()).all()
    if dtype == torch.float32:
        assert float(diff.max()) <= F32_ATOL, float(diff.max())
    else:
        assert float(diff.max()) <= MAX_ABS, float(diff.max())
        assert float(diff.mean()) <= MEAN_ABS, float(diff.mean())


def _exact_plan(dev, q, k, v, *, layout, kernel, **kw):
    kd, vd = (t.permute(0, 2, 1, 3).contiguous() if layout == "BHND" else t for t in (k, v))
    qd, kd, vd = q.to(dev), kd.to(dev), vd.to(dev)
    heads = kd.shape[1] if layout == "BHND" else kd.shape[2]
    out = torch.empty_like(qd) if not kw.get("out_state") else torch.empty(
        q.shape[0], q.shape[2], q.shape[3] + 2, dtype=torch.float32, device=dev)
    ws = native.new_workspace(dev, q.shape[0], q.shape[2], int(heads), q.shape[3], kw.get("num_ctas", 0))
    plan = native.exact_plan(qd, kd, vd, out, ws, kv_layout=layout, kernel=kernel, **kw)
    return plan, out, ws, (qd, kd, vd)


STREAM_EXACT = [n for n, c in cases.EXACT_CASES.items() if c.dim in (64, 128) and c.q_heads // c.kv_heads <= 16]


@pytest.mark.parametrize("layout", ["BNHD", "BHND"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("name", STREAM_EXACT)
def test_exact_stream_kernel(dev, name, dtype, layout):
    case = cases.EXACT_CASES[name]
    q, k, v = (t.to(dtype) for t in cases.exact_inputs(case))
    want = cpu_oracle.exact_decode(q, k, v)
    plan, out, ws, _ = _exact_plan(dev, q, k, v, layout=layout, kernel="stream")
    assert plan.kernel == native.SA_KERNEL_STREAM and plan.launches == 1
    plan.run()
    assert native.workspace_status(ws) == 0
    assert_close(out, want, dtype)
    first = out.clone()
    plan.run()
    torch.cuda.synchronize()
    assert torch.equal(first, out), "replay of a bound plan must be bit-identical"


@pytest.mark.parametrize("layout", ["BNHD", "BHND"])
@pytest.mark.parametrize("name", STREAM_EXACT)
def test_exact_stream_kernel_dynamic_schedule(dev, name, layout):
    """SA_KERNEL_FLAG_DYNAMIC: tiles claimed from a device counter; within tolerance on every launch."""

    case = cases.EXACT_CASES[name]
    q, k, v = (t.to(torch.bfloat16) for t in cases.exact_inputs(case))
    want = cpu_oracle.exact_decode(q, k, v)
    plan, out, ws, _ = _exact_plan(dev, q, k, v, layout=layout, kernel="stream", dynamic=True)
    for _ in range(3):
        out.zero_()
        plan.run()
        assert native.workspace_status(ws) == 0
        assert_close(out, want, torch.bfloat16)


@pytest.mark.parametrize("layout", ["BNHD", "BHND"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("name", list(cases.EXACT_CASES))
def test_exact_generic_kernel(dev, name, dtype, layout):
    case = cases.EXACT_CASES[name]
    q, k, v = (t.to(dtype) for t in cases.exact_inputs(case))
    want = cpu_oracle.exact_decode(q, k, v)
    plan, out, ws, _ = _exact_plan(dev, q, k, v, layout=layout, kernel="generic")
    assert plan.kernel == native.SA_KERNEL_GENERIC
    plan.run()
    assert native.workspace_status(ws) == 0
    assert_close(out, want, dtype)


@pytest.mark.parametrize("name", list(cases.EXACT_CASES))
def test_exact_matches_reference_golden_outputs(dev, golden_exact, name):
    """fp32 inputs -> the reference's own stored outputs (its CPU path)."""

    case = cases.EXACT_CASES[name]
    q, k, v = cases.exact_inputs(case)
    plan, out, _, _ = _exact_plan(dev, q, k, v, layout="BNHD", kernel="auto")
    plan.run()
    want = torch.from_numpy(golden_exact[f"{name}/out"])
    torch.testing.assert_close(out.cpu(), want, atol=F32_ATOL, rtol=1e-4)


@pytest.mark.parametrize("kernel", ["stream", "generic"])
def test_exact_row_lengths_and_empty_rows(dev, kernel):
    case = cases.EXACT_CASES["g8_d64_n300"]
    q, k, v = (t.to(torch.bfloat16) for t in cases.exact_inputs(case))
    for lens_dtype in (torch.int32, torch.int64):
        lengths = torch.tensor([123, 0], dtype=lens_dtype)
        want = cpu_oracle.exact_decode(q, k, v, lengths=lengths)
        plan, out, ws, _ = _exact_plan(dev, q, k, v, layout="BNHD", kernel=kernel, seq_lens=lengths.to(dev))
        out.fill_(7.0)
        plan.run()
        assert native.workspace_status(ws) == 0
        assert_close(out, want, torch.bfloat16)
        assert float(out[1].abs().max()) == 0.0, "a row without tokens yields zeros"


@pytest.mark.parametrize("num_ctas", [1, 3, 16, 148, 500])
def test_exact_split_count_invariance(dev, num_ctas):
    case = cases.EXACT_CASES["g7_d64_n1000"]
    q, k, v = (t.to(torch.bfloat16) for t in cases.exact_inputs(case))
    want = cpu_oracle.exact_decode(q, k, v)
    plan, out, ws, _ = _exact_plan(dev, q, k, v, layout="BHND", kernel="stream", num_ctas=num_ctas)
    for _ in range(3):  # the arrival counters must return to zero after every launch
        out.zero_()
        plan.run()
        assert native.workspace_status(ws) == 0
        assert_close(out, want, torch.bfloat16)


def test_exact_state_output_and_merge(dev):
    """Shard states (o, m, l) merged on the GPU equal the unsharded result."""

    case = cases.EXACT_CASES["g4_d128_n257"]
    q, k, v = (t.to(torch.bfloat16) for t in cases.exact_inputs(case))
    want = cpu_oracle.exact_decode(q, k, v)
    cuts = [0, 100, 132, 257]
    states = []
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        plan, st, _, _ = _exact_plan(dev, q, k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(),
                                     layout="BHND", kernel="stream", out_state=True)
        plan.run()
        states.append(st.reshape(-1, case.dim + 2))
        _, ref_state = cpu_oracle.exact_decode(q, k, v, token_range=(lo, hi), return_state=True)
        # l and the normalised o agree with the oracle's state (m differs by the log base).
        got = st.cpu()
        torch.testing.assert_close(got[..., : case.dim] / got[..., case.dim + 1 :],
                                   ref_state[..., : case.dim] / ref_state[..., case.dim + 1 :],
                                   atol=MAX_ABS, rtol=0)
    stacked = torch.stack(states).contiguous()
    out = torch.empty(case.batch, 1, case.q_heads, case.dim, dtype=torch.bfloat16, device=dev)
    native.merge_states(stacked, out)
    assert_close(out, want, torch.bfloat16)
    merged_ref = cpu_oracle.merge_states(stacked.cpu(), log2_domain=True)
    assert_close(out.reshape(-1, case.dim), merged_ref, torch.bfloat16)


def _paged_plan(dev, case, dtype, layout, kernel, *, table_dtype=torch.int32, lens_dtype=torch.int32):
    q, k, v, table, lengths = cases.paged_inputs(case, layout=layout)
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    want, trav = cpu_oracle.paged_decode(q, k, v, table, lengths, layout=layout, return_traversal=True)
    cache = sa.PagedKVCache(key=k.to(dev), value=v.to(dev), page_table=table.to(dev, table_dtype),
                            sequence_lengths=lengths.to(dev, lens_dtype), layout=layout)
    plan = sa.PagedExactDecodePlan.build(q.to(dev), cache, record_page_walk=True, kernel=kernel)
    return plan, want, trav


STREAM_PAGED = [n for n, c in cases.PAGED_CASES.items() if c.dim in (64, 128) and c.page_size >= 8]


@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("name", STREAM_PAGED)
def test_paged_stream_kernel_and_page_walk(dev, name, layout):
    case = cases.PAGED_CASES[name]
    plan, want, trav = _paged_plan(dev, case, torch.bfloat16, layout, "stream")
    assert plan.backend == sa.PAGED_EXACT_SM100_BACKEND and plan.launches_per_run == 1
    out = plan.run()
    assert plan.device_status() == 0
    assert_close(out, want, torch.bfloat16)
    # Page-table traversal is bit-exact and -1 slots are never touched.
    assert torch.equal(plan.trace.cpu().long(), trav)


@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(cases.PAGED_CASES))
def test_paged_generic_kernel_and_page_walk(dev, name, dtype, layout):
    case = cases.PAGED_CASES[name]
    plan, want, trav = _paged_plan(dev, case, dtype, layout, "generic",
                                   table_dtype=torch.int64, lens_dtype=torch.int64)
    assert plan.backend == sa.PAGED_EXACT_NATIVE_BACKEND
    out = plan.run()
    assert plan.device_status() == 0
    assert_close(out, want, dtype)
    assert torch.equal(plan.trace.cpu().long(), trav)


@pytest.mark.parametrize("layout", ["NHD", "HND"])
def test_paged_reference_fixture_and_golden(dev, golden_paged, layout):
    """The reference's own paged fixture (seed 17) against its stored output."""

    q, k, v, table, lengths = cases.reference_paged_fixture(layout=layout)
    cache = sa.PagedKVCache(key=k.to(dev), value=v.to(dev), page_table=table.to(dev),
                            sequence_lengths=lengths.to(dev), layout=layout)
    out, info = sa.decode(q.to(dev), cache, mode="verified_auto")
    want = torch.from_numpy(golden_paged[f"fixture17_{layout}/out"])
    torch.testing.assert_close(out.cpu(), want, atol=F32_ATOL, rtol=1e-4)
    assert info.plan_reason == "paged_kv_exact_only" and info.seed_only_enabled is False
    assert info.stats["page_size"] == 4 and info.stats["layout"] == layout
    assert info.backend_used == sa.PAGED_EXACT_NATIVE_BACKEND


@pytest.mark.parametrize("name", list(cases.PAGED_CASES))
def test_paged_matches_reference_golden_outputs(dev, golden_paged, name):
    case = cases.PAGED_CASES[name]
    q, k, v, table, lengths = cases.paged_inputs(case, layout="HND")
    cache = sa.PagedKVCache(key=k.to(dev), value=v.to(dev), page_table=table.to(dev),
                            sequence_lengths=lengths.to(dev), layout="HND")
    out = sa.stream_attn_paged_exact_decode(q.to(dev), cache)
    want = torch.from_numpy(golden_paged[f"{name}_HND/out"])
    torch.testing.assert_close(out.cpu(), want, atol=F32_ATOL, rtol=1e-4)


def test_paged_plan_sees_in_place_updates(dev):
    case = cases.PAGED_CASES["p16_g8_d64"]
    q, k, v, table, lengths = cases.paged_inputs(case, layout="HND")
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    cache = sa.PagedKVCache(key=k.to(dev), value=v.to(dev), page_table=table.to(dev),
                            sequence_lengths=lengths.to(dev), layout="HND")
    plan = sa.PagedExactDecodePlan.build(q.to(dev), cache)
    first = plan.run().clone()
    pointer = plan.output.data_ptr()
    cache.value[int(table[0, 0])].add_(0.5)         # page contents change in place
    second = plan.run().clone()
    assert plan.output.data_ptr() == pointer and not torch.equal(first, second)
    cache.sequence_lengths[1] = 17                   # a row gets shorter: lengths are read on the device
    lengths2 = lengths.clone()
    lengths2[1] = 17
    v2 = cache.value.cpu()
    want = cpu_oracle.paged_decode(q, k, v2, table, lengths2, layout="HND")
    assert_close(plan.run(), want, torch.bfloat16)
    assert plan.workspace_bytes > 0 and plan.splits >= 1


@pytest.mark.parametrize("kernel", ["stream", "generic"])
def test_paged_out_of_range_page_is_skipped_and_reported(dev, kernel):
    """A corrupt active entry must not be dereferenced; the status word says so."""

    case = cases.PAGED_CASES["p16_g8_d64"]
    q, k, v, table, lengths = cases.paged_inputs(case, layout="HND")
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    table = table.clone()
    table[0, 1] = 10 ** 6
    cache = sa.PagedKVCache(key=k.to(dev), value=v.to(dev), page_table=table.to(dev),
                            sequence_lengths=lengths.to(dev), layout="HND")
    with pytest.raises(ValueError, match="active page_table"):
        sa.PagedExactDecodePlan.build(q.to(dev), cache)
    plan = sa.PagedExactDecodePlan.build(q.to(dev), cache, validate_metadata=False, kernel=kernel)
    plan.run()
    assert plan.device_status() & native.SA_DEV_BAD_PAGE
    assert plan.device_status() == 0, "reading the status clears it"


def _seed_plan(dev, q, k, v, *, block_size, blocks, kernel):
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out = torch.empty_like(qd)
    ws = native.new_workspace(dev, q.shape[0], q.shape[2], k.shape[2], q.shape[3])
    return native.seed_plan(qd, kd, vd, out, ws, block_size=block_size, blocks=blocks, kernel=kernel), out, ws


@pytest.mark.parametrize("kernel", ["stream", "generic"])
@pytest.mark.parametrize("name", list(cases.SEED_CASES))
def test_seed_only_decode(dev, golden_seed, name, kernel):
    case = cases.SEED_CASES[name]
    if kernel == "stream" and case.dim not in (64, 128):
        pytest.skip("streaming kernel covers head_dim 64/128")
    dtype = torch.bfloat16
    q, k, v = (t.to(dtype) for t in cases.seed_inputs(case))
    blocks = sa.policy_seed_blocks(seq_len=case.kv_len, block_size=case.block_size, sink_blocks=case.sink_blocks,
                                   recent_blocks=case.recent_blocks, middle_seed_blocks=case.middle_seed_blocks,
                                   block_order=case.block_order)
    tokens = sa.seed_token_indices_from_blocks(seq_len=case.kv_len, block_size=case.block_size, blocks=blocks)
    assert torch.equal(tokens, cpu_oracle.seed_indices(
        seq_len=case.kv_len, block_size=case.block_size, sink_blocks=case.sink_blocks,
        recent_blocks=case.recent_blocks, middle_seed_blocks=case.middle_seed_blocks, block_order=case.block_order))
    want = cpu_oracle.seed_decode(q, k, v, tokens)
    plan, out, ws = _seed_plan(dev, q, k, v, block_size=case.block_size, blocks=blocks, kernel=kernel)
    plan.run()
    assert native.workspace_status(ws) == 0
    assert_close(out, want, dtype)
    # fp32 inputs through the generic kernel reproduce the reference's stored output.
    if kernel == "generic":
        q32, k32, v32 = cases.seed_inputs(case)
        plan, out, _ = _seed_plan(dev, q32, k32, v32, block_size=case.block_size, blocks=blocks, kernel="generic")
        plan.run()
        torch.testing.assert_close(out.cpu(), torch.from_numpy(golden_seed[f"{name}/out"]), atol=F32_ATOL, rtol=1e-4)


def test_seed_only_explicit_blocks_qwen_shape(dev):
    """BASELINE config 4 shape: 64 sink + 4x16 middle at seeded offsets + 256 recent tokens."""

    g = torch.Generator().manual_seed(0)
    batch, q_heads, kv_heads, dim, kv_len, bs = 8, 16, 2, 128, 32768, 16
    q = torch.randn(batch, 1, q_heads, dim, generator=g).bfloat16()
    k = torch.randn(batch, kv_len, kv_heads, dim, generator=g).bfloat16()
    v = torch.randn(batch, kv_len, kv_heads, dim, generator=g).bfloat16()
    middle = (torch.randperm(2032 - 4, generator=g)[:4] + 4).tolist()
    blocks = [0, 1, 2, 3, *middle, *range(2032, 2048)]
    tokens = sa.seed_token_indices_from_blocks(seq_len=kv_len, block_size=bs, blocks=blocks)
    assert tokens.numel() == 384
    assert torch.equal(tokens, cpu_oracle.seed_tokens_from_blocks(seq_len=kv_len, block_size=bs, blocks=blocks))
    want = cpu_oracle.seed_decode(q, k, v, tokens)
    for kernel in ("stream", "generic"):
        plan, out, ws = _seed_plan(dev, q, k, v, block_size=bs, blocks=blocks[::-1] + [2, 2], kernel=kernel)
        plan.run()
        assert native.workspace_status(ws) == 0
        assert_close(out, want, torch.bfloat16)


def test_one_shot_c_abi_calls(dev):
    """The one-shot entry points (no plan object), called with raw pointers."""

    lib = native.load()
    case = cases.EXACT_CASES["g8_d64_n300"]
    q, k, v = (t.to(torch.bfloat16) for t in cases.exact_inputs(case))
    want = cpu_oracle.exact_decode(q, k, v)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out = torch.empty_like(qd)
    ws = native.new_workspace(dev, case.batch, case.q_heads, case.kv_heads, case.dim)
    stream = native.stream_handle(dev)
    rc = lib.sa_exact_decode(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(),
                             None, 0, case.batch, case.q_heads, case.kv_heads, case.dim, case.kv_len,
                             qd.stride(0), qd.stride(2), kd.stride(0), kd.stride(1), kd.stride(2),
                             native.SA_DTYPE[torch.bfloat16], native.SA_OUT_FINAL, 0, native.SA_KERNEL_AUTO, stream)
    assert rc == 0, native.last_error()
    assert_close(out, want, torch.bfloat16)

    out.zero_()
    rc = lib.sa_seed_decode(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(),
                            case.batch, case.q_heads, case.kv_heads, case.dim, case.kv_len,
                            qd.stride(0), qd.stride(2), kd.stride(0), kd.stride(1), kd.stride(2),
                            native.SA_DTYPE[torch.bfloat16], 16, 1, 2, 3, native.SA_BLOCK_ORDER["recent_first"],
                            0, native.SA_KERNEL_AUTO, stream)
    assert rc == 0, native.last_error()
    tokens = cpu_oracle.seed_indices(seq_len=case.kv_len, block_size=16, sink_blocks=1, recent_blocks=2,
                                     middle_seed_blocks=3, block_order="recent_first")
    assert_close(out, cpu_oracle.seed_decode(q, k, v, tokens), torch.bfloat16)

    pc = cases.PAGED_CASES["p16_g8_d64"]
    pq, pk, pv, table, lengths = cases.paged_inputs(pc, layout="HND")
    pq, pk, pv = (t.to(torch.bfloat16) for t in (pq, pk, pv))
    pwant = cpu_oracle.paged_decode(pq, pk, pv, table, lengths, layout="HND")
    pqd, pkd, pvd, td, ld = (t.to(dev) for t in (pq, pk, pv, table, lengths))
    pout = torch.empty_like(pqd)
    pws = native.new_workspace(dev, pc.batch, pc.q_heads, pc.kv_heads, pc.dim)
    rc = lib.sa_paged_decode(pqd.data_ptr(), pkd.data_ptr(), pvd.data_ptr(), td.data_ptr(), ld.data_ptr(),
                             pout.data_ptr(), pws.data_ptr(), pws.numel(), None, pc.batch, pc.q_heads, pc.kv_heads,
                             pc.dim, pc.page_size, pc.max_pages, pkd.shape[0], native.SA_LAYOUT["HND"],
                             native.SA_DTYPE[torch.bfloat16], 0, 0, native.SA_OUT_FINAL, 0, native.SA_KERNEL_AUTO,
                             stream)
    assert rc == 0, native.last_error()
    assert_close(pout, pwant, torch.bfloat16)

    # Argument errors come back as status codes with a message; nothing is launched.
    rc = lib.sa_exact_decode(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), out.data_ptr(), ws.data_ptr(), 64,
                             None, 0, case.batch, case.q_heads, case.kv_heads, case.dim, case.kv_len,
                             qd.stride(0), qd.stride(2), kd.stride(0), kd.stride(1), kd.stride(2),
                             native.SA_DTYPE[torch.bfloat16], native.SA_OUT_FINAL, 0, native.SA_KERNEL_AUTO, stream)
    assert rc == native.SA_ERR_INVALID and "workspace too small" in native.last_error()
    rc = lib.sa_exact_decode(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(),
                             None, 0, case.batch, case.q_heads, 3, case.dim, case.kv_len,
                             qd.stride(0), qd.stride(2), kd.stride(0), kd.stride(1), kd.stride(2),
                             native.SA_DTYPE[torch.bfloat16], native.SA_OUT_FINAL, 0, native.SA_KERNEL_AUTO, stream)
    assert rc == native.SA_ERR_INVALID
    torch.cuda.synchronize()


def test_plans_replay_inside_a_cuda_graph(dev):
    """A decode step captured into a CUDA graph (three launches back to back, the way a decode
    loop replays them) gives the bits of the eager run; the kernels are launched with
    programmatic stream serialization, which must survive capture."""

    g = torch.Generator().manual_seed(5)
    batch, q_heads, kv_heads, dim, kv_len = 4, 16, 2, 64, 4096
    q = torch.randn(batch, 1, q_heads, dim, generator=g).bfloat16().to(dev)
    k = torch.randn(batch, kv_heads, kv_len, dim, generator=g).bfloat16().to(dev)
    v = torch.randn(batch, kv_heads, kv_len, dim, generator=g).bfloat16().to(dev)
    out = torch.empty_like(q)
    ws = native.new_workspace(dev, batch, q_heads, kv_heads, dim)
    plan = native.exact_plan(q, k, v, out, ws, kv_layout="BHND", kernel="stream")
    plan.run()
    torch.cuda.synchronize()
    eager = out.clone()
    side = torch.cuda.Stream(device=dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        plan.run()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(3):
                plan.run()
    for _ in range(2):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)
    assert native.workspace_status(ws) == 0
