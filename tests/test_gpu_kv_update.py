"""GPU parity of the KV-cache update step (rotary embedding + append), through the C ABI.

The kernel must reproduce the reference's safe path bit for bit: the stored outputs of the
reference (``tests/golden/rope_append_reference_outputs.npz``) and the oracle restatement of it
on the same seeded inputs, for contiguous and paged caches; then a short decode loop
(append, decode, append, ...) must agree with the oracle's loop.
"""

from pathlib import Path

import numpy as np
import pytest
import torch

import streamattn_b200 as sa
from oracle import cpu_oracle, torch_port
from streamattn_b200 import native
from streamattn_b200.kv_update import PagedKVWriter, PagePool, append_kv, paged_append_kv
from tests.golden import cases

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden" / "rope_append_reference_outputs.npz"


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; refusing to skip")
    return torch.device("cuda:0")


def _positions(case):
    return list(case.positions if len(case.positions) > 1 else case.positions * case.batch)


@pytest.mark.parametrize("kv_layout", ["BHND", "BNHD"])
@pytest.mark.parametrize("name", list(cases.ROPE_APPEND_CASES))
def test_rope_append_contiguous_bit_exact(dev, name, kv_layout):
    case = cases.ROPE_APPEND_CASES[name]
    golden = np.load(GOLDEN)
    q_raw, k_raw, v_raw, cos, sin, k_cache, v_cache = cases.rope_append_inputs(case)
    want_k, want_v = k_cache.clone(), v_cache.clone()
    want_q = torch_port.rope_append(q_raw, k_raw, v_raw, cos, sin, want_k, want_v, _positions(case))

    def cache_to_dev(t):
        return (t.transpose(1, 2).contiguous() if kv_layout == "BNHD" else t.clone()).to(dev)

    kc, vc = cache_to_dev(k_cache), cache_to_dev(v_cache)
    positions = torch.tensor(case.positions, dtype=torch.int64, device=dev)   # one entry or one per row
    lengths_out = torch.zeros(case.batch, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    q_rot = append_kv(kc, vc, k_raw.to(dev), v_raw.to(dev), positions, kv_layout=kv_layout, new_layout="BHND",
                      cos=cos.to(dev), sin=sin.to(dev), query=q_raw.to(dev), query_layout="BHND",
                      lengths_out=lengths_out, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got_k = kc.transpose(1, 2) if kv_layout == "BNHD" else kc
    got_v = vc.transpose(1, 2) if kv_layout == "BNHD" else vc
    assert torch.equal(q_rot.cpu(), want_q)
    assert torch.equal(got_k.cpu(), want_k) and torch.equal(got_v.cpu(), want_v)
    assert lengths_out.cpu().tolist() == [p + 1 for p in _positions(case)]
    # ... and the reference's stored outputs themselves.
    idx, rows = torch.arange(case.batch), torch.tensor(_positions(case))
    assert np.array_equal(q_rot.float().cpu().numpy(), golden[f"{name}/q_rot"])
    assert np.array_equal(got_k.cpu()[idx, :, rows, :].float().numpy(), golden[f"{name}/k_rows"])
    assert np.array_equal(got_v.cpu()[idx, :, rows, :].float().numpy(), golden[f"{name}/v_rows"])


@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rope_append_paged_bit_exact_and_lengths_advance(dev, layout, dtype):
    g = torch.Generator().manual_seed(21)
    batch, q_heads, kv_heads, dim, page, max_pages = 3, 8, 2, 64, 16, 4
    num_pages = batch * max_pages
    shape = (num_pages, page, kv_heads, dim) if layout == "NHD" else (num_pages, kv_heads, page, dim)
    kp = torch.randn(shape, generator=g).to(dtype)
    vp = torch.randn(shape, generator=g).to(dtype)
    table = torch.randperm(num_pages, generator=g).to(torch.int32).view(batch, max_pages)
    lengths = torch.tensor([5, 16, 47], dtype=torch.int32)       # next token: mid page, page start, page end
    q_raw = torch.randn(batch, 1, q_heads, dim, generator=g).to(dtype)
    k_raw = torch.randn(batch, 1, kv_heads, dim, generator=g).to(dtype)
    v_raw = torch.randn(batch, 1, kv_heads, dim, generator=g).to(dtype)
    angles = torch.randn(batch, 1, dim // 2, generator=g)
    emb = torch.cat((angles, angles), dim=-1)
    cos, sin = emb.cos().to(dtype), emb.sin().to(dtype)
    want_k, want_v = kp.clone(), vp.clone()
    want_q = torch_port.paged_rope_append(q_raw.transpose(1, 2), k_raw.transpose(1, 2), v_raw.transpose(1, 2), cos, sin,
                                          want_k, want_v, table, lengths.tolist(), layout=layout)
    cache = sa.PagedKVCache(key=kp.to(dev), value=vp.to(dev), page_table=table.to(dev),
                            sequence_lengths=lengths.to(dev), layout=layout)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    q_rot = paged_append_kv(cache, k_raw.to(dev), v_raw.to(dev), cos=cos.to(dev), sin=sin.to(dev),
                            query=q_raw.to(dev), status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(q_rot.cpu(), want_q.transpose(1, 2))
    assert torch.equal(cache.key.cpu(), want_k) and torch.equal(cache.value.cpu(), want_v)
    assert cache.sequence_lengths.cpu().tolist() == [6, 17, 48]  # advanced in place on the device


def test_append_reports_bad_position_and_unassigned_page(dev):
    batch, kv_heads, dim, page, max_pages = 2, 2, 64, 16, 2
    kp = torch.zeros(4, page, kv_heads, dim, dtype=torch.bfloat16, device=dev)
    vp = torch.zeros_like(kp)
    table = torch.tensor([[0, -1], [1, 2]], dtype=torch.int32, device=dev)
    lengths = torch.tensor([16, 32], dtype=torch.int32, device=dev)   # row 0: page not assigned; row 1: cache full
    cache = sa.PagedKVCache(key=kp, value=vp, page_table=table, sequence_lengths=lengths, layout="NHD")
    ones = torch.ones(batch, 1, kv_heads, dim, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    paged_append_kv(cache, ones, ones, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == native.SA_DEV_BAD_PAGE | native.SA_DEV_BAD_POSITION
    assert float(kp.abs().sum()) == 0.0 and float(vp.abs().sum()) == 0.0     # nothing written
    assert lengths.cpu().tolist() == [16, 32]                                 # skipped rows do not advance
    with pytest.raises(ValueError, match="one entry or one per batch row"):
        append_kv(torch.zeros(2, 2, 8, 64, device=dev), torch.zeros(2, 2, 8, 64, device=dev),
                  torch.zeros(2, 2, 1, 64, device=dev), torch.zeros(2, 2, 1, 64, device=dev),
                  torch.zeros(3, dtype=torch.int64, device=dev))


def test_decode_loop_append_then_decode_matches_oracle(dev):
    """Five steps of append (with RoPE) + paged exact decode on a bound plan, no host sync inside
    the step: the plan must see each new token, pages are assigned ahead by the host allocator."""

    g = torch.Generator().manual_seed(33)
    batch, q_heads, kv_heads, dim, page, max_pages = 2, 8, 2, 64, 16, 6
    num_pages = batch * max_pages
    start = [30, 47]
    kp = torch.zeros(num_pages, kv_heads, page, dim, dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    table = torch.full((batch, max_pages), -1, dtype=torch.int32)
    pool = PagePool(num_pages)
    for b, n in enumerate(start):
        ids = pool.allocate(-(-n // page))
        table[b, : len(ids)] = torch.tensor(ids, dtype=torch.int32)
        for t in range(n):
            kp[ids[t // page], :, t % page] = torch.randn(kv_heads, dim, generator=g).bfloat16()
            vp[ids[t // page], :, t % page] = torch.randn(kv_heads, dim, generator=g).bfloat16()
    ref_k, ref_v, ref_table = kp.clone(), vp.clone(), table.clone()
    cache = sa.PagedKVCache(key=kp.to(dev), value=vp.to(dev), page_table=table.to(dev),
                            sequence_lengths=torch.tensor(start, dtype=torch.int32, device=dev), layout="HND")
    writer = PagedKVWriter.attach(cache, pool)
    q_dev = torch.zeros(batch, 1, q_heads, dim, dtype=torch.bfloat16, device=dev)
    plan = sa.PagedExactDecodePlan.build(q_dev, cache, validate_metadata=False)
    lengths = list(start)
    for step in range(5):
        q_raw = torch.randn(batch, 1, q_heads, dim, generator=g).bfloat16()
        k_raw = torch.randn(batch, 1, kv_heads, dim, generator=g).bfloat16()
        v_raw = torch.randn(batch, 1, kv_heads, dim, generator=g).bfloat16()
        angles = torch.randn(batch, 1, dim // 2, generator=g)
        emb = torch.cat((angles, angles), dim=-1)
        cos, sin = emb.cos().bfloat16(), emb.sin().bfloat16()
        # device: assign pages, append + rotate q straight into the plan's query buffer, decode
        writer.append(k_raw.to(dev), v_raw.to(dev), cos=cos.to(dev), sin=sin.to(dev), query=q_raw.to(dev),
                      query_out=q_dev)
        out = plan.run().clone()
        # oracle: same step on the CPU
        ref_table = cache.page_table.cpu()
        q_rot = torch_port.paged_rope_append(q_raw.transpose(1, 2), k_raw.transpose(1, 2), v_raw.transpose(1, 2),
                                             cos, sin, ref_k, ref_v, ref_table, lengths, layout="HND")
        lengths = [n + 1 for n in lengths]
        want = cpu_oracle.paged_decode(q_rot.transpose(1, 2).contiguous(), ref_k, ref_v, ref_table,
                                       torch.tensor(lengths, dtype=torch.int32), layout="HND")
        want = want[0] if isinstance(want, tuple) else want
        diff = (out.float().cpu() - want.float()).abs()
        assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3, (step, float(diff.max()))
        assert torch.equal(cache.key.cpu(), ref_k) and torch.equal(cache.value.cpu(), ref_v)
    assert writer.lengths == lengths == cache.sequence_lengths.cpu().tolist()
    assert plan.device_status() == 0

@pytest.mark.gpu
def test_released_row_is_reused_from_position_zero(dev):
    """release(row) empties the request on the device too: the next appends start a fresh page at
    position 0, a decode sees exactly the new tokens, and no bad-page status is raised."""

    g = torch.Generator().manual_seed(7)
    batch, q_heads, kv_heads, dim, page, max_pages = 2, 8, 2, 64, 16, 4
    num_pages = 6
    start = [20, 33]
    kp = torch.zeros(num_pages, kv_heads, page, dim, dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    table = torch.full((batch, max_pages), -1, dtype=torch.int32)
    pool = PagePool(num_pages)
    for b, n in enumerate(start):
        ids = pool.allocate(-(-n // page))
        table[b, : len(ids)] = torch.tensor(ids, dtype=torch.int32)
        for t in range(n):
            kp[ids[t // page], :, t % page] = torch.randn(kv_heads, dim, generator=g).bfloat16()
            vp[ids[t // page], :, t % page] = torch.randn(kv_heads, dim, generator=g).bfloat16()
    cache = sa.PagedKVCache(key=kp.to(dev), value=vp.to(dev), page_table=table.to(dev),
                            sequence_lengths=torch.tensor(start, dtype=torch.int32, device=dev), layout="HND")
    writer = PagedKVWriter.attach(cache, pool)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    writer.release(1)
    assert pool.free_pages == num_pages - 2 and cache.sequence_lengths.tolist() == [20, 0]
    q = torch.randn(batch, 1, q_heads, dim, generator=g).bfloat16()
    new_k, new_v = [], []
    for _ in range(3):
        k_new = torch.randn(batch, 1, kv_heads, dim, generator=g).bfloat16()
        v_new = torch.randn(batch, 1, kv_heads, dim, generator=g).bfloat16()
        writer.append(k_new.to(dev), v_new.to(dev), status=status)
        new_k.append(k_new)
        new_v.append(v_new)
    assert int(status.item()) == 0
    assert cache.sequence_lengths.tolist() == [23, 3] == writer.lengths
    first_page = writer.pages[1][0]
    for t in range(3):
        assert torch.equal(cache.key[first_page, :, t].cpu(), new_k[t][1, 0])
        assert torch.equal(cache.value[first_page, :, t].cpu(), new_v[t][1, 0])
    plan = sa.PagedExactDecodePlan.build(q.to(dev), cache)
    want = cpu_oracle.paged_decode(q, cache.key.cpu(), cache.value.cpu(), cache.page_table.cpu(),
                                   cache.sequence_lengths.cpu(), layout="HND")
    want = want[0] if isinstance(want, tuple) else want
    diff = (plan.run().float().cpu() - want.float()).abs()
    assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3
    assert plan.device_status() == 0


def test_bound_append_plan_and_decode_replay_in_a_cuda_graph(dev):
    """append + decode captured once and replayed: positions and lengths live on the device, so
    every replay writes the next token and attends to one token more."""

    g = torch.Generator().manual_seed(44)
    batch, q_heads, kv_heads, dim, cap, start = 2, 8, 2, 64, 256, 100
    k = torch.randn(batch, kv_heads, cap, dim, generator=g).bfloat16()
    v = torch.randn(batch, kv_heads, cap, dim, generator=g).bfloat16()
    q_raw = torch.randn(batch, 1, q_heads, dim, generator=g).bfloat16()
    k_new = torch.randn(batch, kv_heads, 1, dim, generator=g).bfloat16()
    v_new = torch.randn(batch, kv_heads, 1, dim, generator=g).bfloat16()
    kd, vd = k.to(dev), v.to(dev)
    lens = torch.full((batch,), start, dtype=torch.int32, device=dev)
    q_dev = torch.empty(batch, 1, q_heads, dim, dtype=torch.bfloat16, device=dev)
    append = sa.AppendKVPlan.build(kd, vd, k_new.to(dev), v_new.to(dev), lens, kv_layout="BHND",
                                   query=q_raw.to(dev), query_out=q_dev, lengths_out=lens)
    plan = sa.ExactDecodePlan.build(q_dev, kd, vd, kv_layout="BHND", seq_lens=lens)
    side = torch.cuda.Stream(device=dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        append.run()
        plan.run()
        side.synchronize()
        lens.fill_(start)                         # undo the warm-up step
        kd.copy_(k)
        vd.copy_(v)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            append.run()
            plan.run()
    steps = 3
    for _ in range(steps):
        graph.replay()
    torch.cuda.synchronize()
    assert lens.cpu().tolist() == [start + steps] * batch
    want_k, want_v = k.clone(), v.clone()
    for t in range(steps):
        torch_port.rope_append(None, k_new, v_new, None, None, want_k, want_v, [start + t] * batch)
    assert torch.equal(kd.cpu(), want_k) and torch.equal(vd.cpu(), want_v)
    n = start + steps
    want = cpu_oracle.exact_decode(q_raw, want_k[:, :, :n].transpose(1, 2).contiguous(),
                                   want_v[:, :, :n].transpose(1, 2).contiguous())
    diff = (plan.output.float().cpu() - want.float()).abs()
    assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3


def test_back_to_back_steps_that_cross_tile_boundaries_match_the_oracle(dev):
    """Append + decode steps launched back to back, with no host synchronisation in between, while
    rows grow across multiples of the kernel's 128-token tile.

    The decode kernel cuts its tile list before the launch's dependency wait from row lengths that
    the append kernel in front of it may still be writing, and checks them after the wait: a row
    whose tile count changed must make it cut the list again.  Every step's output is compared
    with the oracle's loop."""

    g = torch.Generator().manual_seed(91)
    batch, q_heads, kv_heads, dim, cap, steps = 3, 8, 2, 64, 512, 7
    start = [126, 254, 40]                   # rows 0 and 1 cross 128 / 256 at steps 3 and 2
    k = torch.randn(batch, kv_heads, cap, dim, generator=g).bfloat16()
    v = torch.randn(batch, kv_heads, cap, dim, generator=g).bfloat16()
    q_raw = torch.randn(batch, 1, q_heads, dim, generator=g).bfloat16()      # [B, 1, Hq, D]
    k_new = torch.randn(batch, kv_heads, 1, dim, generator=g).bfloat16()
    v_new = torch.randn(batch, kv_heads, 1, dim, generator=g).bfloat16()
    angles = torch.randn(batch, 1, dim // 2, generator=g)
    emb = torch.cat((angles, angles), dim=-1)
    cos, sin = emb.cos().bfloat16(), emb.sin().bfloat16()

    kd, vd = k.to(dev), v.to(dev)
    lens = torch.tensor(start, dtype=torch.int32, device=dev)
    q_rot = torch.empty(batch, 1, q_heads, dim, dtype=torch.bfloat16, device=dev)
    plan = sa.ExactDecodePlan.build(q_rot, kd, vd, kv_layout="BHND", seq_lens=lens)
    append = sa.AppendKVPlan.build(kd, vd, k_new.to(dev), v_new.to(dev), lens, kv_layout="BHND", cos=cos.to(dev),
                                   sin=sin.to(dev), query=q_raw.to(dev), query_out=q_rot, query_layout="BNHD",
                                   lengths_out=lens)
    outs = torch.empty(steps, batch, 1, q_heads, dim, dtype=torch.bfloat16, device=dev)
    for step in range(steps):                # no host sync: the launches queue up behind one another
        append.run()
        outs[step].copy_(plan.run())
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    assert lens.cpu().tolist() == [n + steps for n in start]

    ref_k, ref_v, lengths = k.clone(), v.clone(), list(start)
    for step in range(steps):
        want_q = torch_port.rope_append(q_raw.transpose(1, 2), k_new, v_new, cos, sin, ref_k, ref_v, lengths)
        lengths = [n + 1 for n in lengths]
        want = cpu_oracle.exact_decode(want_q.transpose(1, 2).contiguous(), ref_k, ref_v, kv_layout="BHND",
                                       lengths=torch.tensor(lengths, dtype=torch.int32))
        diff = (outs[step].float().cpu() - want.float()).abs()
        assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3, (step, lengths, float(diff.max()))
    assert torch.equal(kd.cpu(), ref_k) and torch.equal(vd.cpu(), ref_v)
