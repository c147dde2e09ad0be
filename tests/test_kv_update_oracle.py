"""CPU tests of the KV-cache update step: the oracle against the reference's stored outputs, and
the host-side page allocator."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import torch_port
from streamattn_b200.kv_update import PagePool
from tests.golden import cases

GOLDEN = Path(__file__).resolve().parent / "golden" / "rope_append_reference_outputs.npz"


@pytest.mark.parametrize("name", list(cases.ROPE_APPEND_CASES))
def test_rope_append_oracle_matches_reference_outputs(name):
    case = cases.ROPE_APPEND_CASES[name]
    golden = np.load(GOLDEN)
    q_raw, k_raw, v_raw, cos, sin, k_cache, v_cache = cases.rope_append_inputs(case)
    k_before, v_before = k_cache.clone(), v_cache.clone()
    positions = case.positions if len(case.positions) > 1 else case.positions * case.batch
    q_rot = torch_port.rope_append(q_raw, k_raw, v_raw, cos, sin, k_cache, v_cache, positions)
    idx, rows = torch.arange(case.batch), torch.tensor(positions)
    # Bit-exact: the stored values are the reference's results widened to float32.
    assert np.array_equal(q_rot.float().numpy(), golden[f"{name}/q_rot"])
    assert np.array_equal(k_cache[idx, :, rows, :].float().numpy(), golden[f"{name}/k_rows"])
    assert np.array_equal(v_cache[idx, :, rows, :].float().numpy(), golden[f"{name}/v_rows"])
    changed = [int((k_cache != k_before).sum()), int((v_cache != v_before).sum())]
    assert changed == golden[f"{name}/changed"].tolist()


def test_paged_rope_append_oracle_agrees_with_contiguous():
    case = cases.ROPE_APPEND_CASES["rows_bf16_d64"]
    q_raw, k_raw, v_raw, cos, sin, k_cache, v_cache = cases.rope_append_inputs(case)
    page = 16
    pages_per_row = case.max_seq // page
    for layout in ("NHD", "HND"):
        table = torch.randperm(case.batch * pages_per_row, generator=torch.Generator().manual_seed(3)).view(case.batch, -1)
        shape = (case.batch * pages_per_row, page, case.kv_heads, case.dim) if layout == "NHD" else \
            (case.batch * pages_per_row, case.kv_heads, page, case.dim)
        kp = torch.zeros(shape, dtype=k_cache.dtype)
        vp = torch.zeros(shape, dtype=k_cache.dtype)
        kc, vc = torch.zeros_like(k_cache), torch.zeros_like(v_cache)
        q1 = torch_port.rope_append(q_raw, k_raw, v_raw, cos, sin, kc, vc, case.positions)
        q2 = torch_port.paged_rope_append(q_raw, k_raw, v_raw, cos, sin, kp, vp, table, case.positions, layout=layout)
        assert torch.equal(q1, q2)
        for b, pos in enumerate(case.positions):
            pid = int(table[b, pos // page])
            got = kp[pid, pos % page] if layout == "NHD" else kp[pid, :, pos % page]
            assert torch.equal(got, kc[b, :, pos])
        assert int((kp != 0).sum()) == int((kc != 0).sum())


def test_page_pool_allocates_lowest_first_and_recycles():
    pool = PagePool(6, reserved=[1, 4])
    assert pool.free_pages == 4
    assert pool.allocate(2) == [0, 2]
    pool.release([0])
    assert pool.allocate(1) == [0]
    assert pool.allocate(2) == [3, 5]
    with pytest.raises(RuntimeError, match="out of KV pages"):
        pool.allocate(1)
    with pytest.raises(ValueError):
        pool.release([7])
    with pytest.raises(ValueError):
        PagePool(4, reserved=[9])


def test_append_kv_has_no_cpu_path():
    from streamattn_b200.kv_update import append_kv

    k = torch.zeros(1, 2, 8, 64)
    new = torch.zeros(1, 2, 1, 64)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        append_kv(k, k.clone(), new, new.clone(), torch.zeros(1, dtype=torch.int64))
