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


def _cpu_writer(lengths, page=4, max_pages=3, num_pages=5):
    from streamattn_b200 import PagedKVCache
    from streamattn_b200.kv_update import PagedKVWriter, PagePool

    pool = PagePool(num_pages)
    table = torch.full((len(lengths), max_pages), -1, dtype=torch.int32)
    for b, n in enumerate(lengths):
        ids = pool.allocate(-(-n // page))
        table[b, : len(ids)] = torch.tensor(ids, dtype=torch.int32)
    cache = PagedKVCache(key=torch.zeros(num_pages, page, 1, 8), value=torch.zeros(num_pages, page, 1, 8),
                         page_table=table, sequence_lengths=torch.tensor(lengths, dtype=torch.int32), layout="NHD")
    return PagedKVWriter.attach(cache, pool), pool, cache


def test_failed_reserve_leaves_pool_mirrors_and_table_untouched():
    # rows hold 4 and 8 tokens = 1 + 2 pages of 5; the next token needs a page for each row, 2 are free
    writer, pool, cache = _cpu_writer([4, 8], max_pages=4)
    assert writer.reserve(1) == 2 and pool.free_pages == 0
    writer.lengths = [8, 12]  # both rows full again: each needs another page, none is free
    before = (pool.free_pages, [list(p) for p in writer.pages], cache.page_table.clone())
    with pytest.raises(RuntimeError, match="out of KV pages"):
        writer.reserve(1)
    assert (pool.free_pages, writer.pages) == before[:2] and torch.equal(cache.page_table, before[2])
    # capacity: row 1 would need a fourth table slot; row 0's need must not have been taken first
    writer2, pool2, cache2 = _cpu_writer([4, 12], num_pages=8)
    free = pool2.free_pages
    with pytest.raises(ValueError, match="exceed page_table capacity"):
        writer2.reserve(1)
    assert pool2.free_pages == free and [len(p) for p in writer2.pages] == [1, 3]


def test_release_resets_the_row_on_host_and_device_tensors():
    writer, pool, cache = _cpu_writer([4, 8])
    writer.release(1)
    assert writer.lengths == [4, 0] and writer.pages[1] == [] and pool.free_pages == 4
    assert cache.sequence_lengths.tolist() == [4, 0] and cache.page_table[1].tolist() == [-1, -1, -1]
