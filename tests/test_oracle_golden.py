"""Pin the CPU oracle against outputs of the reference itself.

The fixtures were produced by ``tests/golden/make_golden.py`` by running the
reference's CPU path on the seeded inputs of ``tests/golden/cases.py``.
"""

from __future__ import annotations

import json

import numpy as np
import pytest
import torch

import cases
from oracle import cpu_oracle, torch_port

# float32 reference outputs vs a double-accumulating restatement.
ATOL = 2e-6
RTOL = 1e-5


def _check_inputs(golden, name, tensors):
    stored = golden[f"{name}/checksum"]
    for i, t in enumerate(tensors):
        assert cases.tensor_checksum(t) == pytest.approx(float(stored[i]), rel=1e-12, abs=1e-9), (
            "seeded input generation drifted from the fixture generator"
        )


@pytest.mark.parametrize("name", list(cases.EXACT_CASES))
def test_exact_oracle_matches_reference_output(golden_exact, name):
    case = cases.EXACT_CASES[name]
    q, k, v = cases.exact_inputs(case)
    _check_inputs(golden_exact, name, (q, k, v))
    expected = torch.from_numpy(golden_exact[f"{name}/out"])
    torch.testing.assert_close(cpu_oracle.exact_decode(q, k, v), expected, atol=ATOL, rtol=RTOL)
    torch.testing.assert_close(torch_port.dense_decode(q, k, v), expected, atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("name", ["g8_d64_n300", "g4_d128_n257"])
def test_exact_oracle_head_major_layout_and_shard_merge(golden_exact, name):
    case = cases.EXACT_CASES[name]
    q, k, v = cases.exact_inputs(case)
    expected = torch.from_numpy(golden_exact[f"{name}/out"])
    kh = k.permute(0, 2, 1, 3).contiguous()
    vh = v.permute(0, 2, 1, 3).contiguous()
    torch.testing.assert_close(
        cpu_oracle.exact_decode(q, kh, vh, kv_layout="BHND"), expected, atol=ATOL, rtol=RTOL
    )
    # Three uneven context shards merged from (o, m, l) states equal the whole.
    cuts = [0, case.kv_len // 3, case.kv_len // 3 + 7, case.kv_len]
    states = [
        cpu_oracle.exact_decode(q, k, v, token_range=(cuts[i], cuts[i + 1]), return_state=True)[1]
        for i in range(3)
    ]
    merged = cpu_oracle.merge_states(
        torch.stack([s.reshape(-1, case.dim + 2) for s in states]), log2_domain=False
    ).reshape(expected.shape)
    torch.testing.assert_close(merged, expected, atol=ATOL, rtol=RTOL)


def test_exact_oracle_row_lengths(golden_exact):
    case = cases.EXACT_CASES["g8_d64_n300"]
    q, k, v = cases.exact_inputs(case)
    lengths = torch.tensor([300, 123])
    got = cpu_oracle.exact_decode(q, k, v, lengths=lengths)
    for b, n in enumerate(lengths.tolist()):
        want = torch_port.dense_decode(q[b : b + 1], k[b : b + 1, :n], v[b : b + 1, :n])
        torch.testing.assert_close(got[b : b + 1], want, atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("layout", ["NHD", "HND"])
def test_paged_oracle_matches_reference_fixture(golden_paged, layout):
    q, k, v, table, lengths = cases.reference_paged_fixture(layout=layout)
    np.testing.assert_array_equal(q.numpy(), golden_paged[f"fixture17_{layout}/q"])
    np.testing.assert_array_equal(k.numpy(), golden_paged[f"fixture17_{layout}/k"])
    expected = torch.from_numpy(golden_paged[f"fixture17_{layout}/out"])
    got, trav = cpu_oracle.paged_decode(q, k, v, table, lengths, layout=layout, return_traversal=True)
    torch.testing.assert_close(got, expected, atol=ATOL, rtol=RTOL)
    assert trav.tolist() == [[3, 0, -1], [1, 4, 2]]
    torch.testing.assert_close(
        torch_port.paged_decode(q, k, v, table, lengths, layout=layout), expected, atol=ATOL, rtol=RTOL
    )


@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("name", list(cases.PAGED_CASES))
def test_paged_oracle_matches_reference_output(golden_paged, name, layout):
    case = cases.PAGED_CASES[name]
    q, k, v, table, lengths = cases.paged_inputs(case, layout=layout)
    stored = golden_paged[f"{name}_{layout}/checksum"]
    assert cases.tensor_checksum(k) == pytest.approx(float(stored[1]), rel=1e-12)
    assert float(table.to(torch.float64).sum()) == float(stored[3])
    expected = torch.from_numpy(golden_paged[f"{name}_{layout}/out"])
    got, trav = cpu_oracle.paged_decode(q, k, v, table, lengths, layout=layout, return_traversal=True)
    torch.testing.assert_close(got, expected, atol=ATOL, rtol=RTOL)
    # Traversal = the active prefix of every table row; -1 slots never visited.
    for b in range(case.batch):
        active = -(-int(lengths[b]) // case.page_size)
        assert trav[b, :active].tolist() == table[b, :active].tolist()
        assert (trav[b, active:] == -1).all()


def test_paged_oracle_rejects_bad_metadata():
    q, k, v, table, lengths = cases.reference_paged_fixture()
    bad = table.clone()
    bad[1, 2] = 5
    with pytest.raises(ValueError):
        cpu_oracle.paged_decode(q, k, v, bad, lengths)
    with pytest.raises(ValueError):
        cpu_oracle.paged_decode(q, k, v, table, torch.tensor([13, 10]))
    with pytest.raises(ValueError):
        cpu_oracle.paged_decode(q, k, v, table, torch.tensor([0, 10]))


def test_seed_index_sets_bit_exact(golden_dir):
    payload = json.loads((golden_dir / "seed_index_sets.json").read_text())
    for row in payload["policy_rule"]:
        assert cpu_oracle.seed_blocks(**row["args"]) == row["blocks"], row["args"]
        assert cpu_oracle.seed_indices(**row["args"]).tolist() == row["tokens"], row["args"]
    for row in payload["explicit_blocks"]:
        got = cpu_oracle.seed_tokens_from_blocks(
            seq_len=row["seq_len"], block_size=row["block_size"], blocks=row["blocks"]
        )
        assert got.tolist() == row["tokens"]


def test_seed_index_reference_test_vectors():
    # stream_attention tests: seq 320 / bs 32 / sink 1 / recent 1 / middle 2 / recent_first.
    seed = cpu_oracle.seed_indices(
        seq_len=320, block_size=32, sink_blocks=1, recent_blocks=1, middle_seed_blocks=2,
        block_order="recent_first",
    ).tolist()
    assert len(seed) == 128 and seed[:3] == [0, 1, 2]
    assert {224, 255, 256, 319} <= set(seed)
    assert cpu_oracle.seed_tokens_from_blocks(seq_len=10, block_size=4, blocks=[2, 0, 2]).tolist() == [
        0, 1, 2, 3, 8, 9,
    ]


@pytest.mark.parametrize("name", list(cases.SEED_CASES))
def test_seed_oracle_matches_reference_output(golden_seed, name):
    case = cases.SEED_CASES[name]
    q, k, v = cases.seed_inputs(case)
    _check_inputs(golden_seed, name, (q, k, v))
    tokens = cpu_oracle.seed_indices(
        seq_len=case.kv_len, block_size=case.block_size, sink_blocks=case.sink_blocks,
        recent_blocks=case.recent_blocks, middle_seed_blocks=case.middle_seed_blocks,
        block_order=case.block_order,
    )
    expected = torch.from_numpy(golden_seed[f"{name}/out"])
    torch.testing.assert_close(cpu_oracle.seed_decode(q, k, v, tokens), expected, atol=ATOL, rtol=RTOL)
    torch.testing.assert_close(torch_port.seed_decode(q, k, v, tokens), expected, atol=ATOL, rtol=RTOL)


def test_seed_oracle_manual_known_answer():
    # Softmax over tokens [0,1,4,5] worked by hand (the reference pins the same
    # construction in its seed-only tests): scores q.k/sqrt(D) with D=1.
    q = torch.tensor([[[[1.0]]]])
    k = torch.tensor([0.0, 1.0, 9.0, 9.0, 2.0, 3.0]).view(1, 6, 1, 1)
    v = torch.tensor([1.0, 2.0, 100.0, 100.0, 3.0, 4.0]).view(1, 6, 1, 1)
    w = torch.softmax(torch.tensor([0.0, 1.0, 2.0, 3.0]), dim=0)
    want = float((w * torch.tensor([1.0, 2.0, 3.0, 4.0])).sum())
    got = cpu_oracle.seed_decode(q, k, v, torch.tensor([0, 1, 4, 5]))
    assert float(got) == pytest.approx(want, rel=1e-6)
