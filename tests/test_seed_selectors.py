"""Seed block / token sets of the product's native host code, bit-exact.

``sa_seed_blocks`` / ``sa_seed_token_indices`` are the integer rule the seed-only
launch itself uses.  They are compared with index sets produced by the
reference's own functions (``tests/golden/seed_index_sets.json``).
"""

from __future__ import annotations

import json

import pytest

import streamattn_b200 as sa


@pytest.fixture(scope="module")
def payload(golden_dir):
    return json.loads((golden_dir / "seed_index_sets.json").read_text())


def test_policy_rule_blocks_and_tokens(payload):
    for row in payload["policy_rule"]:
        assert sa.policy_seed_blocks(**row["args"]) == row["blocks"], row["args"]
        assert sa.seed_indices(**row["args"]).tolist() == row["tokens"], row["args"]


def test_explicit_block_lists(payload):
    for row in payload["explicit_blocks"]:
        got = sa.seed_token_indices_from_blocks(seq_len=row["seq_len"], block_size=row["block_size"],
                                                blocks=row["blocks"])
        assert got.tolist() == row["tokens"]


def test_reference_test_vectors():
    seed = sa.seed_indices(seq_len=320, block_size=32, sink_blocks=1, recent_blocks=1,
                           middle_seed_blocks=2, block_order="recent_first").tolist()
    assert len(seed) == 128 and seed[:3] == [0, 1, 2]
    assert {224, 255, 256, 319} <= set(seed)
    assert sa.seed_token_indices_from_blocks(seq_len=10, block_size=4, blocks=[2, 0, 2]).tolist() == [0, 1, 2, 3, 8, 9]
    # BASELINE config 4 stand-in: packaged 3B schedule at 32K = tokens 0-63 and 32448-32767.
    policy = sa.load_packaged_gate0_seed_only_batched_policy("qwen25_3b_l0_32k_seed_only_batched")
    toks = sa.seed_token_indices_from_blocks(seq_len=32768, block_size=policy.block_size,
                                             blocks=policy.seed_blocks(32768)).tolist()
    assert toks == list(range(64)) + list(range(32448, 32768))


def test_bad_arguments():
    with pytest.raises(ValueError):
        sa.policy_seed_blocks(seq_len=0, block_size=32, sink_blocks=1, recent_blocks=1,
                              middle_seed_blocks=1, block_order="recent_first")
    with pytest.raises(ValueError):
        sa.policy_seed_blocks(seq_len=10, block_size=4, sink_blocks=1, recent_blocks=1,
                              middle_seed_blocks=1, block_order="zigzag")
