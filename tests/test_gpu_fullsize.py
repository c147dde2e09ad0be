"""Full-size configurations of the benchmark, checked on the GPU.

The CPU oracle would need minutes for a whole configuration at these sizes, so every
configuration is checked three ways: (1) the pinned C oracle (``oracle/sa_oracle.c``, double
accumulation) on two full-length (row, KV head) pairs - seconds of CPU each; (2) all rows
against a float32 torch formula evaluated on the same GPU; (3) size-independent properties of
exact attention: invariance to the split count, linearity in V, and shard states merging to the
unsharded result.  Tolerance: max-abs 2e-2, mean-abs 2e-3 (bf16 outputs vs fp32).
"""

from __future__ import annotations

import math

import pytest
import torch

import streamattn_b200 as sa
from oracle import cpu_oracle
from streamattn_b200 import native

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
MEAN_ABS = 2e-3


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; refusing to skip")
    return torch.device("cuda:0")


def _close(got, want):
    diff = (got.float() - want.float()).abs()
    assert torch.isfinite(got.float()).all()
    assert float(diff.max()) <= MAX_ABS and float(diff.mean()) <= MEAN_ABS, (float(diff.max()), float(diff.mean()))


def torch_reference(q, k_bhnd, v_bhnd, lengths=None):
    """softmax(q K^T / sqrt(D)) V in float32, one (row, kv head) at a time."""

    batch, _, q_heads, dim = q.shape
    kv_heads = k_bhnd.shape[1]
    group = q_heads // kv_heads
    out = torch.empty(batch, 1, q_heads, dim, dtype=torch.float32, device=q.device)
    for b in range(batch):
        n = int(lengths[b]) if lengths is not None else k_bhnd.shape[2]
        for h in range(kv_heads):
            qg = q[b, 0, h * group:(h + 1) * group].float()
            scores = qg @ k_bhnd[b, h, :n].float().T / math.sqrt(dim)
            out[b, 0, h * group:(h + 1) * group] = torch.softmax(scores, dim=-1) @ v_bhnd[b, h, :n].float()
    return out


def oracle_pairs(out, q, k_bhnd, v_bhnd, pairs, lengths=None):
    """Compare the kernel's output rows of the given (row, kv head) pairs with the C oracle."""

    group = q.shape[2] // k_bhnd.shape[1]
    for b, h in pairs:
        n = int(lengths[b]) if lengths is not None else k_bhnd.shape[2]
        heads = slice(h * group, (h + 1) * group)
        want = cpu_oracle.exact_decode(q[b:b + 1, :, heads].float().cpu(), k_bhnd[b:b + 1, h:h + 1, :n].float().cpu(),
                                       v_bhnd[b:b + 1, h:h + 1, :n].float().cpu(), kv_layout="BHND")
        diff = (out[b:b + 1, :, heads].float().cpu() - want).abs()
        assert float(diff.max()) <= MAX_ABS and float(diff.mean()) <= MEAN_ABS, (b, h, float(diff.max()))


def _randn(shape, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    return torch.randn(shape, generator=g, device=dev, dtype=torch.float32).bfloat16()


def test_config2_exact_contiguous_b8_n65536(dev):
    batch, q_heads, kv_heads, dim, kv_len = 8, 16, 2, 64, 65536
    q = _randn((batch, 1, q_heads, dim), 0, dev)
    k = _randn((batch, kv_heads, kv_len, dim), 1, dev)
    v = _randn((batch, kv_heads, kv_len, dim), 2, dev)
    want = torch_reference(q, k, v)
    plan = sa.ExactDecodePlan.build(q, k, v)
    assert plan.kernel_name == "sm100_tma_mma_stream"
    out = plan.run().clone()
    assert plan.device_status() == 0
    _close(out, want)
    oracle_pairs(out, q, k, v, [(0, 0), (batch - 1, kv_heads - 1)])
    assert torch.equal(plan.run(), out)                             # deterministic replay
    # BNHD view of the same values gives the same answer.
    kb, vb = k.transpose(1, 2).contiguous(), v.transpose(1, 2).contiguous()
    bnhd = sa.ExactDecodePlan.build(q, kb, vb, kv_layout="BNHD")
    first_bnhd = bnhd.run().clone()
    _close(first_bnhd, want)
    assert torch.equal(bnhd.run(), first_bnhd)                      # the round-robin schedule is static too
    # Dynamic schedule (tiles claimed from a device counter): same answer within tolerance on
    # every launch, counters left clean for the next one.
    for layout, kk, vv in (("BHND", k, v), ("BNHD", kb, vb)):
        dyn = sa.ExactDecodePlan.build(q, kk, vv, kv_layout=layout, dynamic_schedule=True)
        for _ in range(3):
            _close(dyn.run(), want)
        assert dyn.device_status() == 0
    # Split-count invariance and linearity in V.
    _close(sa.ExactDecodePlan.build(q, k, v, num_splits=3).run(), want)
    v2 = (v.float() * 2).bfloat16()
    _close(sa.ExactDecodePlan.build(q, k, v2).run().float() / 2, want)
    # Two context shards merged from their (o, m, l) states equal the whole.
    half = kv_len // 2
    states = []
    for lo, hi in ((0, half), (half, kv_len)):
        st = torch.empty(batch, q_heads, dim + 2, dtype=torch.float32, device=dev)
        ws = native.new_workspace(dev, batch, q_heads, kv_heads, dim)
        native.exact_plan(q, k[:, :, lo:hi], v[:, :, lo:hi], st, ws, kv_layout="BHND", out_state=True).run()
        states.append(st.view(-1, dim + 2))
    merged = torch.empty_like(q)
    native.merge_states(torch.stack(states).contiguous(), merged)
    _close(merged, want)


def test_config3_paged_page16_ragged(dev):
    batch, q_heads, kv_heads, dim, page, cap = 8, 16, 2, 64, 16, 65536
    max_pages = cap // page
    pool = batch * max_pages
    g = torch.Generator().manual_seed(17)
    q = _randn((batch, 1, q_heads, dim), 3, dev)
    k = _randn((pool, kv_heads, page, dim), 4, dev)
    v = _randn((pool, kv_heads, page, dim), 5, dev)
    table = torch.randperm(pool, generator=g).to(torch.int32).view(batch, max_pages)
    lengths = torch.randint(16384, 65537, (batch,), generator=g).to(torch.int32)
    for b in range(batch):
        table[b, -(-int(lengths[b]) // page):] = -1
    cache = sa.PagedKVCache(key=k, value=v, page_table=table.to(dev), sequence_lengths=lengths.to(dev), layout="HND")
    plan = sa.PagedExactDecodePlan.build(q, cache, record_page_walk=True)
    assert plan.backend == sa.PAGED_EXACT_SM100_BACKEND
    out = plan.run()
    assert plan.device_status() == 0
    # Reference: gather each row's pages into a contiguous cache, then dense softmax.
    kc = torch.zeros(batch, kv_heads, cap, dim, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    for b in range(batch):
        active = -(-int(lengths[b]) // page)
        ids = table[b, :active].long().to(dev)
        kc[b, :, : active * page] = k[ids].permute(1, 0, 2, 3).reshape(kv_heads, active * page, dim)
        vc[b, :, : active * page] = v[ids].permute(1, 0, 2, 3).reshape(kv_heads, active * page, dim)
    _close(out, torch_reference(q, kc, vc, lengths))
    shortest, longest = int(lengths.argmin()), int(lengths.argmax())
    oracle_pairs(out, q, kc, vc, [(shortest, 0), (longest, kv_heads - 1)], lengths)
    # Bit-exact page walk: every active slot visited with its own physical page, -1 slots untouched.
    assert torch.equal(plan.trace.cpu(), table)
    # Dynamic schedule: within tolerance on every launch, same page walk.
    dyn = sa.PagedExactDecodePlan.build(q, cache, record_page_walk=True, dynamic_schedule=True)
    for _ in range(3):
        _close(dyn.run(), out.float())
    assert dyn.device_status() == 0
    assert torch.equal(dyn.trace.cpu(), table)
    # The same values through an int64 table and a forced split count.
    cache64 = sa.PagedKVCache(key=k, value=v, page_table=table.to(dev).long(), sequence_lengths=lengths.to(dev).long(),
                              layout="HND")
    assert torch.equal(sa.PagedExactDecodePlan.build(q, cache64).run(), out)


def test_config4_seed_only_qwen_shape(dev):
    batch, q_heads, kv_heads, dim, kv_len = 8, 16, 2, 128, 32768
    q = _randn((batch, 1, q_heads, dim), 6, dev)
    k = _randn((batch, kv_len, kv_heads, dim), 7, dev)
    v = _randn((batch, kv_len, kv_heads, dim), 8, dev)
    policy = sa.Gate0SeedOnlyBatchedPolicy(
        policy_id="c4", model_id="m", layer_id=0, dtype="bf16", kv_len_bucket=32768, min_batch=4, heads=16,
        kv_heads=2, dim=128, block_size=32, sink_blocks=2, recent_blocks=2, middle_seed_blocks=8,
        expected_dense_ms=0.1, expected_seed_only_ms=0.03)
    engine = sa.StreamAttnEngine(policy=policy)
    plan = engine.plan(q, k, v, mode="verified_auto", model_id="m", layer_id=0)
    assert plan.reason == "verified_policy_match"
    out, info = plan.run()
    tokens = sa.seed_indices(seq_len=kv_len, block_size=32, sink_blocks=2, recent_blocks=2, middle_seed_blocks=8,
                             block_order="recent_first").to(dev)
    assert tokens.tolist() == list(range(64)) + list(range(32448, 32768))
    ks = k.index_select(1, tokens).transpose(1, 2)
    vs = v.index_select(1, tokens).transpose(1, 2)
    _close(out, torch_reference(q, ks, vs))
    oracle_pairs(out, q, ks, vs, [(0, 0), (batch - 1, kv_heads - 1)])
    assert info.stats["seed_blocks"] == 12 and info.stats["total_blocks"] == 1024


def test_config5_shape_family_d128_g4_long_context(dev):
    """Context-parallel shape (Hq32/Hkv8/D128) on one GPU: 8 shards of a 262144-token row."""

    q_heads, kv_heads, dim, kv_len, shards = 32, 8, 128, 262144, 8
    q = _randn((1, 1, q_heads, dim), 9, dev)
    k = _randn((1, kv_heads, kv_len, dim), 10, dev)
    v = _randn((1, kv_heads, kv_len, dim), 11, dev)
    want = torch_reference(q, k, v)
    whole = sa.ExactDecodePlan.build(q, k, v).run()
    _close(whole, want)
    oracle_pairs(whole, q, k, v, [(0, 0), (0, kv_heads - 1)])
    from streamattn_b200.context_parallel import shard_bounds

    states = []
    for r in range(shards):
        lo, hi = shard_bounds(kv_len, shards, r)
        st = torch.empty(1, q_heads, dim + 2, dtype=torch.float32, device=dev)
        ws = native.new_workspace(dev, 1, q_heads, kv_heads, dim)
        native.exact_plan(q, k[:, :, lo:hi], v[:, :, lo:hi], st, ws, kv_layout="BHND", out_state=True).run()
        states.append(st.view(-1, dim + 2))
    merged = torch.empty_like(q)
    native.merge_states(torch.stack(states).contiguous(), merged)
    _close(merged, want)


def test_result_bits_do_not_depend_on_which_cta_merges(dev, monkeypatch):
    """The split states of a pair are summed in slot order with the merging CTA's own state at its
    slot position, so the two ways of choosing the merging CTA - the pair's first CTA, or the last
    one to arrive by ticket (`STREAMATTN_B200_MERGER=ticket`, read when a plan is built) - must
    give bit-identical outputs, on uniform and on ragged rows."""

    batch, q_heads, kv_heads, dim, kv_len = 4, 16, 2, 64, 16384
    q = _randn((batch, 1, q_heads, dim), 40, dev)
    k = _randn((batch, kv_heads, kv_len, dim), 41, dev)
    v = _randn((batch, kv_heads, kv_len, dim), 42, dev)
    lens = torch.tensor([16384, 9000, 12345, 4097], dtype=torch.int32, device=dev)
    outs = {}
    for form in ("first", "ticket"):
        if form == "ticket":
            monkeypatch.setenv("STREAMATTN_B200_MERGER", "ticket")
        else:
            monkeypatch.delenv("STREAMATTN_B200_MERGER", raising=False)
        uniform = sa.ExactDecodePlan.build(q, k, v)
        ragged = sa.ExactDecodePlan.build(q, k, v, seq_lens=lens)
        outs[form] = (uniform.run().clone(), ragged.run().clone())
        assert uniform.device_status() == 0 and ragged.device_status() == 0
    assert torch.equal(outs["first"][0], outs["ticket"][0])
    assert torch.equal(outs["first"][1], outs["ticket"][1])
    _close(outs["first"][0], torch_reference(q, k, v))
