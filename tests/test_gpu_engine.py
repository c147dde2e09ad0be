"""Engine / service / plan API on the GPU: the reference's public calls, served by the sm_100a kernels."""

from __future__ import annotations

import pytest
import torch

import cases
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
    diff = (got.float().cpu() - want.float().cpu()).abs()
    assert float(diff.max()) <= MAX_ABS and float(diff.mean()) <= MEAN_ABS, (float(diff.max()), float(diff.mean()))


def _policy(q, k, **over):
    base = dict(policy_id="engine-test", model_id="test-model", layer_id=3, dtype="bf16", kv_len_bucket=int(k.shape[1]),
                min_batch=2, heads=int(q.shape[2]), kv_heads=int(k.shape[2]), dim=int(q.shape[3]), block_size=16,
                sink_blocks=1, recent_blocks=2, middle_seed_blocks=3, expected_dense_ms=1.0,
                expected_seed_only_ms=0.5, expected_speedup_vs_dense=2.0)
    base.update(over)
    return sa.Gate0SeedOnlyBatchedPolicy(**base)


def _inputs(dev, batch=4, q_heads=16, kv_heads=2, dim=64, kv_len=512, dtype=torch.bfloat16, seed=11):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(batch, 1, q_heads, dim, generator=g).to(dtype)
    k = torch.randn(batch, kv_len, kv_heads, dim, generator=g).to(dtype)
    v = torch.randn(batch, kv_len, kv_heads, dim, generator=g).to(dtype)
    return (q, k, v), (q.to(dev), k.to(dev), v.to(dev))


def test_exact_native_plan_reuses_buffers_and_tracks_mutation(dev):
    (q, k, v), (qd, kd, vd) = _inputs(dev)
    engine = sa.StreamAttnEngine(policy=_policy(q, k))
    plan = engine.plan(qd, kd, vd, mode="exact_native")
    out, info = plan.run()
    _close(out, cpu_oracle.exact_decode(q, k, v))
    assert plan.uses_fixed_buffers is True and plan.backend == sa.STREAMATTN_EXACT_NATIVE_BACKEND
    assert plan.reason == "explicit_exact_native"
    assert info.backend_used == sa.STREAMATTN_EXACT_NATIVE_BACKEND and info.plan_reason == "planned_exact_native"
    assert (info.batch_size, info.kv_len, info.dtype, info.device) == (4, 512, "bf16", "cuda:0")
    first, pointer = out.clone(), out.data_ptr()
    qd.add_(0.5)
    second = plan.run(return_info=False)
    assert second.data_ptr() == pointer and not torch.equal(first, second)
    _close(second, cpu_oracle.exact_decode(qd.cpu(), k, v))
    alias_out, alias_info = sa.decode(qd, kd, vd, mode="dense", engine=engine)
    _close(alias_out, second)
    assert alias_info.backend_used == sa.STREAMATTN_EXACT_NATIVE_BACKEND


def test_verified_auto_takes_the_seed_only_route_when_the_policy_matches(dev):
    (q, k, v), (qd, kd, vd) = _inputs(dev)
    policy = _policy(q, k)
    engine = sa.StreamAttnEngine(policy=policy, decode_policy=sa.StreamAttnDecodePolicy(min_kv_len_for_gate0_seed_only=1))
    plan = engine.plan(qd, kd, vd, mode="verified_auto", model_id="test-model", layer_id=3)
    assert (plan.backend, plan.reason) == (sa.STREAMATTN_MODE_SEED_ONLY_NATIVE, "verified_policy_match")
    out, info = plan.run()
    tokens = cpu_oracle.seed_indices(seq_len=512, block_size=16, sink_blocks=1, recent_blocks=2,
                                     middle_seed_blocks=3, block_order="recent_first")
    _close(out, cpu_oracle.seed_decode(q, k, v, tokens))
    assert info.backend_used == "gate0_seed_only_batched" and info.seed_only_enabled and info.safety_policy_matched
    assert info.plan_reason == "planned_direct_seed_only"
    assert info.stats == {"batch_size": 4, "heads": 16, "kv_heads": 2, "kv_len": 512, "block_size": 16,
                          "seed_blocks": 6, "total_blocks": 32}
    explicit = engine.plan(qd, kd, vd, mode="seed_only_native", model_id="test-model", layer_id=3)
    assert torch.equal(explicit.run(return_info=False), out)


def test_verified_auto_fails_closed_to_exact_with_the_reason(dev):
    (q, k, v), (qd, kd, vd) = _inputs(dev)
    engine = sa.StreamAttnEngine(policy=_policy(q, k), decode_policy=sa.StreamAttnDecodePolicy(min_kv_len_for_gate0_seed_only=1))
    want = cpu_oracle.exact_decode(q, k, v)
    for kwargs, reason in ((dict(model_id="other-model", layer_id=3), "model_mismatch"),
                           (dict(model_id="test-model", layer_id=9), "layer_mismatch")):
        plan = engine.plan(qd, kd, vd, mode="verified_auto", **kwargs)
        assert plan.backend == sa.STREAMATTN_EXACT_NATIVE_BACKEND and reason in plan.reason
        assert plan.uses_fixed_buffers
        out, info = plan.run()
        _close(out, want)
        assert info.backend_used == sa.STREAMATTN_EXACT_NATIVE_BACKEND and not info.seed_only_enabled
        with pytest.raises(ValueError, match=reason):
            engine.plan(qd, kd, vd, mode="seed_only_native", **kwargs)
    # Default decode policy: 512 tokens is below the 16384-token floor of the seed-only route.
    strict = sa.StreamAttnEngine(policy=_policy(q, k))
    plan = strict.plan(qd, kd, vd, mode="auto", model_id="test-model", layer_id=3)
    assert "kv_len_below_min" in plan.reason
    _close(plan.run(return_info=False), want)


def test_service_run_and_planned_route_on_gpu(dev):
    (q, k, v), (qd, kd, vd) = _inputs(dev)
    policy = _policy(q, k)
    decode_policy = sa.StreamAttnDecodePolicy(min_kv_len_for_gate0_seed_only=1, collect_telemetry_every=0)
    tokens = cpu_oracle.seed_indices(seq_len=512, block_size=16, sink_blocks=1, recent_blocks=2,
                                     middle_seed_blocks=3, block_order="recent_first")
    seed_want = cpu_oracle.seed_decode(q, k, v, tokens)
    exact_want = cpu_oracle.exact_decode(q, k, v)

    service = sa.StreamAttnSeedOnlyDecodeService(policy=policy, decode_policy=decode_policy)
    out, info = service.run(qd, kd, vd, model_id="test-model", layer_id=3, mode="auto")
    _close(out, seed_want)
    assert info.backend_used == "gate0_seed_only_batched"
    again, _ = service.run(qd, kd, vd, model_id="test-model", layer_id=3, mode="auto")
    assert again.data_ptr() == out.data_ptr()                      # cached direct runner, same output buffer
    out, info = service.run(qd, kd, vd, mode="exact_native")
    _close(out, exact_want)
    assert (info.fallback_reason, info.plan_backend) == ("manual_exact_native", "dense")

    wrapper_service = sa.StreamAttnSeedOnlyDecodeService(policy=policy, decode_policy=decode_policy,
                                                         use_planned_direct_seed_only_path=False)
    out, info = wrapper_service.run(qd, kd, vd, model_id="test-model", layer_id=3, mode="auto")
    _close(out, seed_want)
    assert (info.plan_backend, info.plan_reason) == ("gate0_seed_only_batched", "calibrated_gate0_seed_only_batched_policy")
    assert info.runtime_counters == {"backend_counts": {"gate0_seed_only_batched": 1}, "fallback_reasons": {}}

    out, info = sa.stream_attn_seed_only_decode(qd, kd, vd, policy=policy, decode_policy=decode_policy,
                                                model_id="test-model", layer_id=3)
    _close(out, seed_want)
    _close(sa.stream_attn_exact_native_decode(qd, kd, vd), exact_want)


def test_exact_decode_plan_object(dev):
    (q, k, v), (qd, kd, vd) = _inputs(dev, batch=2, kv_len=1024)
    kh, vh = kd.transpose(1, 2).contiguous(), vd.transpose(1, 2).contiguous()
    want = cpu_oracle.exact_decode(q, k, v)
    plan = sa.ExactDecodePlan.build(qd, kh, vh)                    # head-major, like the reference's plan
    _close(plan.run(), want)
    assert plan.backend == "sm100_gqa_exact" and plan.workspace_bytes > 0 and plan.num_splits >= 1
    assert plan.launches_per_run == 1 and plan.device_status() == 0
    forced = sa.ExactDecodePlan.build(qd, kh, vh, num_splits=5)
    assert forced.num_splits == 5 and forced.num_ctas == 5 * 2 * 2
    _close(forced.run_warp_merge(), want)
    bnhd = sa.ExactDecodePlan.build(qd, kd, vd, kv_layout="BNHD", output=torch.empty_like(qd))
    _close(bnhd.run_combined(), want)
    with pytest.raises(ValueError):
        sa.ExactDecodePlan.build(qd, kh, vh, output=torch.empty(1, device=dev))


def test_head_major_buffers_are_recognised_like_the_reference(dev):
    """A promoted head-major cell (B4, Hq16/Hkv2, D64, N16384) passed straight to the engine."""

    g = torch.Generator().manual_seed(3)
    q = torch.randn(4, 1, 16, 64, generator=g).bfloat16()
    kh = torch.randn(4, 2, 16384, 64, generator=g).bfloat16()
    vh = torch.randn(4, 2, 16384, 64, generator=g).bfloat16()
    plan = sa.StreamAttnEngine().plan(q.to(dev), kh.to(dev), vh.to(dev), mode="exact_native")
    assert plan.uses_fixed_buffers and plan.direct_runner.kv_layout == "BHND"
    out, info = plan.run()
    want = cpu_oracle.exact_decode(q, kh, vh, kv_layout="BHND")
    _close(out, want)
    assert info.kv_len == 2   # the reference reports key_cache.shape[1], also for head-major buffers


def test_paged_engine_path(dev):
    case = cases.PAGED_CASES["p16_g8_d64"]
    q, k, v, table, lengths = cases.paged_inputs(case, layout="HND")
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    cache = sa.PagedKVCache(key=k.to(dev), value=v.to(dev), page_table=table.to(dev),
                            sequence_lengths=lengths.to(dev), layout="HND")
    engine = sa.StreamAttnEngine()
    plan = engine.plan(q.to(dev), cache, mode="exact_native")
    assert plan.reason == "explicit_paged_exact_native" and plan.backend == sa.PAGED_EXACT_SM100_BACKEND
    out, info = plan.run()
    _close(out, cpu_oracle.paged_decode(q, k, v, table, lengths, layout="HND"))
    assert info.kv_len == int(lengths.max()) and info.stats["max_pages_per_request"] == case.max_pages
    assert info.stats["workspace_bytes"] == plan.direct_runner.plan.workspace_bytes
    with pytest.raises(ValueError, match="does not yet support paged KV"):
        engine.plan(q.to(dev), cache, mode="seed_only_native")


def test_paged_plan_bound_to_pinned_host_query_and_output(dev):
    """The paged plan, like the exact plan, may read the query from and write the result to pinned
    host memory; the bits equal those of the plan bound to device buffers."""

    g = torch.Generator().manual_seed(9)
    batch, q_heads, kv_heads, dim, page, max_pages = 3, 8, 2, 64, 16, 8
    num_pages = batch * max_pages
    k = torch.randn(num_pages, kv_heads, page, dim, generator=g).bfloat16().to(dev)
    v = torch.randn(num_pages, kv_heads, page, dim, generator=g).bfloat16().to(dev)
    table = torch.randperm(num_pages, generator=g).to(torch.int32).view(batch, max_pages).to(dev)
    lengths = torch.tensor([17, 128, 90], dtype=torch.int32, device=dev)
    cache = sa.PagedKVCache(key=k, value=v, page_table=table, sequence_lengths=lengths, layout="HND")
    q_host = torch.randn(batch, 1, q_heads, dim, generator=g).bfloat16().pin_memory()
    out_host = torch.zeros_like(q_host).pin_memory()
    want = sa.PagedExactDecodePlan.build(q_host.to(dev), cache, validate_metadata=False).run().cpu()
    plan = sa.PagedExactDecodePlan.build(q_host, cache, output=out_host, validate_metadata=False)
    plan.run()
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    assert torch.equal(out_host, want)
