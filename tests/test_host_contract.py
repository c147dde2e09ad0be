"""Host-side routing / policy / split-rule contract, pinned to the reference.

``tests/golden/host_contract.json`` was produced by running the reference's own
functions (see ``tests/golden/make_golden.py``).  These tests need no GPU: they
exercise planning and validation, never a kernel.  Where the reference computes
on CPU tensors this package raises instead (it has no CPU path); that is
asserted explicitly.
"""

from __future__ import annotations

import json
from dataclasses import asdict

import pytest
import torch

import cases
import streamattn_b200 as sa
from streamattn_b200.decode import StreamAttnSeedOnlyDecodeService, _normalize_dtype_name


@pytest.fixture(scope="module")
def golden(golden_dir):
    return json.loads((golden_dir / "host_contract.json").read_text())


def _engine_inputs():
    g = torch.Generator().manual_seed(5)
    q = torch.randn(2, 1, 4, 8, generator=g)
    k = torch.randn(2, 32, 2, 8, generator=g)
    v = torch.randn(2, 32, 2, 8, generator=g)
    return q, k, v


def _test_policy():
    return sa.Gate0SeedOnlyBatchedPolicy(
        policy_id="engine-test", model_id="test-model", layer_id=3, dtype="fp32", kv_len_bucket=32,
        min_batch=2, heads=4, kv_heads=2, dim=8, block_size=8, sink_blocks=1, recent_blocks=1,
        middle_seed_blocks=1, expected_dense_ms=1.0, expected_seed_only_ms=0.5, expected_speedup_vs_dense=2.0,
    )


def _zeros(q, k, v):
    return torch.zeros_like(q)


def test_mode_normalisation(golden):
    for mode, want in golden["normalize_mode"].items():
        assert sa.normalize_stream_attn_mode(mode) == want
    with pytest.raises(ValueError) as err:
        sa.normalize_stream_attn_mode("bogus")
    assert str(err.value) == golden["normalize_mode_error"]
    assert "mode must be one of" in str(err.value)


def test_seq_bucket_and_dtype_names(golden):
    for n, want in golden["seq_bucket"].items():
        assert sa.seq_bucket(int(n)) == want
    for name, want in golden["dtype_names"].items():
        assert _normalize_dtype_name(name) == want
    assert _normalize_dtype_name(torch.bfloat16) == "bf16"
    with pytest.raises(ValueError):
        sa.seq_bucket(0)


def test_split_rules(golden):
    for row in golden["choose_num_splits"]:
        assert sa.choose_num_splits(batch=row["batch"], kv_heads=row["kv_heads"], kv_len=row["kv_len"]) == row["splits"]
    for row in golden["choose_paged_exact_splits"]:
        got = sa.choose_paged_exact_splits(batch=row["batch"], query_heads=row["query_heads"],
                                           max_pages_per_request=row["max_pages_per_request"])
        assert got == row["splits"]
    # Values the reference's tests state outright.
    assert sa.choose_num_splits(batch=2, kv_heads=2, kv_len=32768) == 64
    assert sa.choose_num_splits(batch=8, kv_heads=2, kv_len=32768) == 16
    assert sa.choose_paged_exact_splits(batch=1, query_heads=16, max_pages_per_request=2048) == 32
    assert sa.choose_paged_exact_splits(batch=8, query_heads=16, max_pages_per_request=2048) == 4
    with pytest.raises(ValueError):
        sa.choose_num_splits(batch=1, kv_heads=1, kv_len=100)
    with pytest.raises(ValueError):
        sa.choose_paged_exact_splits(batch=0, query_heads=1, max_pages_per_request=1)


def test_packaged_policies_parse_like_the_reference(golden):
    assert sa.packaged_gate0_seed_only_batched_policy_registry()["default"] == golden["registry_default"]
    assert sa.list_packaged_gate0_seed_only_batched_policies() == golden["policy_names"]
    assert sa.list_packaged_gate0_seed_only_batched_policies(include_aliases=True) == golden["policy_names_with_aliases"]
    for name, want in golden["policies"].items():
        assert asdict(sa.load_packaged_gate0_seed_only_batched_policy(name)) == want, name
    for row in golden["find_policies"]:
        assert sa.find_packaged_gate0_seed_only_batched_policies(**row["query"]) == row["names"], row["query"]
    with pytest.raises(ValueError, match="unknown packaged Gate-0 seed-only policy"):
        sa.load_packaged_gate0_seed_only_batched_policy("nope")


def test_policy_entry_parser_on_reference_format():
    entry = {
        "policy_id": "p", "model": "m", "capture": {"layer_id": 7},
        "shape": {"dtype": "float16", "kv_len": 32768, "batch": 8, "q_heads": 14, "true_kv_heads": 2, "dim": 64},
        "seed_config": {"block_size": 16, "sink_blocks": 0, "recent_blocks": 3, "middle_seed_blocks": 5,
                        "block_order": "sequential"},
        "safety": {"min_top5_overlap": 5, "max_kl": 0.001},
        "quality": {"streamattn_seed_only_ms": 0.03, "flashinfer_tc_ms": 0.06, "speedup": 2.0,
                    "seed_vs_flashinfer_exact": {"max_abs_error": 0.5}},
    }
    p = sa.Gate0SeedOnlyBatchedPolicy.from_entry(entry)
    assert (p.model_id, p.layer_id, p.dtype, p.kv_len_bucket, p.min_batch) == ("m", 7, "fp16", 32768, 8)
    assert (p.heads, p.kv_heads, p.dim) == (14, 2, 64)
    # A zero in the artifact falls through to the default, as in the reference's parser.
    assert (p.block_size, p.sink_blocks, p.recent_blocks, p.middle_seed_blocks) == (16, 2, 3, 5)
    assert (p.expected_seed_only_ms, p.expected_dense_ms, p.expected_speedup_vs_dense) == (0.03, 0.06, 2.0)
    assert p.expected_max_abs_error == 0.5 and p.min_topk_overlap == 5 and p.max_kl == 0.001


def test_policy_validation_errors():
    with pytest.raises(ValueError, match="all_seed_only"):
        sa.Gate0SeedOnlyBatchedPolicy(mode="other")
    with pytest.raises(ValueError, match="block_order"):
        sa.Gate0SeedOnlyBatchedPolicy(block_order="random")
    with pytest.raises(ValueError, match="min_batch"):
        sa.Gate0SeedOnlyBatchedPolicy(min_batch=0)
    with pytest.raises(ValueError, match="safety_margin"):
        sa.StreamAttnDecodePolicy(safety_margin=0.5)


def test_mismatch_reasons(golden):
    policy = sa.Gate0SeedOnlyBatchedPolicy(
        policy_id="golden", model_id="m", layer_id=3, dtype="bf16", kv_len_bucket=32768,
        min_batch=4, heads=16, kv_heads=2, dim=128,
    )
    for name, row in golden["mismatch_reasons"].items():
        sc = row["scenario"]
        dt = getattr(torch, sc["dtype"])
        q = torch.empty(sc["q"], dtype=dt, device="meta")
        k = torch.empty(sc["k"], dtype=dt, device="meta")
        got = policy.mismatch_reasons(q, k, min_kv_len=16384, model_id=sc["model_id"], layer_id=sc["layer_id"],
                                      backend_available=sc.get("backend_available", True))
        assert got == row["reasons"], name


def test_engine_routing_on_cpu_tensors(golden):
    routing = golden["routing"]
    q, k, v = _engine_inputs()
    engine = sa.StreamAttnEngine(policy=_test_policy(), dense_fallback=_zeros,
                                 decode_policy=sa.StreamAttnDecodePolicy(min_kv_len_for_gate0_seed_only=1))

    plan = engine.plan(q, k, v, mode="exact_native")
    want = routing["exact_native"]
    assert (plan.backend, plan.reason, plan.uses_fixed_buffers) == (want["backend"], want["reason"], False)
    out, info = plan.run()
    assert info.to_dict() == want["info"]
    assert torch.equal(out, torch.zeros_like(q))  # came from the injected fallback, not from a CPU path

    plan = engine.plan(q, k, v, mode="verified_auto", model_id="test-model", layer_id=3)
    want = routing["verified_auto_cpu"]
    assert (plan.backend, plan.reason, plan.uses_fixed_buffers) == (want["backend"], want["reason"], False)
    assert "backend_unavailable" in plan.reason
    _, info = plan.run()
    assert info.to_dict() == want["info"]

    plan = engine.plan(q, k, v, mode="auto", model_id="other", layer_id=9)
    assert (plan.backend, plan.reason) == (routing["auto_model_mismatch"]["backend"],
                                           routing["auto_model_mismatch"]["reason"])

    with pytest.raises(ValueError) as err:
        engine.plan(q, k, v, mode="seed_only_native", model_id="test-model", layer_id=3)
    assert str(err.value) == routing["seed_only_native_cpu_error"]
    with pytest.raises(ValueError) as err:
        engine.plan(q, k, None, mode="exact_native")
    assert str(err.value) == routing["missing_value_error"]


def test_no_cpu_execution_path():
    q, k, v = _engine_inputs()
    plan = sa.StreamAttnEngine(policy=_test_policy()).plan(q, k, v, mode="exact_native")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        plan.run()
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        sa.stream_attn_exact_native_decode(q, k, v)
    qf, kf, vf, table, lengths = cases.reference_paged_fixture()
    cache = sa.PagedKVCache(key=kf, value=vf, page_table=table, sequence_lengths=lengths)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        sa.PagedExactDecodePlan.build(qf, cache)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        sa.ExactDecodePlan.build(q, k.transpose(1, 2).contiguous(), v.transpose(1, 2).contiguous())


def test_paged_contract_errors(golden):
    routing = golden["routing"]
    qf, kf, vf, table, lengths = cases.reference_paged_fixture()
    cache = sa.PagedKVCache(key=kf, value=vf, page_table=table, sequence_lengths=lengths)
    assert (cache.num_pages, cache.page_size, cache.kv_heads, cache.head_dim) == (5, 4, 2, 8)
    assert (cache.batch_size, cache.max_pages_per_request, cache.max_sequence_length) == (2, 3, 12)
    cache.validate(qf)

    with pytest.raises(ValueError) as err:
        sa.decode(qf, cache, mode="seed_only_native")
    assert str(err.value) == routing["paged_seed_only_error"]
    assert "does not yet support paged KV" in str(err.value)
    with pytest.raises(ValueError) as err:
        sa.decode(qf, cache, vf, mode="exact_native")
    assert str(err.value) == routing["paged_value_cache_error"]
    assert "value_cache must be omitted" in str(err.value)

    bad_table = table.clone()
    bad_table[1, 2] = 5
    bad_lengths = lengths.clone()
    bad_lengths[0] = 13
    for label, kwargs in {
        "paged_bad_table_error": dict(page_table=bad_table, sequence_lengths=lengths),
        "paged_bad_length_error": dict(page_table=table, sequence_lengths=bad_lengths),
        "paged_zero_length_error": dict(page_table=table, sequence_lengths=torch.tensor([0, 10], dtype=torch.int32)),
    }.items():
        with pytest.raises(ValueError) as err:
            sa.PagedKVCache(key=kf, value=vf, **kwargs).validate(qf)
        assert str(err.value) == routing[label], label
    assert "active page_table" in routing["paged_bad_table_error"]
    assert "exceed page_table capacity" in routing["paged_bad_length_error"]
    # A -1 in an inactive trailing slot is legal; metadata checks can be skipped.
    sa.PagedKVCache(key=kf, value=vf, page_table=bad_table, sequence_lengths=lengths).validate(
        qf, validate_metadata=False)
    with pytest.raises(ValueError, match="layout"):
        sa.PagedKVCache(key=kf, value=vf, page_table=table, sequence_lengths=lengths, layout="XYZ").validate(qf)
    with pytest.raises(ValueError, match="int32 or int64"):
        sa.PagedKVCache(key=kf, value=vf, page_table=table.float(), sequence_lengths=lengths).validate(qf)


def test_service_fail_closed_telemetry(golden):
    q, k, v = _engine_inputs()
    service = StreamAttnSeedOnlyDecodeService(
        policy=_test_policy(), decode_policy=sa.StreamAttnDecodePolicy(min_kv_len_for_gate0_seed_only=1),
        dense_fallback=_zeros,
    )
    calls = {
        "auto_cpu": dict(mode="auto", model_id="test-model", layer_id=3),
        "dense_alias": dict(mode="dense"),
        "exact_native": dict(mode="exact_native"),
        "layer_mismatch": dict(mode="verified_auto", model_id="test-model", layer_id=4),
    }
    for label, kwargs in calls.items():
        out, info = service.run(q, k, v, **kwargs)
        assert info.to_dict() == golden["service_run"][label], label
        assert torch.equal(out, torch.zeros_like(q))
    assert service.run(q, k, v, mode="dense", return_info=False).shape == q.shape


def test_planned_route_decision(golden):
    q, k, _ = _engine_inputs()
    q4, k4 = q.repeat(2, 1, 1, 1), k.repeat(2, 1, 1, 1)
    policy = _test_policy()
    decode_policy = sa.StreamAttnDecodePolicy(min_kv_len_for_gate0_seed_only=1)
    for label, (qq, kk, pol) in {
        "seed_selected": (q4, k4, policy), "no_policy": (q4, k4, None), "min_batch": (q[:1], k[:1], policy),
    }.items():
        plan = sa.stream_attn_decode_plan(qq, kk, gate0_seed_only_batched_policy=pol, policy=decode_policy,
                                          active_fraction_hint=1.0, block_size=16, tile_size_q=16)
        got = asdict(plan)
        got["gate0_seed_only_batched_policy"] = plan.gate0_seed_only_batched_policy is not None
        got.pop("gate0_fused_hybrid_policy")
        assert got == golden["decode_plan"][label], label
    slow = sa.Gate0SeedOnlyBatchedPolicy(**{**asdict(policy), "expected_seed_only_ms": 0.95,
                                            "expected_speedup_vs_dense": None})
    plan = sa.stream_attn_decode_plan(q4, k4, gate0_seed_only_batched_policy=slow, policy=decode_policy,
                                      active_fraction_hint=1.0, block_size=16, tile_size_q=16)
    want = golden["decode_plan"]["not_profitable"]
    assert (plan.backend, plan.reason, plan.fallback_reason) == (want["backend"], want["reason"], want["fallback_reason"])


def test_planned_route_runs_fail_closed_on_cpu():
    q, k, v = _engine_inputs()
    q4, k4, v4 = (t.repeat(2, 1, 1, 1) for t in (q, k, v))
    plan = sa.stream_attn_decode_plan(q4, k4, gate0_seed_only_batched_policy=_test_policy(),
                                      policy=sa.StreamAttnDecodePolicy(min_kv_len_for_gate0_seed_only=1),
                                      active_fraction_hint=1.0, block_size=16, tile_size_q=16)
    assert plan.backend == "gate0_seed_only_batched"
    out, info = sa.stream_attn_decode_run(q4, k4, v4, plan=plan, dense_fallback=_zeros, return_info=True)
    assert (info.backend_used, info.fallback_reason, info.stats) == ("dense", "seed_only_batched_requires_cuda", None)
    assert torch.equal(out, torch.zeros_like(q4))

    workspace = sa.StreamAttnDecodeWorkspace.allocate(device="cpu", max_batch=4, max_query_len=1, max_kv_len=32,
                                                      max_heads=4, head_dim=8, block_size=8, dtype=torch.float32)
    wrapper = sa.StreamAttnDecodeWrapper(workspace, gate0_seed_only_batched_policy=_test_policy(),
                                         policy=sa.StreamAttnDecodePolicy(min_kv_len_for_gate0_seed_only=1),
                                         dense_fallback=_zeros, dense_fallback_backend="custom_dense")
    with pytest.raises(RuntimeError, match="plan"):
        wrapper.run(q4, k4, v4)
    wrapper.plan(query_shape=q4.shape, kv_shape=k4.shape)
    wrapper.run(q4, k4, v4)
    wrapper.run(q4, k4, v4)
    assert wrapper.runtime_counters() == {"backend_counts": {"custom_dense": 2},
                                          "fallback_reasons": {"seed_only_batched_requires_cuda": 2}}
    with pytest.raises(ValueError, match="query shape"):
        wrapper.run(q, k, v)
    with pytest.raises(NotImplementedError):
        sa.stream_attn_decode_plan(q4, k4, router=object())


def test_cost_model_json_round_trip(tmp_path):
    q, k, _ = _engine_inputs()
    key = sa.DecodeCostKey.from_tensors(q, k, block_size=16, tile_size_q=16, num_warps=4, num_stages=3)
    assert (key.device_class, key.dtype, key.kv_bucket, key.kv_heads) == ("cpu", "float32", 32, 2)
    model = sa.DecodeCostModel()
    model.update(key, sa.DecodeCostEntry(dense_ms=2.0))
    path = tmp_path / "cost.json"
    model.to_json(path)
    loaded = sa.DecodeCostModel.from_json(path)
    assert loaded.lookup(key).dense_ms == 2.0
    plan = sa.stream_attn_decode_plan(q, k, decode_cost_model=loaded, block_size=16, tile_size_q=16)
    assert (plan.backend, plan.reason, plan.dense_ms) == ("dense", "dense_fallback", 2.0)
    with pytest.raises(ValueError):
        sa.DecodeCostEntry(dense_ms=0.0)


def test_kv_layout_inference_matches_the_reference_gate():
    def layout(qs, ks, dtype=torch.bfloat16):
        return sa.infer_kv_layout(torch.empty(qs, dtype=dtype, device="meta"),
                                  torch.empty(ks, dtype=dtype, device="meta"))

    # Head-major buffers of the promoted cells are recognised from their shape...
    assert layout((8, 1, 16, 64), (8, 2, 65536, 64)) == "BHND"
    assert layout((4, 1, 32, 128), (4, 8, 32768, 128)) == "BHND"
    assert layout((16, 1, 16, 64), (16, 4, 16384, 64)) == "BHND"
    # ...everything else keeps the public BNHD meaning.
    assert layout((8, 1, 16, 64), (8, 65536, 2, 64)) == "BNHD"
    assert layout((8, 1, 16, 64), (8, 2, 65536, 64), torch.float16) == "BNHD"
    assert layout((3, 1, 16, 64), (3, 2, 65536, 64)) == "BNHD"
    assert layout((1, 1, 16, 64), (1, 4, 65536, 64)) == "BNHD"


def test_seed_only_launcher_failure_falls_closed_to_exact_with_the_reason(monkeypatch):
    """A seed-only launch that raises must not reach the caller when the policy's fallback is
    dense: the service runs exact instead and records ``seed_only_batched_backend_error:<Exc>``
    (reference decode.py:2573-2591; its tests/test_decode_plan.py:649, 1126).  The failure is
    made on the host - the launcher is replaced by one that raises - so no GPU is involved."""

    q, k, v = _engine_inputs()
    service = sa.StreamAttnSeedOnlyDecodeService(
        policy=_test_policy(), decode_policy=sa.StreamAttnDecodePolicy(min_kv_len_for_gate0_seed_only=1),
        dense_fallback=_zeros, use_planned_direct_seed_only_path=True)
    monkeypatch.setattr(service, "_preflight_reasons", lambda *a, **kw: [])   # pretend the device qualifies

    def broken_launcher(*args, **kwargs):
        raise MemoryError("simulated launch failure")

    monkeypatch.setattr(service, "_allocate_direct_runner", broken_launcher)
    out, info = service.run(q, k, v, model_id="test-model", layer_id=3, mode="verified_auto")
    assert torch.equal(out, torch.zeros_like(q))                               # the injected exact path
    assert info.fallback_reason == "seed_only_batched_backend_error:MemoryError"
    assert info.backend_used == sa.STREAMATTN_EXACT_NATIVE_BACKEND
    assert info.runtime_counters["fallback_reasons"] == {"seed_only_batched_backend_error:MemoryError": 1}
    assert info.seed_only_enabled is False
    # Output only: the same fallback, no record.
    assert torch.equal(service.run(q, k, v, model_id="test-model", layer_id=3, mode="auto", return_info=False),
                       torch.zeros_like(q))
    # A policy that forbids the dense fallback lets the error through.
    strict = sa.StreamAttnSeedOnlyDecodeService(
        policy=sa.Gate0SeedOnlyBatchedPolicy(**{**_test_policy().__dict__, "fallback": "error"}),
        decode_policy=sa.StreamAttnDecodePolicy(min_kv_len_for_gate0_seed_only=1), dense_fallback=_zeros,
        use_planned_direct_seed_only_path=True)
    monkeypatch.setattr(strict, "_preflight_reasons", lambda *a, **kw: [])
    monkeypatch.setattr(strict, "_allocate_direct_runner", broken_launcher)
    with pytest.raises(MemoryError):
        strict.run(q, k, v, model_id="test-model", layer_id=3, mode="verified_auto")
