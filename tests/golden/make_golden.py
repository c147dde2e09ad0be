"""Generate the golden fixtures in this directory from the reference itself.

Run in a container where the StreamAttn reference checkout is importable:

    python tests/golden/make_golden.py --reference /path/to/StreamAttn

The script imports the reference's ``stream_attention`` package (CPU only),
feeds it the seeded inputs of ``cases.py`` and stores what it returns.  The
fixtures are what pins the CPU oracle (``oracle/``) and the host-side routing
logic of ``streamattn_b200``; the GPU box never needs the reference.
"""

from __future__ import annotations

import argparse
import json
import sys
from dataclasses import asdict
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))

import cases  # noqa: E402


def _np(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def exact_goldens(ref) -> None:
    out = {}
    for name, case in cases.EXACT_CASES.items():
        q, k, v = cases.exact_inputs(case)
        engine = ref.StreamAttnEngine()
        result, info = engine.plan(q, k, v, mode="exact_native").run()
        assert info.backend_used == "streamattn_exact_native"
        out[f"{name}/out"] = _np(result.float())
        out[f"{name}/checksum"] = np.array(
            [cases.tensor_checksum(q), cases.tensor_checksum(k), cases.tensor_checksum(v)]
        )
    np.savez_compressed(HERE / "exact_reference_outputs.npz", **out)


def paged_goldens(ref) -> None:
    out = {}
    for layout in ("NHD", "HND"):
        q, k, v, table, lengths = cases.reference_paged_fixture(layout=layout)
        cache = ref.PagedKVCache(key=k, value=v, page_table=table, sequence_lengths=lengths, layout=layout)
        out[f"fixture17_{layout}/out"] = _np(ref.paged_exact_reference(q, cache))
        out[f"fixture17_{layout}/q"] = _np(q)
        out[f"fixture17_{layout}/k"] = _np(k)
        out[f"fixture17_{layout}/v"] = _np(v)
    for name, case in cases.PAGED_CASES.items():
        for layout in ("NHD", "HND"):
            q, k, v, table, lengths = cases.paged_inputs(case, layout=layout)
            cache = ref.PagedKVCache(key=k, value=v, page_table=table, sequence_lengths=lengths, layout=layout)
            out[f"{name}_{layout}/out"] = _np(ref.paged_exact_reference(q, cache))
            out[f"{name}_{layout}/checksum"] = np.array(
                [cases.tensor_checksum(q), cases.tensor_checksum(k), cases.tensor_checksum(v),
                 float(table.to(torch.float64).sum()), float(lengths.sum())]
            )
    np.savez_compressed(HERE / "paged_reference_outputs.npz", **out)


def seed_goldens(ref, ref_root: Path) -> None:
    from stream_attention.seed_selectors import (
        policy_seed_blocks,
        seed_indices,
        seed_token_indices_from_blocks,
    )

    index_rows = []
    for seq_len, bs, sink, recent, middle, order in cases.SEED_INDEX_GRID:
        kwargs = dict(seq_len=seq_len, block_size=bs, sink_blocks=sink, recent_blocks=recent,
                      middle_seed_blocks=middle, block_order=order)
        index_rows.append({
            "args": kwargs,
            "blocks": [int(b) for b in policy_seed_blocks(**kwargs)],
            "tokens": [int(t) for t in seed_indices(**kwargs).tolist()],
        })
    explicit = []
    for seq_len, bs, blocks in [(10, 4, [2, 0, 2]), (100, 16, [6, 1, 0, 5]), (64, 16, [3, 9, 0]),
                                (32768, 16, [0, 1, 2, 3, 777, 1200, 90, 1999, *range(2032, 2048)])]:
        toks = seed_token_indices_from_blocks(seq_len=seq_len, block_size=bs, blocks=blocks,
                                              device=torch.device("cpu"))
        explicit.append({"seq_len": seq_len, "block_size": bs, "blocks": list(blocks),
                         "tokens": [int(t) for t in toks.tolist()]})
    (HERE / "seed_index_sets.json").write_text(
        json.dumps({"policy_rule": index_rows, "explicit_blocks": explicit}, indent=1) + "\n"
    )

    sys.path.insert(0, str(ref_root))
    from benchmarks.profile_seed_only_route_bundle_decode import (
        _fixed_seed_attention_reference_bhnd,
    )

    out = {}
    for name, case in cases.SEED_CASES.items():
        q, k, v = cases.seed_inputs(case)
        policy = ref.Gate0SeedOnlyBatchedPolicy(
            block_size=case.block_size, sink_blocks=case.sink_blocks, recent_blocks=case.recent_blocks,
            middle_seed_blocks=case.middle_seed_blocks, block_order=case.block_order,
        )
        q_bhmd = q.permute(0, 2, 1, 3).contiguous()
        k_bhnd = k.permute(0, 2, 1, 3).contiguous()
        v_bhnd = v.permute(0, 2, 1, 3).contiguous()
        result = torch.empty_like(q)
        _fixed_seed_attention_reference_bhnd(q_bhmd, k_bhnd, v_bhnd, seq_len=case.kv_len,
                                             policy=policy, out=result)
        out[f"{name}/out"] = _np(result)
        out[f"{name}/checksum"] = np.array(
            [cases.tensor_checksum(q), cases.tensor_checksum(k), cases.tensor_checksum(v)]
        )
    np.savez_compressed(HERE / "seed_reference_outputs.npz", **out)


def _info_dict(info) -> dict:
    return json.loads(json.dumps(info.to_dict(), default=str))


def host_contract_goldens(ref) -> None:
    from stream_attention.backends.sm90.transposed_gqa_exact import choose_num_splits
    from stream_attention.decode import StreamAttnSeedOnlyDecodeService, _normalize_dtype_name
    from stream_attention.telemetry import seq_bucket

    payload: dict = {}
    payload["normalize_mode"] = {m: ref.normalize_stream_attn_mode(m)
                                 for m in ["auto", "dense", "exact_native", "seed_only_native", "verified_auto"]}
    try:
        ref.normalize_stream_attn_mode("bogus")
    except ValueError as exc:
        payload["normalize_mode_error"] = str(exc)
    payload["seq_bucket"] = {str(n): seq_bucket(n) for n in [1, 2, 3, 31, 32, 33, 16384, 32767, 32768, 32769, 65536]}
    payload["dtype_names"] = {str(k): _normalize_dtype_name(k) for k in
                              ["float16", "half", "bf16", "bfloat16", "torch.float32", "fp32", "int8"]}
    payload["choose_num_splits"] = [
        {"batch": b, "kv_heads": h, "kv_len": n, "splits": choose_num_splits(batch=b, kv_heads=h, kv_len=n)}
        for b in (1, 2, 4, 8, 16, 64) for h in (1, 2, 8) for n in (64, 4096, 32768, 65536)
    ]
    payload["choose_paged_exact_splits"] = [
        {"batch": b, "query_heads": h, "max_pages_per_request": p,
         "splits": ref.choose_paged_exact_splits(batch=b, query_heads=h, max_pages_per_request=p)}
        for b in (1, 4, 8, 32) for h in (4, 16, 32) for p in (1, 3, 64, 2048, 4096)
    ]

    # Packaged policy cells, parsed by the reference's own loader.
    registry = ref.packaged_gate0_seed_only_batched_policy_registry()
    payload["registry_default"] = registry.get("default")
    payload["policy_names"] = ref.list_packaged_gate0_seed_only_batched_policies()
    payload["policy_names_with_aliases"] = ref.list_packaged_gate0_seed_only_batched_policies(include_aliases=True)
    payload["policies"] = {
        name: asdict(ref.load_packaged_gate0_seed_only_batched_policy(name))
        for name in payload["policy_names_with_aliases"]
    }
    payload["registry_entries"] = [
        {k: entry.get(k) for k in ("name", "policy_id", "aliases", "status", "model_id", "layer_id",
                                   "dtype", "kv_len_bucket", "min_batch")}
        for entry in registry.get("policies") or []
    ]
    payload["find_policies"] = [
        {"query": q, "names": ref.find_packaged_gate0_seed_only_batched_policies(**q)}
        for q in [
            {},
            {"model_id": "Qwen/Qwen2.5-3B-Instruct"},
            {"model_id": "Qwen/Qwen2.5-3B-Instruct", "layer_id": 0},
            {"dtype": "float16", "kv_len_bucket": 32768, "min_batch": 4},
            {"model_id": "Qwen/Qwen2.5-0.5B-Instruct", "min_batch": 2},
            {"status": None},
        ]
    ]

    # Policy mismatch reasons on shape-only (meta) tensors.
    policy = ref.Gate0SeedOnlyBatchedPolicy(
        policy_id="golden", model_id="m", layer_id=3, dtype="bf16", kv_len_bucket=32768,
        min_batch=4, heads=16, kv_heads=2, dim=128,
    )
    scenarios = {
        "match": dict(q=(8, 1, 16, 128), k=(8, 32768, 2, 128), dtype="bfloat16", model_id="m", layer_id=3),
        "model_layer": dict(q=(8, 1, 16, 128), k=(8, 32768, 2, 128), dtype="bfloat16", model_id="x", layer_id=4),
        "batch_small": dict(q=(2, 1, 16, 128), k=(2, 32768, 2, 128), dtype="bfloat16", model_id="m", layer_id=3),
        "short_kv": dict(q=(8, 1, 16, 128), k=(8, 4096, 2, 128), dtype="bfloat16", model_id="m", layer_id=3),
        "bucket": dict(q=(8, 1, 16, 128), k=(8, 65536, 2, 128), dtype="bfloat16", model_id="m", layer_id=3),
        "dtype": dict(q=(8, 1, 16, 128), k=(8, 32768, 2, 128), dtype="float16", model_id="m", layer_id=3),
        "heads": dict(q=(8, 1, 32, 64), k=(8, 32768, 4, 64), dtype="bfloat16", model_id="m", layer_id=3),
        "gqa": dict(q=(8, 1, 16, 128), k=(8, 32768, 3, 128), dtype="bfloat16", model_id="m", layer_id=3),
        "rank": dict(q=(8, 16, 128), k=(8, 32768, 2, 128), dtype="bfloat16", model_id="m", layer_id=3),
        "qlen": dict(q=(8, 2, 16, 128), k=(8, 32768, 2, 128), dtype="bfloat16", model_id="m", layer_id=3),
        "backend": dict(q=(8, 1, 16, 128), k=(8, 32768, 2, 128), dtype="bfloat16", model_id="m", layer_id=3,
                        backend_available=False),
    }
    rows = {}
    for name, sc in scenarios.items():
        dt = getattr(torch, sc["dtype"])
        qm = torch.empty(sc["q"], dtype=dt, device="meta")
        km = torch.empty(sc["k"], dtype=dt, device="meta")
        rows[name] = {
            "scenario": {k: (list(v) if isinstance(v, tuple) else v) for k, v in sc.items()},
            "reasons": policy.mismatch_reasons(
                qm, km, min_kv_len=16384, model_id=sc["model_id"], layer_id=sc["layer_id"],
                backend_available=sc.get("backend_available", True)),
        }
    payload["mismatch_reasons"] = rows

    # Engine routing on CPU tensors (reasons/backends only; numbers live elsewhere).
    g = torch.Generator().manual_seed(5)
    q = torch.randn(2, 1, 4, 8, generator=g)
    k = torch.randn(2, 32, 2, 8, generator=g)
    v = torch.randn(2, 32, 2, 8, generator=g)
    test_policy = ref.Gate0SeedOnlyBatchedPolicy(
        policy_id="engine-test", model_id="test-model", layer_id=3, dtype="fp32", kv_len_bucket=32,
        min_batch=2, heads=4, kv_heads=2, dim=8, block_size=8, sink_blocks=1, recent_blocks=1,
        middle_seed_blocks=1, expected_dense_ms=1.0, expected_seed_only_ms=0.5, expected_speedup_vs_dense=2.0,
    )
    engine = ref.StreamAttnEngine(policy=test_policy,
                                  decode_policy=ref.StreamAttnDecodePolicy(min_kv_len_for_gate0_seed_only=1))
    routing = {}
    plan = engine.plan(q, k, v, mode="exact_native")
    _, info = plan.run()
    routing["exact_native"] = {"backend": plan.backend, "reason": plan.reason,
                               "uses_fixed_buffers": plan.uses_fixed_buffers, "info": _info_dict(info)}
    plan = engine.plan(q, k, v, mode="verified_auto", model_id="test-model", layer_id=3)
    _, info = plan.run()
    routing["verified_auto_cpu"] = {"backend": plan.backend, "reason": plan.reason,
                                    "uses_fixed_buffers": plan.uses_fixed_buffers, "info": _info_dict(info)}
    plan = engine.plan(q, k, v, mode="auto", model_id="other", layer_id=9)
    routing["auto_model_mismatch"] = {"backend": plan.backend, "reason": plan.reason}
    try:
        engine.plan(q, k, v, mode="seed_only_native", model_id="test-model", layer_id=3)
    except ValueError as exc:
        routing["seed_only_native_cpu_error"] = str(exc)
    try:
        engine.plan(q, k, None, mode="exact_native")
    except ValueError as exc:
        routing["missing_value_error"] = str(exc)

    qf, kf, vf, table, lengths = cases.reference_paged_fixture(layout="NHD")
    cache = ref.PagedKVCache(key=kf, value=vf, page_table=table, sequence_lengths=lengths, layout="NHD")
    out, info = ref.decode(qf, cache, mode="verified_auto")
    routing["paged_verified_auto"] = {"info": _info_dict(info)}
    plan = ref.StreamAttnEngine().plan(qf, cache, mode="exact_native")
    routing["paged_exact_native"] = {"backend": plan.backend, "reason": plan.reason}
    for label, call in {
        "paged_seed_only_error": lambda: ref.decode(qf, cache, mode="seed_only_native"),
        "paged_value_cache_error": lambda: ref.decode(qf, cache, vf, mode="exact_native"),
    }.items():
        try:
            call()
        except ValueError as exc:
            routing[label] = str(exc)
    bad_table = table.clone()
    bad_table[1, 2] = 5
    bad_lengths = lengths.clone()
    bad_lengths[0] = 13
    for label, kwargs in {
        "paged_bad_table_error": dict(page_table=bad_table, sequence_lengths=lengths),
        "paged_bad_length_error": dict(page_table=table, sequence_lengths=bad_lengths),
        "paged_zero_length_error": dict(page_table=table, sequence_lengths=torch.tensor([0, 10], dtype=torch.int32)),
    }.items():
        try:
            ref.PagedKVCache(key=kf, value=vf, layout="NHD", **kwargs).validate(qf)
        except ValueError as exc:
            routing[label] = str(exc)
    payload["routing"] = routing

    # Service-level fail-closed telemetry on CPU tensors.
    service = StreamAttnSeedOnlyDecodeService(
        policy=test_policy, decode_policy=ref.StreamAttnDecodePolicy(min_kv_len_for_gate0_seed_only=1),
        dense_fallback=lambda a, b, c: torch.zeros_like(a),
    )
    svc = {}
    for label, kwargs in {
        "auto_cpu": dict(mode="auto", model_id="test-model", layer_id=3),
        "dense_alias": dict(mode="dense"),
        "exact_native": dict(mode="exact_native"),
        "layer_mismatch": dict(mode="verified_auto", model_id="test-model", layer_id=4),
    }.items():
        _, info = service.run(q, k, v, **kwargs)
        svc[label] = _info_dict(info)
    payload["service_run"] = svc

    # Planned route: dense vs gate0_seed_only_batched decision.
    plans = {}
    q4 = q.repeat(2, 1, 1, 1)
    k4 = k.repeat(2, 1, 1, 1)
    for label, (qq, kk, pol) in {
        "seed_selected": (q4, k4, test_policy),
        "no_policy": (q4, k4, None),
        "min_batch": (q[:1], k[:1], test_policy),
    }.items():
        p = ref.stream_attn_decode_plan(
            qq, kk, gate0_seed_only_batched_policy=pol,
            policy=ref.StreamAttnDecodePolicy(min_kv_len_for_gate0_seed_only=1),
            active_fraction_hint=1.0, block_size=16, tile_size_q=16,
        )
        d = asdict(p)
        d["gate0_seed_only_batched_policy"] = p.gate0_seed_only_batched_policy is not None
        d.pop("gate0_fused_hybrid_policy", None)
        plans[label] = d
    slow = ref.Gate0SeedOnlyBatchedPolicy(**{**asdict(test_policy), "expected_seed_only_ms": 0.95,
                                             "expected_speedup_vs_dense": None})
    p = ref.stream_attn_decode_plan(q4, k4, gate0_seed_only_batched_policy=slow,
                                    policy=ref.StreamAttnDecodePolicy(min_kv_len_for_gate0_seed_only=1),
                                    active_fraction_hint=1.0, block_size=16, tile_size_q=16)
    plans["not_profitable"] = {"backend": p.backend, "reason": p.reason, "fallback_reason": p.fallback_reason}
    payload["decode_plan"] = plans

    (HERE / "host_contract.json").write_text(json.dumps(payload, indent=1, sort_keys=True) + "\n")


def route_policy_goldens(ref) -> None:
    """Pure-Python routing helpers next to the decode path: the Qwen2.5-3B bucket route decisions
    (bucket_policy.py:52-211) and the shape record of the seed-kernel autotuner
    (seed_autotune.py:17-104, 333-354), as the reference computes them."""

    import itertools

    buckets = [None, "", "default", "needle", "code", "long_doc", "chat_doc", "mixed_validated",
               "chat_instruction", "json_tool", "needle_rag", "noisy_neartie", "never_seen"]
    tiers = [None, "bucket_only", "validated", "stress", "unknown"]
    decisions = []
    for bucket, strict, tier in itertools.product(buckets, [True, False], tiers):
        d = ref.qwen25_3b_bucket_route_decision(bucket, product_strict=strict, risk_tier=tier)
        decisions.append({"bucket": bucket, "product_strict": strict, "risk_tier": tier, "decision": asdict(d),
                          "policy_names": list(ref.qwen25_3b_policy_names_for_bucket(
                              bucket, product_strict=strict, risk_tier=tier))})
    shapes = []
    for batch, q_heads, kv_heads, kv_len, dim, bs, sink, recent, middle in [
            (8, 16, 2, 32768, 128, 32, 2, 2, 8), (1, 16, 2, 32768, 128, 32, 2, 3, 0), (4, 14, 2, 32768, 64, 32, 2, 6, 12),
            (2, 8, 8, 100, 64, 16, 4, 4, 4), (3, 32, 8, 65536, 128, 16, 4, 16, 4)]:
        shape = ref.SeedKernelShape(batch=batch, q_heads=q_heads, kv_heads=kv_heads, kv_len=kv_len, dim=dim,
                                    block_size=bs, sink_blocks=sink, recent_blocks=recent, middle_seed_blocks=middle)
        shapes.append(shape.to_dict())
    from_policy = []
    for name in ref.list_packaged_gate0_seed_only_batched_policies():
        policy = ref.load_packaged_gate0_seed_only_batched_policy(name)
        if policy.kv_len_bucket is None or policy.heads is None or policy.kv_heads is None or policy.dim is None:
            continue
        from_policy.append({"policy": name, "batch": None,
                            "shape": ref.seed_shape_from_policy(policy).to_dict()})
        from_policy.append({"policy": name, "batch": 3,
                            "shape": ref.seed_shape_from_policy(policy, batch=3, dtype_bytes=4).to_dict()})
    payload = {"bucket_decisions": decisions, "seed_shapes": shapes, "seed_shapes_from_policy": from_policy}
    (HERE / "route_policy.json").write_text(json.dumps(payload, indent=1, sort_keys=True) + "\n")


def seed_selection_goldens(ref) -> None:
    """Run-time seed selection as the reference computes it (seed_selectors.py:274-396): block
    scores of `_score_tensor_for_runtime_selector` and the blocks `select_seed_blocks_by_profile`
    picks, per (row, head), for the selectors that need only q and K."""

    from types import SimpleNamespace

    from stream_attention import seed_selectors as ref_sel

    out = {}
    for name, case in cases.SELECT_CASES.items():
        q, k = cases.select_inputs(case)
        policy = SimpleNamespace(block_size=case.block_size, sink_blocks=case.sink_blocks,
                                 recent_blocks=case.recent_blocks, middle_seed_blocks=case.middle_seed_blocks,
                                 block_order=case.block_order)
        entry = {}
        for selector in cases.SELECTORS:
            scores, selected = [], []
            for b in range(case.batch):
                scores.append([])
                selected.append([])
                for h in range(case.q_heads):
                    s = ref_sel._score_tensor_for_runtime_selector(q[b, 0, h], k[b, :, h], block_size=case.block_size,
                                                                   selector=selector)
                    pick = ref_sel.select_seed_blocks_by_profile(q=q[b, 0, h], k=k[b, :, h], policy=policy,
                                                                 selector=selector)
                    scores[b].append([float(x) for x in s.tolist()])
                    selected[b].append(sorted(int(x) for x in pick.selected_blocks))
            entry[selector] = {"scores": scores, "selected": selected}
        out[name] = entry
    (HERE / "seed_selection.json").write_text(json.dumps(out, indent=None, sort_keys=True) + "\n")


def rope_append_goldens(ref_root: Path) -> None:
    """RoPE + append through the reference's own safe path (`_apply_qwen_rope` + `copy_`,
    benchmarks/profile_seed_only_fused_rope_parity.py:24-30, 97-102), on CPU tensors."""

    import importlib

    parity = importlib.import_module("benchmarks.profile_seed_only_fused_rope_parity")
    out = {}
    for name, case in cases.ROPE_APPEND_CASES.items():
        q_raw, k_raw, v_raw, cos, sin, k_cache, v_cache = cases.rope_append_inputs(case)
        cos_ref = cos.expand(case.batch, -1, -1) if case.shared_cos else cos
        sin_ref = sin.expand(case.batch, -1, -1) if case.shared_cos else sin
        q_rot = parity._apply_qwen_rope(q_raw, cos_ref, sin_ref)
        k_rot = parity._apply_qwen_rope(k_raw, cos_ref, sin_ref)
        k_ref, v_ref = k_cache.clone(), v_cache.clone()
        positions = case.positions if len(case.positions) > 1 else case.positions * case.batch
        for b, pos in enumerate(positions):
            k_ref[b, :, pos : pos + 1, :].copy_(k_rot[b])
            v_ref[b, :, pos : pos + 1, :].copy_(v_raw[b])
        # Stored: the rotated query, the rows the reference wrote, and how many cache elements
        # differ from the input caches afterwards (only the written rows may).
        rows = torch.tensor(positions)
        idx = torch.arange(case.batch)
        out[f"{name}/q_rot"] = _np(q_rot.float())
        out[f"{name}/k_rows"] = _np(k_ref[idx, :, rows, :].float())
        out[f"{name}/v_rows"] = _np(v_ref[idx, :, rows, :].float())
        out[f"{name}/changed"] = np.array([int((k_ref != k_cache).sum()), int((v_ref != v_cache).sum())])
    np.savez_compressed(HERE / "rope_append_reference_outputs.npz", **out)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="path of the StreamAttn reference checkout")
    args = parser.parse_args()
    ref_root = Path(args.reference)
    sys.path.insert(0, str(ref_root))
    import stream_attention as ref

    torch.set_num_threads(max(1, torch.get_num_threads()))
    exact_goldens(ref)
    paged_goldens(ref)
    seed_goldens(ref, ref_root)
    host_contract_goldens(ref)
    route_policy_goldens(ref)
    seed_selection_goldens(ref)
    rope_append_goldens(ref_root)
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
