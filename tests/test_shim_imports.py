"""The ``stream_attention`` import name resolves to this package (drop-in boundary).

Every import path the reference's decode surface offers (``stream_attention/__init__.py:69-125``)
must work, name the same objects as ``streamattn_b200`` and keep the reference's behaviour for
the host-side checks its own tests make by that path (tests/test_paged_decode.py:136-175,
tests/test_engine.py argument errors, tests/test_qwen_o_proj_triton.py:11-16).
"""

from __future__ import annotations

import pytest
import torch

import stream_attention as stream_attn
import streamattn_b200

DECODE_SURFACE = """
DecodeCostEntry DecodeCostKey DecodeCostModel Gate0SeedOnlyBatchedPolicy Gate0SeedOnlyBatchedRunInfo
Gate0SeedOnlyBatchedStats STREAMATTN_EXACT_NATIVE_BACKEND STREAMATTN_MODE_EXACT_NATIVE
STREAMATTN_MODE_SEED_ONLY_NATIVE STREAMATTN_MODE_VERIFIED_AUTO STREAMATTN_NATIVE_MODES StreamAttnDecodePlan
StreamAttnDecodePolicy StreamAttnDecodeWorkspace StreamAttnDecodeWrapper StreamAttnExactNativeDirectRunner
StreamAttnSeedOnlyDirectRunner StreamAttnSeedOnlyDecodeService StreamAttnServingInfo
find_packaged_gate0_seed_only_batched_policies list_packaged_gate0_seed_only_batched_policies
load_packaged_gate0_seed_only_batched_policy packaged_gate0_seed_only_batched_policy_registry
normalize_stream_attn_mode stream_attn_decode_plan stream_attn_decode_run stream_attn_exact_native_decode
stream_attn_seed_only_decode StreamAttnEngine StreamAttnEnginePlan stream_attn_decode ExactDecodePlan
PAGED_EXACT_NATIVE_BACKEND PAGED_EXACT_SM90_FRAGMENTED_RAGGED_BACKEND PagedExactDecodePlan PagedKVCache
choose_paged_exact_splits paged_exact_reference stream_attn_paged_exact_decode decode SeedKernelAutotuneResult
SeedKernelCandidate SeedKernelShape autotune_seed_kernel_mode seed_kernel_candidates seed_shape_from_policy
BucketRouteDecision qwen25_3b_bucket_route_decision qwen25_3b_policy_names_for_bucket normalize_device_class
""".split()


def test_every_decode_surface_name_of_the_reference_is_importable():
    missing = [name for name in DECODE_SURFACE if not hasattr(stream_attn, name)]
    assert not missing, missing
    assert stream_attn.decode is streamattn_b200.stream_attn_decode


def test_submodule_paths_name_the_same_objects():
    from stream_attention.backends.sm90 import ExactDecodePlan
    from stream_attention.bucket_policy import qwen25_3b_bucket_route_decision
    from stream_attention.decode import (STREAMATTN_MODE_EXACT_NATIVE, Gate0SeedOnlyBatchedPolicy,
                                         StreamAttnDecodePolicy)
    from stream_attention.engine import StreamAttnEngine
    from stream_attention.kernels.gate0_exact_refresh_triton import (
        TRITON_AVAILABLE, exact_decode_attention_rows_triton_forward_out_bhnd)
    from stream_attention.kernels.gate0_seed_only_triton import (
        gate0_seed_only_attention_triton_forward_out, gate0_seed_only_attention_triton_forward_out_prechecked)
    from stream_attention.kernels.paged_exact_triton import (make_paged_exact_workspace,
                                                             paged_exact_decode_triton_forward_out)
    from stream_attention.paged import PagedKVCache, choose_paged_exact_splits, paged_exact_reference
    from stream_attention.seed_autotune import SeedKernelShape
    from stream_attention.seed_selectors import policy_seed_blocks, seed_indices, seed_token_indices_from_blocks
    from stream_attention.telemetry import seq_bucket

    assert ExactDecodePlan is streamattn_b200.ExactDecodePlan
    assert StreamAttnEngine is streamattn_b200.StreamAttnEngine
    assert Gate0SeedOnlyBatchedPolicy is streamattn_b200.Gate0SeedOnlyBatchedPolicy
    assert PagedKVCache is streamattn_b200.PagedKVCache
    assert STREAMATTN_MODE_EXACT_NATIVE == "exact_native" and TRITON_AVAILABLE is False
    assert seq_bucket(4097) == 8192 and choose_paged_exact_splits is streamattn_b200.choose_paged_exact_splits
    assert policy_seed_blocks(seq_len=320, block_size=32, sink_blocks=1, recent_blocks=1, middle_seed_blocks=2,
                              block_order="recent_first") == [0, 9, 8, 7]
    assert callable(exact_decode_attention_rows_triton_forward_out_bhnd) and callable(paged_exact_reference)
    assert callable(make_paged_exact_workspace) and callable(paged_exact_decode_triton_forward_out)
    assert gate0_seed_only_attention_triton_forward_out_prechecked is gate0_seed_only_attention_triton_forward_out
    assert StreamAttnDecodePolicy().safety_margin == 1.10
    assert qwen25_3b_bucket_route_decision("code").mode == "seed_only_bundle"
    assert SeedKernelShape is streamattn_b200.SeedKernelShape and callable(seed_indices)
    assert callable(seed_token_indices_from_blocks)


def _paged_inputs():
    g = torch.Generator().manual_seed(17)
    query = torch.randn(2, 1, 4, 8, generator=g)
    key = torch.randn(5, 4, 2, 8, generator=g)
    value = torch.randn(5, 4, 2, 8, generator=g)
    table = torch.tensor([[3, 0, -1], [1, 4, 2]], dtype=torch.int32)
    lengths = torch.tensor([7, 10], dtype=torch.int32)
    return query, stream_attn.PagedKVCache(key, value, table, lengths, "NHD")


def test_paged_host_checks_by_the_reference_import_path():
    from stream_attention.paged import PagedKVCache, choose_paged_exact_splits

    query, cache = _paged_inputs()
    with pytest.raises(ValueError, match="does not yet support paged KV"):
        stream_attn.decode(query, cache, mode="seed_only_native")
    with pytest.raises(ValueError, match="value_cache must be omitted"):
        stream_attn.decode(query, cache, torch.empty_like(query), mode="exact_native")
    bad_table = cache.page_table.clone()
    bad_table[0, 1] = cache.num_pages
    with pytest.raises(ValueError, match="active page_table"):
        PagedKVCache(cache.key, cache.value, bad_table, cache.sequence_lengths, cache.layout).validate(query)
    bad_lengths = cache.sequence_lengths.clone()
    bad_lengths[1] = cache.max_sequence_length + 1
    with pytest.raises(ValueError, match="exceed page_table capacity"):
        PagedKVCache(cache.key, cache.value, cache.page_table, bad_lengths, cache.layout).validate(query)
    assert choose_paged_exact_splits(batch=1, query_heads=16, max_pages_per_request=2048) == 32
    assert choose_paged_exact_splits(batch=4, query_heads=16, max_pages_per_request=2048) == 8
    assert choose_paged_exact_splits(batch=8, query_heads=16, max_pages_per_request=2048) == 4
    with pytest.raises(ValueError, match="mode must be one of"):
        stream_attn.decode(query, cache, mode="fastest")


def test_paged_reference_utility_reproduces_the_reference_fixture(golden_paged):
    """``paged_exact_reference`` is a checking utility (never on the decode path): on the
    reference's own fixture it returns what the reference returned."""

    query, key, value = (torch.from_numpy(golden_paged[f"fixture17_NHD/{name}"]) for name in ("q", "k", "v"))
    _, layout_cache = _paged_inputs()
    cache = stream_attn.PagedKVCache(key, value, layout_cache.page_table, layout_cache.sequence_lengths, "NHD")
    got = stream_attn.paged_exact_reference(query, cache)
    want = torch.from_numpy(golden_paged["fixture17_NHD/out"])
    torch.testing.assert_close(got, want, atol=1e-6, rtol=1e-5)


def test_o_proj_launcher_refuses_cpu_tensors_like_the_reference():
    from stream_attention.kernels.qwen_o_proj_triton import qwen_o_proj_triton_forward

    x = torch.randn(2, 1, 8, dtype=torch.float16)
    weight = torch.randn(8, 8, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="Triton|CUDA"):
        qwen_o_proj_triton_forward(x, weight)
