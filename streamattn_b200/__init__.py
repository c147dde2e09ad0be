"""B200-native decode attention, a drop-in for the ``stream_attention`` decode path.

``import streamattn_b200 as stream_attn`` and call ``stream_attn.decode(...)``,
``StreamAttnEngine.plan(...).run()``, ``PagedKVCache`` / ``PagedExactDecodePlan``
exactly as with the reference package.  Everything executes in hand-written
sm_100a CUDA kernels behind a C ABI (``include/streamattn_b200.h``); there is
no Triton, no multi-backend dispatch and no CPU execution path.
"""

__version__ = "0.1.0"

from .decode import (
    DecodeCostEntry,
    DecodeCostKey,
    DecodeCostModel,
    Gate0SeedOnlyBatchedPolicy,
    Gate0SeedOnlyBatchedRunInfo,
    Gate0SeedOnlyBatchedStats,
    STREAMATTN_EXACT_NATIVE_BACKEND,
    STREAMATTN_MODE_EXACT_NATIVE,
    STREAMATTN_MODE_SEED_ONLY_NATIVE,
    STREAMATTN_MODE_VERIFIED_AUTO,
    STREAMATTN_NATIVE_MODES,
    StreamAttnDecodePlan,
    StreamAttnDecodePolicy,
    StreamAttnDecodeWorkspace,
    StreamAttnDecodeWrapper,
    StreamAttnExactNativeDirectRunner,
    StreamAttnSeedOnlyDecodeService,
    StreamAttnSeedOnlyDirectRunner,
    StreamAttnServingInfo,
    find_packaged_gate0_seed_only_batched_policies,
    infer_kv_layout,
    list_packaged_gate0_seed_only_batched_policies,
    load_packaged_gate0_seed_only_batched_policy,
    normalize_device_class,
    normalize_stream_attn_mode,
    packaged_gate0_seed_only_batched_policy_registry,
    seq_bucket,
    stream_attn_decode_plan,
    stream_attn_decode_run,
    stream_attn_exact_native_decode,
    stream_attn_seed_only_decode,
)
from .engine import StreamAttnEngine, StreamAttnEnginePlan, stream_attn_decode
from .exact import ExactDecodePlan, choose_num_splits
from .paged import (
    PAGED_EXACT_NATIVE_BACKEND,
    PAGED_EXACT_SM100_BACKEND,
    PAGED_EXACT_SM90_FRAGMENTED_RAGGED_BACKEND,
    PagedExactDecodePlan,
    PagedKVCache,
    choose_paged_exact_splits,
    paged_exact_reference,
    stream_attn_paged_exact_decode,
)
from .seed_autotune import (
    SeedKernelAutotuneResult,
    SeedKernelCandidate,
    SeedKernelShape,
    autotune_seed_kernel_mode,
    seed_kernel_candidates,
    seed_shape_from_policy,
)
from .bucket_policy import (
    BucketRouteDecision,
    qwen25_3b_bucket_route_decision,
    qwen25_3b_policy_names_for_bucket,
)
from .o_proj import OProjPlan, qwen_o_proj_forward
from .kv_update import AppendKVPlan, PagedKVWriter, PagePool, append_kv, paged_append_kv
from .seed_selectors import (
    DynamicSeedDecodePlan,
    SeedBlockSelection,
    parse_selector_profiles,
    policy_seed_blocks,
    seed_indices,
    seed_token_indices_from_blocks,
    select_seed_blocks_by_profile,
)

# ``import streamattn_b200 as stream_attn; stream_attn.decode(...)``
decode = stream_attn_decode

__all__ = [name for name in dir() if not name.startswith("_")]
