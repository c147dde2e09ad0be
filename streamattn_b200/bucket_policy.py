"""Which layers of Qwen2.5-3B may run seed-only decode for a given prompt bucket.

Behaviour-compatible with the reference's ``stream_attention/bucket_policy.py:52-211``
(``qwen25_3b_bucket_route_decision`` and ``qwen25_3b_policy_names_for_bucket``): the
same decision record for the same (bucket, risk tier, strictness), pinned by
reference-generated golden records in ``tests/golden/host_contract.json``.

The decision is a short ordered rule table.  Each rule names the condition under
which it fires and the route it yields; the first rule that fires wins.  A route is
one of three layer sets - every layer exact, the full seed-only bundle, or the
reduced bundle that keeps the late layers exact (research screens only).  Serving
("product strict") never leaves exact decode unless the bucket passed the
validated-bucket gate; everything unknown fails closed to exact.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, NamedTuple, Optional, Tuple

MODEL_ID = "Qwen/Qwen2.5-3B-Instruct"

# Layers whose packaged seed-only policy passed the per-layer gate, and the policy cell of each.
QWEN25_3B_POLICY_BY_LAYER: Dict[int, str] = {
    layer: f"qwen25_3b_l{layer}_{'s416_' if layer == 2 else ''}32k_seed_only_batched"
    for layer in (0, 2, 14, 16, 24, 26, 27, 35)
}
QWEN25_3B_FULL_SEED_LAYERS: Tuple[int, ...] = tuple(QWEN25_3B_POLICY_BY_LAYER)
# The reduced bundle drops layer 2 and keeps the late layers 26/27 exact.
QWEN25_3B_REDUCED_STRESS_SEED_LAYERS: Tuple[int, ...] = (0, 14, 16, 24, 35)

QWEN25_3B_STRESS_RISK_BUCKETS = frozenset({"chat_instruction", "json_tool", "needle_rag", "noisy_neartie"})
QWEN25_3B_MARGIN_EXACT_BUCKETS = frozenset({"noisy_neartie"})
QWEN25_3B_VALIDATED_DEFAULT_BUCKETS = frozenset({"needle", "code", "long_doc", "chat_doc", "default",
                                                 "mixed_validated"})
QWEN25_3B_RISK_TIERS = frozenset({"bucket_only", "validated", "stress", "unknown"})


@dataclass(frozen=True)
class BucketRouteDecision:
    model_id: str
    prompt_bucket: str
    mode: str
    seed_only_layers: Tuple[int, ...]
    exact_layers: str
    policy_names: Tuple[str, ...]
    strict_gate_passed: bool
    status: str
    reason: str
    evidence: str
    risk_tier: str = "bucket_only"


class _Route(NamedTuple):
    mode: str
    layers: Tuple[int, ...]
    exact_layers: str


_ALL_EXACT = _Route("exact_native", (), "all")
_FULL_BUNDLE = _Route("seed_only_bundle", QWEN25_3B_FULL_SEED_LAYERS, "all non-listed layers")
_REDUCED_BUNDLE = _Route("reduced_seed_only_bundle", QWEN25_3B_REDUCED_STRESS_SEED_LAYERS,
                         "all non-listed layers plus L26/L27")


class _Rule(NamedTuple):
    fires: Callable[[str, str, bool], bool]  # (bucket, risk tier, product_strict)
    route: _Route
    status: str
    reason: str
    evidence: str
    gate_passed: Optional[bool]  # None: the bucket's own validation status


def _validated(bucket: str) -> bool:
    return bucket in QWEN25_3B_VALIDATED_DEFAULT_BUCKETS


_EXACT_STATUS = "product_exact_fallback"
_RULES: Tuple[_Rule, ...] = (
    _Rule(lambda bucket, tier, strict: tier in ("stress", "unknown"),
          _ALL_EXACT, _EXACT_STATUS, "risk_tier_requires_exact",
          "32-step hybrid stress matrix: no tested L27/L26/L24 hybrid route passed the strict gate; "
          "coarse bucket names are insufficient", True),
    _Rule(lambda bucket, tier, strict: tier == "validated" and not _validated(bucket),
          _ALL_EXACT, _EXACT_STATUS, "bucket_not_validated_for_validated_tier",
          "validated risk tier can only use explicitly validated buckets", True),
    _Rule(lambda bucket, tier, strict: bucket in QWEN25_3B_MARGIN_EXACT_BUCKETS,
          _ALL_EXACT, _EXACT_STATUS, "margin_sensitive_stress_bucket",
          "minimal repair sweep: noisy_neartie still changed top1 under minus_l26_l27", True),
    _Rule(lambda bucket, tier, strict: bucket in QWEN25_3B_STRESS_RISK_BUCKETS and strict,
          _ALL_EXACT, _EXACT_STATUS, "stress_bucket_failed_strict_gate",
          "32-step hybrid stress matrix: no tested hybrid route passed strict gate", True),
    _Rule(lambda bucket, tier, strict: bucket in QWEN25_3B_STRESS_RISK_BUCKETS,
          _REDUCED_BUNDLE, "research_only", "late_layers_exact_for_repair_screen",
          "research-only reduced route; 32-step hybrid stress matrix confirmed that even L24/L26/L27 exact "
          "did not pass", False),
    _Rule(lambda bucket, tier, strict: strict and not _validated(bucket),
          _ALL_EXACT, _EXACT_STATUS, "bucket_not_validated_by_stress_or_default_gate",
          "unknown buckets fail closed until separately validated", True),
)
_BUNDLE_EVIDENCE = ("Qwen3B L2-S416 8-layer route passed the validated-bucket 32-step gate; 128-step long-horizon "
                    "screen stayed top1/sample stable but exceeded max-KL/top-k strictness")


def qwen25_3b_bucket_route_decision(prompt_bucket: Optional[str], *, product_strict: bool = True,
                                    risk_tier: Optional[str] = None) -> BucketRouteDecision:
    """Route of a Qwen2.5-3B request: which layers decode seed-only, which stay exact, and why.

    ``product_strict=True`` is the serving selector: anything but a validated bucket decodes
    exact.  ``product_strict=False`` additionally hands out the research routes (reduced bundle
    for the stress buckets, full bundle for unknown buckets) with ``strict_gate_passed=False``.
    """

    bucket = str(prompt_bucket or "default")
    tier = str(risk_tier or "bucket_only")
    if tier not in QWEN25_3B_RISK_TIERS:
        raise ValueError(f"unsupported Qwen2.5-3B route risk tier {tier!r}")
    strict = bool(product_strict)
    for rule in _RULES:
        if rule.fires(bucket, tier, strict):
            route, status, reason, evidence, passed = rule.route, rule.status, rule.reason, rule.evidence, rule.gate_passed
            break
    else:  # no rule objects: the full bundle, a product candidate only for validated buckets
        route, evidence, passed = _FULL_BUNDLE, _BUNDLE_EVIDENCE, _validated(bucket)
        status = "product_candidate" if passed else "unknown_bucket_exact_recommended"
        reason = "validated_default_bucket" if passed else "bucket_not_validated_by_stress_or_default_gate"
    return BucketRouteDecision(
        model_id=MODEL_ID, prompt_bucket=bucket, mode=route.mode, seed_only_layers=route.layers,
        exact_layers=route.exact_layers,
        policy_names=tuple(QWEN25_3B_POLICY_BY_LAYER[layer] for layer in route.layers),
        strict_gate_passed=bool(passed), status=status, reason=reason, evidence=evidence, risk_tier=tier)


def qwen25_3b_policy_names_for_bucket(prompt_bucket: Optional[str], *, product_strict: bool = True,
                                      risk_tier: Optional[str] = None) -> Tuple[str, ...]:
    """Names of the packaged policy cells the bucket's route uses (empty: every layer exact)."""

    return qwen25_3b_bucket_route_decision(prompt_bucket, product_strict=product_strict,
                                           risk_tier=risk_tier).policy_names


__all__ = ["BucketRouteDecision", "QWEN25_3B_FULL_SEED_LAYERS", "QWEN25_3B_MARGIN_EXACT_BUCKETS",
           "QWEN25_3B_POLICY_BY_LAYER", "QWEN25_3B_REDUCED_STRESS_SEED_LAYERS", "QWEN25_3B_RISK_TIERS",
           "QWEN25_3B_STRESS_RISK_BUCKETS", "QWEN25_3B_VALIDATED_DEFAULT_BUCKETS",
           "qwen25_3b_bucket_route_decision", "qwen25_3b_policy_names_for_bucket"]
