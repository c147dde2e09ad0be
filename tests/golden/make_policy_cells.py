"""Condense a StreamAttn checkout's seed-only policy artifacts into ``seed_only_cells.json``.

    python tests/golden/make_policy_cells.py /path/to/StreamAttn/stream_attention/policies

Each registry entry of the checkout becomes one cell: the registry metadata used
for discovery plus the policy fields this package's loader
(``Gate0SeedOnlyBatchedPolicy.from_entry``) extracts from the artifact.  Evidence
blocks of the artifacts (rollout logs, per-prompt statistics) are not carried
over.  The expected_*_ms timings inside a cell are the H100 measurements the
artifacts record; they only feed the planned-route profitability test.
"""

from __future__ import annotations

import json
import sys
from dataclasses import asdict
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]  # repository root
sys.path.insert(0, str(ROOT))

from streamattn_b200.decode import Gate0SeedOnlyBatchedPolicy  # noqa: E402

REGISTRY_KEYS = ("name", "policy_id", "aliases", "status", "model_id", "layer_id", "mode", "tensor_space",
                 "dtype", "kv_len_bucket", "min_batch", "q_heads", "kv_heads", "head_dim", "attention_type")


def main(argv) -> None:
    source = Path(argv[1])
    registry = json.loads((source / "registry.json").read_text(encoding="utf-8"))
    cells = []
    for entry in registry.get("policies") or []:
        artifact = source.parent / entry["path"]
        policy = Gate0SeedOnlyBatchedPolicy.from_json(artifact)
        cells.append({
            "registry": {key: entry[key] for key in REGISTRY_KEYS if key in entry},
            "policy": asdict(policy),
        })
    payload = {
        "schema": "streamattn_b200.seed_only_cells.v1",
        "default": registry.get("default"),
        "cells": cells,
    }
    out = ROOT / "streamattn_b200" / "policies" / "seed_only_cells.json"
    out.write_text(json.dumps(payload, indent=1, sort_keys=True) + "\n", encoding="utf-8")
    print(f"wrote {len(cells)} cells to {out}")


if __name__ == "__main__":
    main(sys.argv)
