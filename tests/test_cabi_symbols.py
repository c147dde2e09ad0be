"""The C-ABI library builds, loads and exports every symbol the header declares.

No compute call is made here (this runs without a GPU); only host-side
queries that never touch a device.
"""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

from streamattn_b200 import build, native

HEADER = Path(__file__).resolve().parents[1] / "include" / "streamattn_b200.h"


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"SA_API\s+[\w\s\*]+?\b(sa_\w+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 20
    lib = ctypes.CDLL(str(build.build()))
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert sorted(native.exported_symbols()) == names


def test_host_only_queries():
    lib = native.load()
    assert lib.sa_version() >= 100
    # Sizing depends only on the arguments (no device query).
    small = native.workspace_bytes(8, 16, 2, 64)
    assert small > 0 and small % 4 == 0
    assert native.workspace_bytes(8, 16, 2, 128) > small
    assert lib.sa_workspace_bytes(8, 16, 3, 64, 0) == 0
    assert "bad shape" in native.last_error()


def test_no_cpu_tensors_reach_the_library():
    import pytest
    import torch

    q = torch.zeros(1, 1, 4, 8)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        native.require_cuda(q)
