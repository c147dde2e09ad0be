"""``sa_exact_decode_static``: exact decode for callers that cannot allocate.

A serving engine that hands every free byte of HBM to its KV-cache pool, or a
plugin that only ever receives the tensors of one call, has nowhere to get the
split-state workspace ``sa_exact_decode`` asks for.  The static variant keeps
that scratch in a fixed 2 MiB array inside the library, so the caller passes
inputs and outputs only.  Here it is called through the C ABI twice in a row
(the array keeps the previous call's contents, so the second call proves the
counters are re-armed) and compared with the workspace-taking entry point;
``sa_static_status`` must report a clean status word afterwards.
"""

from __future__ import annotations

import pytest
import torch

import cases
from oracle import cpu_oracle
from streamattn_b200 import native

pytestmark = pytest.mark.gpu


def _raw_static_call(lib, q, k, v, out, case, stream, num_ctas=0):
    return lib.sa_exact_decode_static(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), None, 0,
        case.batch, case.q_heads, case.kv_heads, case.dim, case.kv_len,
        q.stride(0), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
        native.SA_DTYPE[q.dtype], native.SA_OUT_FINAL, num_ctas, native.SA_KERNEL_AUTO, stream)


@pytest.mark.parametrize("name", ["g7_d64_n1000", "g4_d128_n257", "g2_d8_n32"])
def test_static_scratch_entry_point_matches_workspace_entry_point(name):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; refusing to skip")
    dev = torch.device("cuda:0")
    lib = native.load()
    case = cases.EXACT_CASES[name]
    q, k, v = (t.to(torch.bfloat16) for t in cases.exact_inputs(case))
    want = cpu_oracle.exact_decode(q, k, v)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    stream = native.stream_handle(dev)

    # Existing entry point, caller-provided workspace.
    expected = torch.empty_like(qd)
    ws = native.new_workspace(dev, case.batch, case.q_heads, case.kv_heads, case.dim)
    native.exact_plan(qd, kd, vd, expected, ws, kv_layout="BNHD").run()
    torch.cuda.synchronize()

    # New entry point: nothing but inputs and outputs, two calls back to back.
    for attempt in range(2):
        got = torch.full_like(qd, float("nan"))
        rc = _raw_static_call(lib, qd, kd, vd, got, case, stream)
        assert rc == 0, native.last_error()
        torch.cuda.synchronize()
        diff = (got.float() - expected.float()).abs()
        assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3, (attempt, float(diff.max()))
        assert torch.equal(got, expected), "same kernels, same schedule: results are bit-identical"
        ref = (got.float().cpu() - want).abs()
        assert float(ref.max()) <= 2e-2 and float(ref.mean()) <= 2e-3

    assert native.static_status(dev) == 0, "no wait gave up, no bad page: the status word stays clean"

    # A different split count re-uses the same array with another slot layout.
    got = torch.empty_like(qd)
    rc = _raw_static_call(lib, qd, kd, vd, got, case, stream, num_ctas=7)
    assert rc == 0, native.last_error()
    torch.cuda.synchronize()
    diff = (got.float() - expected.float()).abs()
    assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3


def test_static_scratch_rejects_shapes_beyond_its_size():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; refusing to skip")
    dev = torch.device("cuda:0")
    batch, q_heads, kv_heads, dim, kv_len = 64, 32, 2, 128, 64
    q = torch.zeros(batch, 1, q_heads, dim, dtype=torch.bfloat16, device=dev)
    k = torch.zeros(batch, kv_len, kv_heads, dim, dtype=torch.bfloat16, device=dev)
    out = torch.empty_like(q)
    # 4096 CTAs x 16 heads x 130 floats of split state is far beyond 2 MiB.
    with pytest.raises(ValueError, match="built-in scratch"):
        native.exact_decode_static(q, k, k, out, num_ctas=4096)
    # The same shape with the automatic grid fits and runs (zeros in, zeros out).
    native.exact_decode_static(q, k, k, out)
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0
