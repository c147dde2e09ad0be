"""Randomised shapes: the streaming kernel against the generic kernel (itself pinned to the oracle
by the parity tests) over batch sizes, head groupings, layouts, ragged lengths and schedules that
the fixed cases do not enumerate - every partition mode (pair-aligned blocked / round-robin /
claims, flat slices) is reached."""

import random

import pytest
import torch

from streamattn_b200 import native

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; refusing to skip")
    return torch.device("cuda:0")


def _case(rng: random.Random):
    dim = rng.choice([64, 128])
    kv_heads = rng.choice([1, 2, 4, 8])
    group = rng.choice([1, 2, 3, 4, 8] + ([16] if dim == 64 else []))
    if rng.random() < 0.15:
        group, kv_heads = rng.choice([24, 32, 48]), rng.choice([1, 2])   # served as 2-3 virtual KV heads of <= 16
    batch = rng.choice([1, 2, 3, 5, 8, 17, 40])
    kv_len = rng.choice([1, 7, 31, 64, 65, 300, 1000, 2049, 5000])
    layout = rng.choice(["BHND", "BNHD"])
    ragged = rng.random() < 0.6
    dynamic = rng.random() < 0.4
    num_ctas = rng.choice([0, 0, 0, 7, 33, 148])
    return batch, kv_heads, group, dim, kv_len, layout, ragged, dynamic, num_ctas


@pytest.mark.parametrize("seed", range(40))
def test_stream_kernel_matches_generic_kernel_on_random_shapes(dev, seed):
    rng = random.Random(1000 + seed)
    batch, kv_heads, group, dim, kv_len, layout, ragged, dynamic, num_ctas = _case(rng)
    q_heads = kv_heads * group
    g = torch.Generator(device=dev).manual_seed(seed)
    q = torch.randn(batch, 1, q_heads, dim, generator=g, device=dev).bfloat16()
    shape = (batch, kv_heads, kv_len, dim) if layout == "BHND" else (batch, kv_len, kv_heads, dim)
    k = torch.randn(shape, generator=g, device=dev).bfloat16()
    v = torch.randn(shape, generator=g, device=dev).bfloat16()
    lens = None
    if ragged:
        values = [rng.randint(0, kv_len) for _ in range(batch)]   # zero-length rows included
        lens = torch.tensor(values, dtype=rng.choice([torch.int32, torch.int64]), device=dev)
    outs = {}
    for kernel in ("stream", "generic"):
        out = torch.full_like(q, float("nan"))
        ws = native.new_workspace(dev, batch, q_heads, kv_heads, dim, num_ctas)
        plan = native.exact_plan(q, k, v, out, ws, kv_layout=layout, seq_lens=lens, num_ctas=num_ctas, kernel=kernel,
                                 dynamic=dynamic and kernel == "stream")
        for _ in range(2):                                        # second run: counters were left clean
            plan.run()
        assert native.workspace_status(ws) == 0
        outs[kernel] = out
    got, want = outs["stream"].float(), outs["generic"].float()
    assert torch.isfinite(got).all()
    diff = (got - want).abs()
    assert float(diff.max()) <= MAX_ABS and float(diff.mean()) <= MEAN_ABS, \
        (batch, kv_heads, group, dim, kv_len, layout, ragged, dynamic, num_ctas, float(diff.max()))


@pytest.mark.parametrize("seed", range(24))
def test_paged_stream_kernel_matches_generic_kernel_on_random_shapes(dev, seed):
    rng = random.Random(5000 + seed)
    dim = rng.choice([64, 128])
    kv_heads = rng.choice([1, 2, 4])
    group = rng.choice([1, 2, 4, 8])
    q_heads = kv_heads * group
    batch = rng.choice([1, 2, 4, 9, 20])
    page = rng.choice([8, 16, 32, 64, 128])
    max_pages = rng.choice([1, 3, 10, 40])
    layout = rng.choice(["NHD", "HND"])
    dynamic = rng.random() < 0.4
    num_pages = batch * max_pages + rng.randint(0, 5)
    g = torch.Generator(device=dev).manual_seed(seed)
    q = torch.randn(batch, 1, q_heads, dim, generator=g, device=dev).bfloat16()
    shape = (num_pages, page, kv_heads, dim) if layout == "NHD" else (num_pages, kv_heads, page, dim)
    k = torch.randn(shape, generator=g, device=dev).bfloat16()
    v = torch.randn(shape, generator=g, device=dev).bfloat16()
    order = list(range(num_pages))
    rng.shuffle(order)
    lengths = [rng.randint(1, max_pages * page) for _ in range(batch)]
    table = torch.full((batch, max_pages), -1, dtype=rng.choice([torch.int32, torch.int64]))
    for b, n in enumerate(lengths):
        active = -(-n // page)
        table[b, :active] = torch.tensor(order[b * max_pages:b * max_pages + active])
    table = table.to(dev)
    lens = torch.tensor(lengths, dtype=rng.choice([torch.int32, torch.int64]), device=dev)
    outs, traces = {}, {}
    for kernel in ("stream", "generic"):
        out = torch.full_like(q, float("nan"))
        trace = torch.full(table.shape, -1, dtype=torch.int32, device=dev)
        ws = native.new_workspace(dev, batch, q_heads, kv_heads, dim)
        plan = native.paged_plan(q, k, v, table, lens, out, ws, layout=layout, trace=trace, kernel=kernel,
                                 dynamic=dynamic and kernel == "stream")
        for _ in range(2):
            plan.run()
        assert native.workspace_status(ws) == 0
        outs[kernel], traces[kernel] = out, trace
    # The page walk is integer work: both kernels visit exactly the active table entries.
    assert torch.equal(traces["stream"].cpu(), table.to(torch.int32).cpu())
    assert torch.equal(traces["generic"].cpu(), table.to(torch.int32).cpu())
    diff = (outs["stream"].float() - outs["generic"].float()).abs()
    assert torch.isfinite(outs["stream"].float()).all()
    assert float(diff.max()) <= MAX_ABS and float(diff.mean()) <= MEAN_ABS, \
        (batch, kv_heads, group, dim, page, max_pages, layout, dynamic, float(diff.max()))


@pytest.mark.parametrize("group,kv_heads,dim,layout", [(32, 1, 128, "BHND"), (48, 1, 64, "BNHD"), (24, 2, 64, "BHND"),
                                                       (32, 2, 64, "BNHD")])
def test_large_query_groups_run_on_the_streaming_kernel(dev, group, kv_heads, dim, layout):
    """More than 16 query heads per KV head (multi-query models): the streaming kernel serves the
    group as several virtual KV heads that read the same K/V rows."""

    g = torch.Generator(device=dev).manual_seed(group)
    batch, kv_len, q_heads = 3, 1500, group * kv_heads
    q = torch.randn(batch, 1, q_heads, dim, generator=g, device=dev).bfloat16()
    shape = (batch, kv_heads, kv_len, dim) if layout == "BHND" else (batch, kv_len, kv_heads, dim)
    k = torch.randn(shape, generator=g, device=dev).bfloat16()
    v = torch.randn(shape, generator=g, device=dev).bfloat16()
    outs = {}
    for kernel in ("stream", "generic"):
        out = torch.full_like(q, float("nan"))
        ws = native.new_workspace(dev, batch, q_heads, kv_heads, dim)
        plan = native.exact_plan(q, k, v, out, ws, kv_layout=layout, kernel=kernel)
        assert plan.kernel == (native.SA_KERNEL_STREAM if kernel == "stream" else native.SA_KERNEL_GENERIC)
        plan.run()
        plan.run()
        assert native.workspace_status(ws) == 0
        outs[kernel] = out
    diff = (outs["stream"].float() - outs["generic"].float()).abs()
    assert float(diff.max()) <= MAX_ABS and float(diff.mean()) <= MEAN_ABS
