"""Output projection after attention (``sa_o_proj``) and the reference-named launchers, on the GPU.

Parity: float32 ``F.linear`` of the same input values on the CPU (``oracle/torch_port.o_proj``),
the checker the reference's own test uses for its Triton kernel, at the reference's tolerance
(1e-2) and at the tighter one the float32 accumulation should meet (one rounding of the output).
"""

from __future__ import annotations

import pytest
import torch

import cases
import streamattn_b200 as sa
from oracle import cpu_oracle, torch_port
from streamattn_b200 import launchers, native

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; refusing to skip")
    return torch.device("cuda:0")


def _close(got, want, atol=2e-2, mean=2e-3):
    diff = (got.float().cpu() - want.float()).abs()
    assert float(diff.max()) <= atol and float(diff.mean()) <= mean, (float(diff.max()), float(diff.mean()))


def _one_rounding(got, want, dtype=torch.bfloat16, slack=1e-3):
    """|got - want| within one rounding of the output dtype (projection outputs are not O(1))."""

    ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    diff = (got.float().cpu() - want.float()).abs()
    assert bool((diff <= want.float().abs() * ulp + slack).all()), float(diff.max())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("batch,in_features,out_features,has_bias", [
    (5, 64, 96, False), (5, 64, 96, True),          # the reference test's shape
    (8, 2048, 2048, False), (1, 2048, 2048, True),  # Qwen2.5-3B: 16 heads x 128 -> hidden 2048
    (16, 2048, 2048, True), (19, 896, 1000, True),  # a second batch tile; K and N that are not multiples of 32 / 8 rows
    (3, 4104, 24, False),                           # more than one round of chunks per warp
])
def test_o_proj_matches_float32_linear(dev, dtype, batch, in_features, out_features, has_bias):
    g = torch.Generator().manual_seed(123)
    x = torch.randn(batch, 1, in_features, generator=g).to(dtype)
    weight = (torch.randn(out_features, in_features, generator=g) / 8.0).to(dtype)
    bias = (torch.randn(out_features, generator=g) / 8.0).to(dtype) if has_bias else None
    want = torch_port.o_proj(x, weight, bias)
    got = sa.qwen_o_proj_forward(x.to(dev), weight.to(dev), None if bias is None else bias.to(dev))
    assert got.shape == (batch, 1, out_features) and got.dtype == dtype
    torch.testing.assert_close(got.float().cpu(), want, rtol=1e-2, atol=1e-2)          # the reference's bar
    _one_rounding(got, want, dtype)


def test_o_proj_plan_reads_a_strided_attention_buffer_and_allocates_nothing(dev):
    g = torch.Generator().manual_seed(7)
    batch, heads, dim, hidden = 8, 16, 128, 2048
    attn = torch.randn(batch, 1, heads, dim, generator=g).bfloat16().to(dev)       # a decode plan's output buffer
    weight = (torch.randn(hidden, heads * dim, generator=g) / 16.0).bfloat16().to(dev)
    out = torch.empty(batch, 1, hidden, dtype=torch.bfloat16, device=dev)
    plan = sa.OProjPlan.build(attn.view(batch, 1, heads * dim), weight, output=out)
    want = torch_port.o_proj(attn.view(batch, 1, -1), weight)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(dev)
    for _ in range(3):
        assert plan.run() is out
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(dev) == before
    _one_rounding(out, want)
    # in-place update of the bound input is seen by the next run
    attn.mul_(-1)
    plan.run()
    _one_rounding(out, -want)
    # without the early weight fetch the result is the same bits
    late = sa.OProjPlan.build(attn.view(batch, 1, heads * dim), weight, prefetch_weights=False)
    assert torch.equal(late.run(), out)


def test_o_proj_argument_errors(dev):
    x = torch.randn(2, 2, 8, dtype=torch.float16, device=dev)
    weight = torch.randn(8, 8, dtype=torch.float16, device=dev)
    with pytest.raises(ValueError, match=r"\[batch, 1, hidden\]"):
        sa.qwen_o_proj_forward(x, weight)
    with pytest.raises(ValueError, match="in_features must match"):
        sa.qwen_o_proj_forward(x[:, :1], weight[:, :4].contiguous())
    with pytest.raises(ValueError, match="fp16 or bf16"):
        sa.qwen_o_proj_forward(x[:, :1].float(), weight.float())
    with pytest.raises(ValueError, match="multiples of 8"):
        sa.qwen_o_proj_forward(torch.zeros(2, 1, 12, dtype=torch.float16, device=dev),
                               torch.zeros(8, 12, dtype=torch.float16, device=dev))


def test_decode_then_projection_chain_matches_the_oracle(dev):
    """attention -> output projection as two back-to-back launches on one stream (the projection
    starts fetching its weights before the attention kernel has finished)."""

    case = cases.EXACT_CASES["g4_d128_n257"]
    q, k, v = (t.bfloat16() for t in cases.exact_inputs(case))
    g = torch.Generator().manual_seed(3)
    hidden = case.q_heads * case.dim
    weight = (torch.randn(hidden, hidden, generator=g) / 16.0).bfloat16()
    attn_want = cpu_oracle.exact_decode(q, k, v).bfloat16()
    want = torch_port.o_proj(attn_want.view(case.batch, 1, hidden), weight)
    plan = sa.ExactDecodePlan.build(q.to(dev), k.to(dev), v.to(dev), kv_layout="BNHD")
    proj = sa.OProjPlan.build(plan.output.view(case.batch, 1, hidden), weight.to(dev))
    for _ in range(3):
        plan.run()
        out = proj.run()
    # the attention output itself is within 2e-2 of the oracle's; through a 1/16-scaled weight of
    # `hidden` columns that is at most a few hundredths on outputs of magnitude ~1
    _close(out, want, atol=6e-2, mean=1e-2)


def test_reference_named_launchers(dev):
    # paged
    pc = cases.PAGED_CASES["p16_g8_d64"]
    q, kp, vp, table, lengths = cases.paged_inputs(pc, layout="NHD")
    q, kp, vp = (t.bfloat16() for t in (q, kp, vp))
    want = cpu_oracle.paged_decode(q, kp, vp, table, lengths, layout="NHD")
    want = want[0] if isinstance(want, tuple) else want
    out = torch.empty_like(q, device=dev)
    ws = launchers.make_paged_exact_workspace(batch=int(q.shape[0]), heads=int(q.shape[2]), splits=4,
                                              dim=int(q.shape[3]), device=dev)
    got = launchers.paged_exact_decode_triton_forward_out(q.to(dev), kp.to(dev), vp.to(dev), table.to(dev),
                                                          lengths.to(dev), out, layout="NHD", splits=4, workspace=ws,
                                                          tokens_per_tile=512, partial_num_warps=4)
    assert got is out
    _close(out, want)
    # seed-only, both cache layouts
    sc = cases.SEED_CASES["s_bs32_d128"]
    sq, sk, sv = (t.bfloat16() for t in cases.seed_inputs(sc))
    tokens = cpu_oracle.seed_indices(seq_len=sc.kv_len, block_size=sc.block_size, sink_blocks=sc.sink_blocks,
                                     recent_blocks=sc.recent_blocks, middle_seed_blocks=sc.middle_seed_blocks,
                                     block_order=sc.block_order)
    swant = cpu_oracle.seed_decode(sq, sk, sv, tokens)
    kwargs = dict(block_size=sc.block_size, sink_blocks=sc.sink_blocks, recent_blocks=sc.recent_blocks,
                  middle_seed_blocks=sc.middle_seed_blocks, block_order=sc.block_order, num_warps=4, num_stages=2)
    sout = torch.empty_like(sq, device=dev)
    launchers.gate0_seed_only_attention_triton_forward_out(sq.to(dev), sk.to(dev), sv.to(dev), sout, **kwargs)
    _close(sout, swant)
    sout2 = torch.empty_like(sq, device=dev)
    launchers.gate0_seed_only_attention_triton_forward_out_dynamic_n_bhnd(
        sq.to(dev), sk.transpose(1, 2).contiguous().to(dev), sv.transpose(1, 2).contiguous().to(dev), sout2, **kwargs)
    assert torch.equal(sout2, sout)
    with pytest.raises(RuntimeError, match="CUDA"):
        launchers.gate0_seed_only_attention_triton_forward_out(sq, sk, sv, torch.empty_like(sq), **kwargs)
