"""Output projection of a decode step on the sm_100a weight-streaming kernel.

Counterpart of the reference's ``qwen_o_proj_triton_forward``
(``stream_attention/kernels/qwen_o_proj_triton.py:77-145``): ``F.linear`` for
``[batch, 1, hidden]`` decode tensors with a ``[out_features, in_features]`` weight.
The kernel (``csrc/sa_oproj.cu``) is launched with programmatic stream serialization and
requests its weights before it waits for the preceding kernel, so in a decode step the 8 MB
weight stream of a 2048 x 2048 projection overlaps the tail of the attention launch.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import native


def _check(attn_output: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> tuple:
    if not attn_output.is_cuda or not weight.is_cuda or (bias is not None and not bias.is_cuda):
        raise RuntimeError("qwen_o_proj_forward requires CUDA tensors (streamattn_b200 has no CPU fallback)")
    if attn_output.dim() != 3 or attn_output.shape[1] != 1:
        raise ValueError("attn_output must be [batch, 1, hidden]")
    if weight.dim() != 2:
        raise ValueError("weight must be [out_features, in_features]")
    batch, in_features, out_features = int(attn_output.shape[0]), int(attn_output.shape[2]), int(weight.shape[0])
    if int(weight.shape[1]) != in_features:
        raise ValueError("weight in_features must match attn_output hidden size")
    if bias is not None and (bias.dim() != 1 or int(bias.numel()) != out_features):
        raise ValueError("bias must be [out_features]")
    if attn_output.device != weight.device or (bias is not None and bias.device != weight.device):
        raise ValueError("attn_output, weight, and bias must be on the same CUDA device")
    if attn_output.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("attn_output must be fp16 or bf16")
    if weight.dtype != attn_output.dtype:
        raise ValueError("weight dtype must match attn_output dtype")
    if bias is not None and bias.dtype != attn_output.dtype:
        raise ValueError("bias dtype must match attn_output dtype")
    return batch, in_features, out_features


@dataclass
class OProjPlan:
    """Projection bound to stable buffers: ``run()`` is one launch and allocates nothing.

    ``attn_output`` is typically the output buffer of a decode plan viewed as
    ``[batch, 1, heads * dim]``.  ``prefetch_weights=False`` makes the kernel wait for earlier
    work on the stream before it touches the weights (needed only if the weights themselves
    were just written on that stream).
    """

    attn_output: torch.Tensor
    weight: torch.Tensor
    bias: Optional[torch.Tensor]
    output: torch.Tensor
    prefetch_weights: bool = True

    @classmethod
    def build(cls, attn_output: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *,
              output: Optional[torch.Tensor] = None, prefetch_weights: bool = True) -> "OProjPlan":
        batch, in_features, out_features = _check(attn_output, weight, bias)
        if attn_output.stride(2) != 1:
            raise ValueError("attn_output's hidden dimension must be contiguous")
        if not weight.is_contiguous() or (bias is not None and not bias.is_contiguous()):
            raise ValueError("weight and bias must be contiguous")
        if output is None:
            output = torch.empty((batch, 1, out_features), dtype=attn_output.dtype, device=attn_output.device)
        if tuple(output.shape) != (batch, 1, out_features) or output.dtype != attn_output.dtype \
                or not output.is_contiguous() or output.device != attn_output.device:
            raise ValueError("output must be a contiguous [batch, 1, out_features] tensor of the input dtype")
        plan = cls(attn_output, weight, bias, output, bool(prefetch_weights))
        plan._args = (attn_output.data_ptr(), weight.data_ptr(), None if bias is None else bias.data_ptr(),
                      output.data_ptr(), batch, in_features, out_features, int(attn_output.stride(0)),
                      native.SA_DTYPE[attn_output.dtype], int(bool(prefetch_weights)))
        plan._fn = native.load().sa_o_proj
        plan._device_index = attn_output.device.index if attn_output.device.index is not None \
            else torch.cuda.current_device()
        with torch.cuda.device(attn_output.device):
            plan.run()  # validates the arguments in the library once (raises on unsupported shapes)
        return plan

    def run(self) -> torch.Tensor:
        rc = self._fn(*self._args, native._current_raw_stream(self._device_index))
        if rc:
            native.check(rc)
        return self.output


def qwen_o_proj_forward(attn_output: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                        *, out: Optional[torch.Tensor] = None, **_launch_hints) -> torch.Tensor:
    """``F.linear(attn_output, weight, bias)`` for ``[batch, 1, hidden]`` decode tensors.

    Same call as the reference's ``qwen_o_proj_triton_forward``; its Triton block-size and
    warp-count hints are accepted and ignored.  ``out`` reuses a result buffer.
    """

    _check(attn_output, weight, bias)
    x = attn_output if attn_output.stride(2) == 1 else attn_output.contiguous()
    with torch.cuda.device(x.device):
        return OProjPlan.build(x, weight.contiguous(), None if bias is None else bias.contiguous(), output=out).output


__all__ = ["OProjPlan", "qwen_o_proj_forward"]
