"""RMSNorm oracle (test infrastructure; parity unpinned, see oracle/__init__.py)."""
from __future__ import annotations

import torch


def rms_norm_reference(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """out = bf16( x * rsqrt(mean(x^2) + eps) * w ), all arithmetic in fp32, one rounding.

    Follows custom_rms_norm_kernel (custom_kernels/custom_kernels.cu:343-344 formula, :351-360 fp32 sum
    of squares over the last axis, :362 rsqrt of mean + eps, :365 product with weight and input) but keeps
    the scale and the products in fp32 where the kernel rounds them to bf16."""
    xf = x.detach().cpu().float()
    wf = weight.detach().cpu().float()
    inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return ((xf * inv) * wf).to(torch.bfloat16)
