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


def rms_norm_reference_rounding(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm with the rounding order of the reference's kernel: the sum of squares in fp32
    (custom_kernels/custom_kernels.cu:354-360), then `inv = bf16(rsqrt(ss / E + eps))` (:362) and
    `out = bf16(bf16(inv * w) * x)` (:365, two bf16 multiplications evaluated left to right).  Three roundings
    where `rms_norm_reference` has one; the two differ by at most 2 bf16 ulp."""
    xf = x.detach().cpu().float()
    inv = torch.rsqrt(xf.pow(2).sum(dim=-1, keepdim=True) / x.shape[-1] + eps).to(torch.bfloat16)
    iw = (inv.float() * weight.detach().cpu().float()).to(torch.bfloat16)
    return (iw.float() * xf).to(torch.bfloat16)


def add_rms_norm_reference(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """(s, rmsnorm(s)) with s = x + residual as a bf16 tensor add gives it: Block.forward's residual add
    followed by the next norm (model.py:147-148), the two steps kept separate as the reference runs them."""
    s = (x.detach().cpu().float() + residual.detach().cpu().float()).to(torch.bfloat16)
    return s, rms_norm_reference(s, weight, eps)


def silu_mul_reference(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """F.silu(gate) * up on bf16 tensors (MLP.forward, model.py:134): silu in fp32 rounded to bf16, then
    the product rounded to bf16."""
    g = gate.detach().cpu().float()
    s = (g / (1.0 + torch.exp(-g))).to(torch.bfloat16)
    return (s.float() * up.detach().cpu().float()).to(torch.bfloat16)
