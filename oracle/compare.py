"""Comparators used by the parity tests (test infrastructure)."""
from __future__ import annotations

import torch


def bf16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in units of bf16 representable values between two bf16 tensors (int64, elementwise).

    bf16 bit patterns are mapped to a monotonic integer line (sign-magnitude to two's complement), so
    that neighbouring values differ by 1 and +0/-0 coincide."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16

    def key(t: torch.Tensor) -> torch.Tensor:
        bits = t.contiguous().view(torch.int16).to(torch.int64) & 0xFFFF
        mag = bits & 0x7FFF
        return torch.where(bits >= 0x8000, -mag, mag)

    return (key(a) - key(b)).abs()


def max_bf16_ulp(a: torch.Tensor, b: torch.Tensor) -> int:
    return int(bf16_ulp_distance(a.cpu(), b.cpu()).max().item()) if a.numel() else 0


def assert_close_attention(actual: torch.Tensor, expected_fp32: torch.Tensor, atol: float = 2e-2, rtol: float = 1e-2,
                           max_rel_l2: float = 1e-2) -> None:
    """The stated attention tolerance (2e-2 absolute, 1e-2 relative, against an fp32 reference), plus a
    relative L2 bound over the whole output: at long sequence lengths the outputs of N(0,1) values are
    themselves ~1e-2, where the absolute bound alone would accept all-zeros."""
    a = actual.detach().float().cpu()
    e = expected_fp32.detach().float().cpu()
    assert a.shape == e.shape, (a.shape, e.shape)
    assert torch.isfinite(a).all(), "non-finite values in the kernel output"
    err = (a - e).abs()
    bound = atol + rtol * e.abs()
    worst = (err - bound).max().item()
    assert worst <= 0, f"max |err| {err.max().item():.4g} exceeds atol {atol} + rtol {rtol}*|ref| by {worst:.4g}"
    denom = e.norm().item()
    if denom > 0:
        rel = (a - e).norm().item() / denom
        assert rel <= max_rel_l2, f"relative L2 error {rel:.4g} > {max_rel_l2}"
