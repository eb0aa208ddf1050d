"""Rotary-embedding oracle (test infrastructure): table pinned by golden rows of the reference's model.py,
rotation pinned by outputs of the reference's CUDA kernel (tests/golden/reference_cuda_vectors.pt)."""
from __future__ import annotations

import math

import numpy as np
import torch


def apply_scaling_reference(freqs: torch.Tensor, scale_factor: float = 8, low_freq_factor: float = 1,
                            high_freq_factor: float = 4, old_context_len: int = 8192) -> torch.Tensor:
    """One frequency at a time, as model.py:27-49 walks them (fp32 scalars throughout)."""
    low_freq_wavelen = old_context_len / low_freq_factor
    high_freq_wavelen = old_context_len / high_freq_factor
    out = []
    for f in freqs:  # f is a 0-dim fp32 tensor, so every operation below rounds to fp32
        wavelen = 2 * math.pi / f
        if wavelen < high_freq_wavelen:
            out.append(f)
        elif wavelen > low_freq_wavelen:
            out.append(f / scale_factor)
        else:
            smooth = (old_context_len / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
            out.append((1 - smooth) * f / scale_factor + smooth * f)
    return torch.tensor(out, dtype=freqs.dtype)


def freqs_cis_reference(dim: int, end: int, theta: float = 10000.0, use_scaled: bool = False, **scaling) -> torch.Tensor:
    """fp32 [end, dim] interleaved (cos, sin) table, model.py:51-60."""
    freqs = 1.0 / (theta ** (torch.arange(0, dim, 2)[: dim // 2].float() / dim))
    if use_scaled:
        freqs = apply_scaling_reference(freqs, **scaling)
    angles = torch.outer(torch.arange(end, dtype=torch.float32), freqs)
    cis = torch.polar(torch.ones_like(angles), angles)
    return torch.view_as_real(cis).flatten(1)


def rot_embed_reference_unfused(x: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """x [B,S,H,D] bf16, freq fp32 [S,D] -> dense bf16 [B,S,H,D].

    custom_rot_embed_kernel (custom_kernels/custom_kernels.cu:400-412): pair (x, y) = in[2i], in[2i+1];
    (c, s) = freq[tok*D + 2i], freq[tok*D + 2i + 1]; x' = x*c - y*s, y' = x*s + y*c in fp32 with each
    product rounded on its own (the source as written, without the compiler's contraction), one rounding to
    bf16.  Differs from the compiled kernel's outputs in about 1e-5 of the elements (by up to 10 bf16 ulp where
    the two terms nearly cancel); kept as the baseline those differences are recorded against."""
    xf = x.detach().cpu().float()
    B, S, H, D = xf.shape
    f = freq.detach().cpu().float().reshape(S, D // 2, 2)
    c = f[:, :, 0].view(1, S, 1, D // 2)
    s = f[:, :, 1].view(1, S, 1, D // 2)
    xe, xo = xf[..., 0::2], xf[..., 1::2]
    re = xe * c - xo * s
    im = xe * s + xo * c
    return torch.stack([re, im], dim=-1).flatten(-2).to(torch.bfloat16)


def _fma_f32(a: np.ndarray, b: np.ndarray, c: np.ndarray) -> np.ndarray:
    """Correctly rounded fp32 fused multiply-add a*b + c of fp32 values, computed in float64: the product of two
    fp32 numbers is exact in float64; the sum is rounded to 53 bits, and where that lands exactly half way between
    two fp32 numbers the exact residual of the sum (TwoSum) decides the direction."""
    a64, b64, c64 = a.astype(np.float64), b.astype(np.float64), c.astype(np.float64)
    p = a64 * b64
    s = p + c64
    bb = s - p
    e = (p - (s - bb)) + (c64 - bb)
    half_way = (s.view(np.uint64) & np.uint64(0x1FFFFFFF)) == np.uint64(0x10000000)
    nudge = half_way & (e != 0)
    s = np.where(nudge, np.nextafter(s, np.where(e > 0, np.inf, -np.inf)), s)
    return s.astype(np.float32)


def rot_embed_reference_fma(x: torch.Tensor, freq: torch.Tensor, form: str = "ab") -> torch.Tensor:
    """The rotation as the reference's COMPILED kernel evaluates it: nvcc contracts each of the two expressions of
    custom_kernels/custom_kernels.cu:408,410 into one rounded product and one fused multiply-add.  `form` names
    which product stays a separate rounding in (x', y'): 'a' = the first of the expression, 'b' = the second.
      x' = x*c - y*s:  'a' -> fma(-y, s, rn(x*c));  'b' -> fma(x, c, -rn(y*s))
      y' = x*s + y*c:  'a' -> fma(y, c, rn(x*s));   'b' -> fma(x, s, rn(y*c))
    Which form the compiler took is read off the reference's own outputs (tests/test_oracle_golden.py)."""
    xf = x.detach().cpu().float()
    B, S, H, D = xf.shape
    f = freq.detach().cpu().float().reshape(S, D // 2, 2)
    c = np.broadcast_to(f[:, :, 0].view(1, S, 1, D // 2).numpy(), (B, S, H, D // 2))
    s = np.broadcast_to(f[:, :, 1].view(1, S, 1, D // 2).numpy(), (B, S, H, D // 2))
    xe, xo = xf[..., 0::2].numpy(), xf[..., 1::2].numpy()
    re = _fma_f32(-xo, s, xe * c) if form[0] == "a" else _fma_f32(xe, c, -(xo * s))
    im = _fma_f32(xo, c, xe * s) if form[1] == "a" else _fma_f32(xe, s, xo * c)
    out = torch.stack([torch.from_numpy(re), torch.from_numpy(im)], dim=-1).flatten(-2)
    return out.to(torch.bfloat16)


def rot_embed_reference(x: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """x [B,S,H,D] bf16, freq fp32 [S,D] -> dense bf16 [B,S,H,D]: `rot_embed(input, freq)`
    (custom_kernels/custom_kernels.cu:391-442) with the rounding of the compiled kernel, form 'bb' of
    `rot_embed_reference_fma`.  PINNED: bit-equal to the reference kernel's outputs on every element of
    configuration 4 and of the small shapes (tests/golden/reference_cuda_vectors.pt)."""
    return rot_embed_reference_fma(x, freq, "bb")
