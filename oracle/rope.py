"""Rotary-embedding oracle (test infrastructure): table pinned by golden rows, rotation unpinned."""
from __future__ import annotations

import math

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


def rot_embed_reference(x: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """x [B,S,H,D] bf16, freq fp32 [S,D] -> dense bf16 [B,S,H,D].

    custom_rot_embed_kernel (custom_kernels/custom_kernels.cu:400-412): pair (x, y) = in[2i], in[2i+1];
    (c, s) = freq[tok*D + 2i], freq[tok*D + 2i + 1]; x' = x*c - y*s, y' = x*s + y*c in fp32 (each
    product rounded on its own), one rounding to bf16."""
    xf = x.detach().cpu().float()
    B, S, H, D = xf.shape
    f = freq.detach().cpu().float().reshape(S, D // 2, 2)
    c = f[:, :, 0].view(1, S, 1, D // 2)
    s = f[:, :, 1].view(1, S, 1, D // 2)
    xe, xo = xf[..., 0::2], xf[..., 1::2]
    re = xe * c - xo * s
    im = xe * s + xo * c
    return torch.stack([re, im], dim=-1).flatten(-2).to(torch.bfloat16)
