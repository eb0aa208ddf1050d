"""Rotary-embedding table for the rot_embed kernels, with the Llama-3 frequency scaling as parameters.

Host-side mirror of `precompute_freqs_cis` / `apply_scaling` (model.py:51-60, 27-49).  The reference
hard-codes scale_factor=8, low_freq_factor=1, high_freq_factor=4 and an original context of 8192
(model.py:29-32); here they are arguments (Llama-3.2 checkpoints use a factor of 32).  With the
reference's values the table is bit-identical to the reference's, which the tests check against
vectors produced by the reference itself.

The table is fp32 [end, dim]: row t holds (cos(t*f_0), sin(t*f_0), cos(t*f_1), sin(t*f_1), ...),
the layout `custom_rot_embed_kernel` reads as float2 per rotation pair
(custom_kernels/custom_kernels.cu:400-401).
"""
from __future__ import annotations

import math

import torch


def apply_scaling(freqs: torch.Tensor, scale_factor: float = 8, low_freq_factor: float = 1,
                  high_freq_factor: float = 4, old_context_len: int = 8192) -> torch.Tensor:
    """Llama-3 scaling of the rotary frequencies, all frequencies at once in fp32.

    A frequency whose wavelength is shorter than old_context_len/high_freq_factor is kept, one whose
    wavelength is longer than old_context_len/low_freq_factor is divided by scale_factor, and the band
    in between is blended linearly in old_context_len/wavelength (model.py:34-48).
    """
    if low_freq_factor == high_freq_factor:
        raise ValueError("low_freq_factor and high_freq_factor must differ")
    low_freq_wavelen = old_context_len / low_freq_factor
    high_freq_wavelen = old_context_len / high_freq_factor
    # Same operation order as the scalar reference: python_scalar / tensor is reciprocal() * scalar.
    wavelen = freqs.reciprocal() * (2 * math.pi)
    smooth = (wavelen.reciprocal() * old_context_len - low_freq_factor) / (high_freq_factor - low_freq_factor)
    blended = (1 - smooth) * freqs / scale_factor + smooth * freqs
    scaled = torch.where(wavelen > low_freq_wavelen, freqs / scale_factor, blended)
    return torch.where(wavelen < high_freq_wavelen, freqs, scaled).to(freqs.dtype)


def precompute_freqs_cis(dim: int, end: int, theta: float = 10000.0, use_scaled: bool = False,
                         scale_factor: float = 8, low_freq_factor: float = 1, high_freq_factor: float = 4,
                         old_context_len: int = 8192) -> torch.Tensor:
    """fp32 [end, dim] table of interleaved (cos, sin) for positions 0..end-1 (model.py:51-60)."""
    freqs = 1.0 / (theta ** (torch.arange(0, dim, 2)[: (dim // 2)].float() / dim))
    if use_scaled:
        freqs = apply_scaling(freqs, scale_factor, low_freq_factor, high_freq_factor, old_context_len)
    t = torch.arange(end, dtype=torch.float32)
    angles = torch.outer(t, freqs)
    return torch.view_as_real(torch.polar(torch.ones_like(angles), angles)).flatten(1)
