"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations
(test infrastructure).  Values are drawn in fp32 on the CPU from torch.Generator().manual_seed(seed)
(42 is the reference's seed, benchmark_kernel.py:126,158) and rounded to bf16; K and V are built as
[B, S, Hkv, D] and returned transposed to [B, Hkv, S, D], the strided layout the model hands to the
kernel (model.py:89,107,111; benchmark_kernel.py:165-173)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class DecodeCase:
    q: torch.Tensor                    # [B, Hq, 1, D] view of [B, 1, Hq, D]
    k: torch.Tensor                    # [B, Hkv, S, D] view of [B, S, Hkv, D]
    v: torch.Tensor
    seq_lens: Optional[torch.Tensor]   # int32 [B] or None

    def to(self, device) -> "DecodeCase":
        mv = lambda t: None if t is None else t.to(device)
        # .to() keeps the strides of these dense-but-permuted tensors
        return DecodeCase(mv(self.q), mv(self.k), mv(self.v), mv(self.seq_lens))


def decode_case(B: int, Hq: int, Hkv: int, D: int, S: int, seed: int = 42, ragged: bool = False,
                min_len: int = 1, dist: str = "normal") -> DecodeCase:
    g = torch.Generator().manual_seed(seed)
    draw = (lambda *s: torch.randn(*s, generator=g)) if dist == "normal" else (lambda *s: torch.rand(*s, generator=g))
    q = draw(B, 1, Hq, D).bfloat16().transpose(1, 2)
    k = draw(B, S, Hkv, D).bfloat16().transpose(1, 2)
    v = draw(B, S, Hkv, D).bfloat16().transpose(1, 2)
    lens = None
    if ragged:
        lens = torch.randint(min_len, S + 1, (B,), generator=g, dtype=torch.int32)
    return DecodeCase(q, k, v, lens)


def config1(seed: int = 42) -> DecodeCase:
    """Llama-3.2-1B decode step: B=1, 32 q / 8 kv heads, D=64, 256 cached tokens."""
    return decode_case(1, 32, 8, 64, 256, seed)


def config2(seed: int = 42) -> DecodeCase:
    """Llama-3.1-8B batched decode: B=16, 32/8 heads, D=128, lengths uniform in [1024, 2048], cache padded
    to 2048 with N(0,1) values that the kernel must ignore."""
    return decode_case(16, 32, 8, 128, 2048, seed, ragged=True, min_len=1024)


def config3(seed: int = 42, S: int = 131072) -> DecodeCase:
    """Long-context decode: B=1, 32/8 heads, D=128, S=131072."""
    return decode_case(1, 32, 8, 128, S, seed)


def config4(seed: int = 42, B: int = 2, S: int = 2048, hidden: int = 2048, n_head: int = 32, n_kv_head: int = 8,
            D: int = 64):
    """Pre-attention block: x [B,S,hidden] ~ N(0,1), w ~ N(1,0.02), eps 1e-5; fused projection output
    qkv [B,S,(n_head+2*n_kv_head)*D] ~ N(0,1) whose q / k parts are the strided rot_embed inputs."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, S, hidden, generator=g).bfloat16()
    w = (1.0 + 0.02 * torch.randn(hidden, generator=g)).bfloat16()
    qkv = torch.randn(B, S, (n_head + 2 * n_kv_head) * D, generator=g).bfloat16()
    return x, w, 1e-5, qkv


ROPE_CONFIG4 = dict(theta=500000.0, use_scaled=True, scale_factor=32, low_freq_factor=1, high_freq_factor=4,
                    old_context_len=8192)


def prefill_case(B: int, Hq: int, Hkv: int, D: int, T: int, seed: int = 42):
    """Seeded q [B,Hq,T,D], k, v [B,Hkv,T,D] in the model's layout (views of [B,T,H,D], model.py:96-112), bf16,
    N(0,1): the operands of the reference's prefill attention call (model.py:114-116)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, Hq, D, generator=g).bfloat16().transpose(1, 2)
    k = torch.randn(B, T, Hkv, D, generator=g).bfloat16().transpose(1, 2)
    v = torch.randn(B, T, Hkv, D, generator=g).bfloat16().transpose(1, 2)
    return q, k, v


def rms_case(B: int, S: int, E: int, seed: int):
    """x [B,S,E] ~ N(0,1) and weight [E] ~ N(1,0.02) in bf16: the operands of `rms_norm(input, weight, eps)`
    (custom_kernels/custom_kernels.cu:369-373) for a shape other than config 4's."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, S, E, generator=g).bfloat16()
    w = (1.0 + 0.02 * torch.randn(E, generator=g)).bfloat16()
    return x, w


def rope_case(B: int, S: int, H: int, D: int, seed: int, extra_heads: int = 0):
    """x [B,S,H,D] ~ N(0,1) in bf16, the operand of `rot_embed(input, freq)` (custom_kernels.cu:418-427).  With
    `extra_heads` the tensor is a strided view of a wider [B,S,(H+extra_heads)*D] buffer, as q and k are views
    of the fused projection output (model.py:95-97)."""
    g = torch.Generator().manual_seed(seed)
    buf = torch.randn(B, S, (H + extra_heads) * D, generator=g).bfloat16()
    return buf[..., : H * D].view(B, S, H, D)


# name -> (B, S, E, seed) of rms_case / (B, S, H, D, seed, extra_heads) of rope_case: the small shapes whose
# reference-CUDA outputs are held whole in tests/golden/reference_cuda_vectors.pt
RMS_GOLDEN_CASES = {"e64": (1, 3, 64, 31), "e512": (2, 5, 512, 32), "e2048_decode": (4, 1, 2048, 33),
                    "e4096": (3, 7, 4096, 34), "e8192": (1, 2, 8192, 35)}
ROPE_GOLDEN_CASES = {"d64": (1, 5, 3, 64, 41, 0), "d128_strided": (2, 17, 4, 128, 42, 2), "d64_decode": (8, 1, 32, 64, 43, 16)}
# rows of config 4 whose reference-CUDA outputs are held (the whole outputs are 17 MB each)
C4_GOLDEN_ROW_STEP = 64
