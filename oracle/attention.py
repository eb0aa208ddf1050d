"""Decode-attention oracle (test infrastructure): the reference's PyTorch path, pinned by golden vectors."""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F


def length_mask(seq_lens: torch.Tensor, n_seq: int) -> torch.Tensor:
    """bool [B,1,1,S]: True where the cached position is valid (s < len[b])."""
    pos = torch.arange(n_seq).view(1, 1, 1, n_seq)
    return pos < seq_lens.detach().cpu().to(torch.int64).view(-1, 1, 1, 1)


def sdpa_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_lens: Optional[torch.Tensor] = None,
                   scale: Optional[float] = None, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """`F.scaled_dot_product_attention(q, k, v, enable_gqa=True)` on CPU (model.py:115-116,
    benchmark_kernel.py:27-28), by default evaluated in fp32 on the bf16 inputs widened exactly.

    q [B,Hq,1,D]; k, v [B,Hkv,S,D]; scale None = 1/sqrt(D) (custom_kernels/custom_kernels.cu:253).
    `seq_lens` (optional, [B]) masks cached positions >= len[b]; a sequence with no valid position
    yields zeros (SDPA itself would yield NaN; the kernels define it as zeros)."""
    qc, kc, vc = (t.detach().cpu().to(dtype) for t in (q, k, v))
    mask = None
    if seq_lens is not None:
        mask = length_mask(seq_lens, k.shape[2])
    out = F.scaled_dot_product_attention(qc, kc, vc, attn_mask=mask, scale=scale, enable_gqa=True)
    if seq_lens is not None:
        empty = seq_lens.detach().cpu().view(-1) <= 0
        if empty.any():
            out = out.clone()
            out[empty] = 0
    return out


def attention_float64(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_lens: Optional[torch.Tensor] = None,
                      scale: Optional[float] = None) -> Tuple[np.ndarray, np.ndarray]:
    """Independent restatement in float64 numpy: returns (out [B,Hq,1,D], lse [B,Hq]).

    Query head h reads KV head h // (Hq // Hkv) (the grouping of custom_kernels/custom_kernels.cu:55,
    `head * QKV_HEAD_RATIO + query_idx`, and of SDPA's enable_gqa).  lse is the natural-log sum-exp of the
    scaled scores, -inf for an empty sequence."""
    qn = q.detach().cpu().float().numpy().astype(np.float64)
    kn = k.detach().cpu().float().numpy().astype(np.float64)
    vn = v.detach().cpu().float().numpy().astype(np.float64)
    B, Hq, _, D = qn.shape
    Hkv, S = kn.shape[1], kn.shape[2]
    R = Hq // Hkv
    sc = 1.0 / np.sqrt(D) if scale is None else scale
    lens = [S] * B if seq_lens is None else [int(x) for x in seq_lens.detach().cpu().tolist()]
    out = np.zeros((B, Hq, 1, D))
    lse = np.full((B, Hq), -np.inf)
    for b in range(B):
        n = max(0, min(S, lens[b]))
        if n == 0:
            continue
        for h in range(Hq):
            s = (kn[b, h // R, :n] @ qn[b, h, 0]) * sc
            m = s.max()
            p = np.exp(s - m)
            out[b, h, 0] = (p @ vn[b, h // R, :n]) / p.sum()
            lse[b, h] = m + np.log(p.sum())
    return out, lse


def lse_merge_reference(o_parts: torch.Tensor, lse_parts: torch.Tensor) -> torch.Tensor:
    """fp32 merge of shard results: out = sum_p softmax_p(lse)[p] * o[p]; o_parts [P,B,Hq,D], lse_parts [P,B,Hq].
    The formula the reference's combine kernel aims at (custom_kernels/custom_kernels.cu:198-222)."""
    o = o_parts.detach().cpu().double()
    l = lse_parts.detach().cpu().double()
    m = l.max(dim=0, keepdim=True).values
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(l - m)
    tot = w.sum(dim=0, keepdim=True)
    w = torch.where(tot > 0, w / tot.clamp_min(1e-300), torch.zeros_like(w))
    return (w.unsqueeze(-1) * o).sum(dim=0).float()


def prefill_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, start_pos: int = 0,
                      scale: Optional[float] = None, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Causal attention of T new tokens: the reference's prefill call (model.py:114-116,
    `F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)` over the first T cache rows),
    on CPU in fp32 by default.  q [B,Hq,T,D]; k, v [B,Hkv,S,D].  With start_pos > 0 (a later chunk) the same call
    takes the explicit mask j <= start_pos + t instead of `is_causal`."""
    qc, kc, vc = (t.detach().cpu().to(dtype) for t in (q, k, v))
    T, S = q.shape[2], k.shape[2]
    if start_pos == 0 and S == T:
        return F.scaled_dot_product_attention(qc, kc, vc, is_causal=True, scale=scale, enable_gqa=True)
    mask = torch.arange(S).view(1, S) <= (start_pos + torch.arange(T)).view(T, 1)
    return F.scaled_dot_product_attention(qc, kc, vc, attn_mask=mask.view(1, 1, T, S), scale=scale, enable_gqa=True)
