"""Nucleus (top-p) sampling oracle (test infrastructure).

`sample_top_p_reference` restates the reference's `sample_top_p` (model.py:400-423) operation for operation, so
that under the same torch RNG state it returns the same tokens; PINNED by tokens the reference's own function drew
(tests/golden/reference_vectors.pt, keys top_p_*).  `nucleus_reference` gives what the sampler draws from: the kept
set and its renormalised probabilities, with the preceding mass of every entry in float64 so that a test can tell
entries that sit on the boundary within fp32 rounding from entries that are clearly in or out."""
from __future__ import annotations

import torch


def softmax_with_temperature(logits: torch.Tensor, temperature: float, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """`torch.softmax(logits[:, -1] / temperature, dim=-1)` (model.py:368) on the widened logits (model.py:226).
    The reference evaluates it in fp32; over 128 256 entries torch's fp32 sum of exponentials can be off by up to
    ~1e-4 relative (many equal small terms round the same way), which moves the nucleus boundary by dozens of
    entries.  `dtype=torch.float64` gives the formula's exact value, which is what a kernel is held to."""
    return torch.softmax(logits.detach().cpu().to(dtype) / temperature, dim=-1)


def sample_top_p_reference(probs: torch.Tensor, p: float) -> torch.Tensor:
    """model.py:400-423: sort descending, cumulative sum, zero the entries whose preceding mass exceeds p,
    renormalise, one multinomial draw per row, map back through the sort permutation.  Returns [rows, 1]."""
    probs_sort, probs_idx = torch.sort(probs, dim=-1, descending=True)
    probs_sum = torch.cumsum(probs_sort, dim=-1)
    mask = probs_sum - probs_sort > p
    probs_sort[mask] = 0.0
    probs_sort.div_(probs_sort.sum(dim=-1, keepdim=True))
    next_token = torch.multinomial(probs_sort, num_samples=1)
    return torch.gather(probs_idx, -1, next_token)


def nucleus_reference(probs: torch.Tensor, p: float):
    """For probs [rows, vocab]: (kept [rows, vocab] bool, renormalised probabilities of the kept entries
    [rows, vocab] float64, preceding mass of every entry [rows, vocab] float64).  Descending order with equal
    entries in index order (a stable sort); an entry is kept iff the mass before it is <= p (model.py:416)."""
    pr = probs.detach().cpu().double()
    order = torch.sort(pr, dim=-1, descending=True, stable=True).indices
    sorted_p = torch.gather(pr, -1, order)
    before_sorted = torch.cumsum(sorted_p, dim=-1) - sorted_p
    before = torch.empty_like(pr).scatter_(-1, order, before_sorted)
    kept = before <= p
    renorm = torch.where(kept, pr, torch.zeros_like(pr))
    renorm = renorm / renorm.sum(dim=-1, keepdim=True)
    return kept, renorm, before
