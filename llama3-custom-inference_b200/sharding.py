"""Partition of decode attention over the GPUs of one box (one process per GPU).

The reference is single-GPU (README.md:13); this is the host logic for the two ways its decode
attention shards:

* by (sequence, kv head): units are independent, every rank owns the outputs of its sequences and no
  data crosses GPUs (`partition_batch`);
* by KV sequence for one very long context: rank r holds the tokens [lo_r, hi_r) of every sequence,
  computes attention over them as an fp32 (o, lse) pair, the pairs are all-gathered
  ((D + 1) * Hq * 4 bytes per sequence and rank) and merged by log-sum-exp on every rank
  (`kv_shard_bounds`, `local_seq_lens`, `exchange_partials`, `decode_kv_sharded`).

Only `decode_kv_sharded` touches a GPU; the rest is integer arithmetic and `torch.distributed`
plumbing that also runs over gloo on CPU.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def partition_batch(seq_lens: Sequence[int], world: int) -> List[List[int]]:
    """Deals sequence indices to `world` ranks so that the cached tokens per rank are as even as a
    greedy longest-first assignment makes them.  Every index appears exactly once; ranks may be empty
    when there are fewer sequences than ranks."""
    if world <= 0:
        raise ValueError("world must be positive")
    order = sorted(range(len(seq_lens)), key=lambda i: (-int(seq_lens[i]), i))
    loads = [0] * world
    parts: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (loads[j], j))
        parts[r].append(i)
        loads[r] += int(seq_lens[i])
    for p in parts:
        p.sort()
    return parts


def kv_shard_bounds(n_seq: int, world: int, align: int = 64) -> List[Tuple[int, int]]:
    """Contiguous token ranges [lo, hi) of the `world` KV shards; boundaries are multiples of `align`
    (whole tiles of the decode kernel) except the last, and ranges may be empty for short sequences."""
    if world <= 0 or n_seq < 0 or align <= 0:
        raise ValueError("bad arguments")
    blocks = (n_seq + align - 1) // align
    bounds = []
    for r in range(world):
        lo = min(n_seq, (blocks * r // world) * align)
        hi = min(n_seq, (blocks * (r + 1) // world) * align)
        bounds.append((lo, hi))
    return bounds


def local_seq_lens(seq_lens: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    """Valid tokens of each sequence that fall into the shard [lo, hi): clamp(len - lo, 0, hi - lo)."""
    return (seq_lens.to(torch.int64) - lo).clamp_(0, hi - lo).to(torch.int32)


def exchange_partials(o: torch.Tensor, lse: torch.Tensor, group: Optional[dist.ProcessGroup] = None
                      ) -> Tuple[torch.Tensor, torch.Tensor]:
    """All-gathers the per-rank fp32 results o [B,Hq,D] and lse [B,Hq]; returns o_parts [W,B,Hq,D] and
    lse_parts [W,B,Hq] in rank order.  One collective: o and lse travel in one packed buffer."""
    world = dist.get_world_size(group)
    B, Hq, D = o.shape
    packed = torch.cat([o, lse.unsqueeze(-1)], dim=-1).contiguous()  # [B, Hq, D + 1]
    gathered = [torch.empty_like(packed) for _ in range(world)]
    dist.all_gather(gathered, packed, group=group)
    allp = torch.stack(gathered, dim=0)
    return allp[..., :D].contiguous(), allp[..., D].contiguous()


def decode_kv_sharded(ext, q: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor,
                      seq_lens_local: Optional[torch.Tensor] = None,
                      group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Decode attention of q [B,Hq,1,D] (replicated) over a KV cache whose sequence axis is sharded
    across the ranks of `group`; k_local / v_local are this rank's [B,Hkv,S_local,D] slices.
    `ext` is the extension module (`custom_kernels_extension`).  Returns bf16 [B,Hq,1,D] on every rank."""
    o, lse = ext.flash_attention_decode_partial(q, k_local, v_local, seq_lens=seq_lens_local)
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return ext.lse_merge(o.unsqueeze(0), lse.unsqueeze(0))
    o_parts, lse_parts = exchange_partials(o, lse, group)
    return ext.lse_merge(o_parts, lse_parts)
