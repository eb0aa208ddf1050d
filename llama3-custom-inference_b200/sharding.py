"""Partition of decode attention over the GPUs of one box (one process per GPU).

The reference is single-GPU (README.md:13); this is the host logic for the two ways its decode
attention shards:

* by (sequence, kv head): units are independent, every rank owns the outputs of its sequences and no
  data crosses GPUs (`partition_batch`);
* by KV sequence for one very long context: rank r holds the tokens [lo_r, hi_r) of every sequence,
  computes attention over them as an fp32 (o, lse) pair, the pairs are all-gathered
  ((D + 1) * Hq * 4 bytes per sequence and rank) and merged by log-sum-exp on every rank
  (`kv_shard_bounds`, `local_seq_lens`, `exchange_partials`, `decode_kv_sharded`).

`KvShardExchange` + `decode_kv_sharded_fused` replace the all-gather and the merge kernel by pushes of the rank's
result into its peers' memory over NVLink and a merge of what the peers pushed; the buffers are torch symmetric
memory.  Where the shard goes to the static-deal decode kernel (the usual case) all of that happens in the decode
kernel's own tail, ONE launch per rank and step (`flash_attention_decode_exchange`); otherwise the decode kernel is
followed by one exchange + merge kernel (`lse_exchange_merge`).

Only `decode_kv_sharded*` touch a GPU; the rest is integer arithmetic and `torch.distributed`
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


class KvShardExchange:
    """Peer-addressable buffers for the fused exchange + merge of shard results on one box.

    One instance per (process group, B, Hq, D).  Construction is collective (every rank of `group` must create
    it in the same order): it allocates torch symmetric memory of `lse_exchange_bytes` bytes, zero-fills it and
    exchanges the handles.  `slot()` gives the fp32 views this rank's decode kernel writes its shard result to;
    `merge()` launches the fused kernel.  Calls are numbered by an epoch that advances identically on all
    ranks, so every rank must make the same sequence of `slot()` / `merge()` calls."""

    def __init__(self, ext, B: int, Hq: int, D: int, device, group: Optional[dist.ProcessGroup] = None):
        import torch.distributed._symmetric_memory as symm_mem

        self.ext, self.B, self.Hq, self.D = ext, B, Hq, D
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        nbytes = ext.lse_exchange_bytes(self.world, B, Hq, D)
        self.buf = symm_mem.empty(nbytes // 4, dtype=torch.float32, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, self.group.group_name)
        self.bufs = torch.tensor(list(self.handle.buffer_ptrs), dtype=torch.int64, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.rows = B * Hq
        self.slot_floats = self.rows * D + ((self.rows + 3) & ~3)
        # behind the data and the flags: a staging slot for this rank's own result, then the control words
        self.staging_base = 2 * self.world * self.slot_floats + ((2 * self.world * self.rows + 3) & ~3)
        self.epoch = 0
        # second buffer: the exchange done in the decode kernel's own tail (one launch per step), with its own layout
        nbytes1 = ext.flash_decode_exchange_bytes(self.world, B, Hq, D)
        self.buf1 = symm_mem.empty(nbytes1 // 8, dtype=torch.int64, device=device)
        self.buf1.zero_()
        self.handle1 = symm_mem.rendezvous(self.buf1, self.group.group_name)
        self.bufs1 = torch.tensor(list(self.handle1.buffer_ptrs), dtype=torch.int64, device=device)
        self.epoch1 = 0
        self.one_launch = None         # None: not tried yet; False: these sizes take the two-launch path
        torch.cuda.synchronize(device)
        self.handle.barrier()          # every rank's buffers are zeroed before anyone may push into them
        self.handle1.barrier()

    def slot(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Starts the next exchange and returns (o [B,Hq,D], lse [B,Hq]) views of this rank's own slot."""
        self.epoch += 1
        base = ((self.epoch & 1) * self.world + self.rank) * self.slot_floats
        o = self.buf[base: base + self.rows * self.D].view(self.B, self.Hq, self.D)
        lse = self.buf[base + self.rows * self.D: base + self.rows * self.D + self.rows].view(self.B, self.Hq)
        return o, lse

    def staging(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(o [B,Hq,D], lse [B,Hq]) views of the staging slot: where this rank's shard result goes when the call
        number is kept on the device (`merge_auto`).  The address never changes, so a decode step that writes
        there and calls `merge_auto` can be captured in a CUDA graph."""
        base = self.staging_base
        o = self.buf[base: base + self.rows * self.D].view(self.B, self.Hq, self.D)
        lse = self.buf[base + self.rows * self.D: base + self.rows * self.D + self.rows].view(self.B, self.Hq)
        return o, lse

    def merge_auto(self) -> torch.Tensor:
        """`merge` with the call number kept in the buffer itself (no host state); use either this or
        `slot()` / `merge()` on an instance, not both."""
        return self.ext.lse_exchange_merge(self.bufs, self.rank, 0, self.B, self.Hq, self.D, status=self.status)

    def merge(self) -> torch.Tensor:
        """Pushes this rank's slot to the peers, waits for theirs, merges: bf16 [B,Hq,1,D] on every rank."""
        return self.ext.lse_exchange_merge(self.bufs, self.rank, self.epoch, self.B, self.Hq, self.D,
                                           status=self.status)

    def check(self) -> int:
        """Synchronises and returns the device status word (0 = every wait was satisfied)."""
        return int(self.status.item())


def decode_kv_sharded_fused(ext, q: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor,
                            xchg: KvShardExchange, seq_lens_local: Optional[torch.Tensor] = None,
                            device_epoch: bool = False) -> torch.Tensor:
    """`decode_kv_sharded` with the exchange and the merge over peer memory and no collective call: one launch per
    step where the shard takes the static-deal decode kernel (exchange in its tail), else two (shard attention into
    the exchange buffer, then push + wait + merge).  With `device_epoch` the step keeps no host state (fixed
    addresses, call number in the buffer) and can be captured in a CUDA graph."""
    if xchg.one_launch is not False and xchg.world <= 8:
        # the exchange in the decode kernel's tail; the library says when the head layout has no such kernel (more
        # than 8 query heads per KV head), which is the same answer on every rank
        epoch = 0
        if not device_epoch:
            xchg.epoch1 += 1
            epoch = xchg.epoch1
        # (max_ctas = -1: the static-deal kernel whatever the shard's length, so that every rank takes the same
        # path even when the last shard is shorter than the others)
        out = ext.flash_attention_decode_exchange(q, k_local, v_local, xchg.bufs1, xchg.rank, epoch,
                                                  seq_lens=seq_lens_local, status=xchg.status, max_ctas=-1)
        xchg.one_launch = out is not None
        if out is not None:
            return out
        if not device_epoch:
            xchg.epoch1 -= 1
    o, lse = xchg.staging() if device_epoch else xchg.slot()
    ext.flash_attention_decode_partial(q, k_local, v_local, seq_lens=seq_lens_local, out_o=o, out_lse=lse)
    return xchg.merge_auto() if device_epoch else xchg.merge()
