"""Host-side multi-GPU logic on the CPU: batch partition, KV-sequence shard bounds, and the exchange of
shard results between two gloo ranks followed by a log-sum-exp merge (the oracle plays the kernel)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import load_package
from oracle import attention, inputs


def test_partition_batch_balances_tokens(pkg):
    lens = [2048, 1024, 1500, 1100, 1900, 1300, 1700, 1200, 2000, 1050, 1450, 1850, 1250, 1650, 1950, 1150]
    for world in (1, 2, 4, 8):
        parts = pkg.sharding.partition_batch(lens, world)
        assert sorted(i for p in parts for i in p) == list(range(16))
        loads = [sum(lens[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(lens)
        assert max(loads) <= 1.1 * sum(lens) / world
    parts = pkg.sharding.partition_batch([5, 9], 4)
    assert sorted(map(len, parts)) == [0, 0, 1, 1]
    with pytest.raises(ValueError):
        pkg.sharding.partition_batch(lens, 0)


def test_kv_shard_bounds_cover_the_sequence(pkg):
    for n_seq in (0, 1, 63, 64, 65, 1000, 131072):
        for world in (1, 2, 3, 4, 8):
            b = pkg.sharding.kv_shard_bounds(n_seq, world)
            assert len(b) == world and b[0][0] == 0 and b[-1][1] == n_seq
            assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
            assert all(lo % 64 == 0 and lo <= hi for lo, hi in b)
    assert pkg.sharding.kv_shard_bounds(131072, 8) == [(i * 16384, (i + 1) * 16384) for i in range(8)]


def test_local_seq_lens(pkg):
    lens = torch.tensor([0, 10, 64, 100, 200], dtype=torch.int32)
    assert pkg.sharding.local_seq_lens(lens, 64, 128).tolist() == [0, 0, 0, 36, 64]
    assert pkg.sharding.local_seq_lens(lens, 0, 64).tolist() == [0, 10, 64, 64, 64]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, result_queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pkg = load_package()
        case = inputs.decode_case(2, 8, 2, 64, 300, seed=23, ragged=True, min_len=10)
        lo, hi = pkg.sharding.kv_shard_bounds(300, world)[rank]
        lens = pkg.sharding.local_seq_lens(case.seq_lens, lo, hi)
        # the oracle stands in for flash_attention_decode_partial on this rank's shard
        o, lse = attention.attention_float64(case.q, case.k[:, :, lo:hi], case.v[:, :, lo:hi], lens)
        o = torch.from_numpy(o[:, :, 0]).float()
        lse = torch.from_numpy(lse).float()
        o_parts, lse_parts = pkg.sharding.exchange_partials(o, lse)
        assert o_parts.shape == (world, 2, 8, 64) and lse_parts.shape == (world, 2, 8)
        assert torch.equal(o_parts[rank], o) and torch.equal(lse_parts[rank], lse)
        merged = attention.lse_merge_reference(o_parts, lse_parts)
        full = attention.sdpa_reference(case.q, case.k, case.v, case.seq_lens)[:, :, 0]
        result_queue.put((rank, float((merged - full).abs().max())))
    finally:
        dist.destroy_process_group()


def test_two_rank_exchange_and_merge_over_gloo():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r for r, _ in results) == [0, 1]
    assert all(err < 1e-5 for _, err in results)
