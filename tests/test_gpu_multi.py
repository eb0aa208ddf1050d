"""Two ranks on two GPUs (NCCL): a KV sequence sharded across the ranks, shard results exchanged and merged,
and a batch sharded by sequence with no exchange.  Skipped on a box with one GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import load_package
from oracle import attention, compare, inputs

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        pkg = load_package()
        ext = pkg.extension()
        # --- KV sequence sharded over the ranks, one all_gather, merge on every rank
        case = inputs.decode_case(2, 32, 8, 128, 6000, seed=61, ragged=True, min_len=100)
        lo, hi = pkg.sharding.kv_shard_bounds(6000, world)[rank]
        dc = case.to(dev)
        lens = pkg.sharding.local_seq_lens(dc.seq_lens, lo, hi)
        out = pkg.sharding.decode_kv_sharded(ext, dc.q, dc.k[:, :, lo:hi], dc.v[:, :, lo:hi], lens)
        torch.cuda.synchronize()
        want = attention.sdpa_reference(case.q, case.k, case.v, case.seq_lens)
        compare.assert_close_attention(out, want)
        # --- the same with the exchange over peer memory (plain stores over NVLink) in the decode kernel's tail,
        #     three steps in a row so that both parities of the exchange buffer and their reuse are exercised
        xchg = pkg.sharding.KvShardExchange(ext, 2, 32, 128, dev)
        for step in range(3):
            c = inputs.decode_case(2, 32, 8, 128, 6000, seed=70 + step, ragged=True, min_len=100)
            d = c.to(dev)
            ll = pkg.sharding.local_seq_lens(d.seq_lens, lo, hi)
            got = pkg.sharding.decode_kv_sharded_fused(ext, d.q, d.k[:, :, lo:hi], d.v[:, :, lo:hi], xchg, ll)
            torch.cuda.synchronize()
            compare.assert_close_attention(got, attention.sdpa_reference(c.q, c.k, c.v, c.seq_lens))
        assert xchg.check() == 0 and xchg.one_launch is True     # exchange in the decode kernel's own tail
        # --- the two-launch form (decode kernel, then exchange + merge kernel), kept for head layouts and sizes
        #     that go to the persistent decode kernel
        x2 = pkg.sharding.KvShardExchange(ext, 2, 32, 128, dev)
        x2.one_launch = False
        for step in range(3):
            c = inputs.decode_case(2, 32, 8, 128, 6000, seed=75 + step, ragged=True, min_len=100)
            d = c.to(dev)
            ll = pkg.sharding.local_seq_lens(d.seq_lens, lo, hi)
            got = pkg.sharding.decode_kv_sharded_fused(ext, d.q, d.k[:, :, lo:hi], d.v[:, :, lo:hi], x2, ll)
            torch.cuda.synchronize()
            compare.assert_close_attention(got, attention.sdpa_reference(c.q, c.k, c.v, c.seq_lens))
        assert x2.check() == 0
        # --- the call number kept on the device: no host state, so the two launches of a step can be captured in
        #     a CUDA graph; eager steps first (both parities), then replays of one captured step on new inputs
        xa = pkg.sharding.KvShardExchange(ext, 2, 32, 128, dev)
        for step in range(3):
            c = inputs.decode_case(2, 32, 8, 128, 6000, seed=80 + step, ragged=True, min_len=100)
            d = c.to(dev)
            ll = pkg.sharding.local_seq_lens(d.seq_lens, lo, hi)
            got = pkg.sharding.decode_kv_sharded_fused(ext, d.q, d.k[:, :, lo:hi], d.v[:, :, lo:hi], xa, ll, device_epoch=True)
            torch.cuda.synchronize()
            compare.assert_close_attention(got, attention.sdpa_reference(c.q, c.k, c.v, c.seq_lens))
        c0 = inputs.decode_case(2, 32, 8, 128, 6000, seed=90, ragged=True, min_len=100)
        sq, sk, sv = c0.q.to(dev), c0.k[:, :, lo:hi].to(dev).contiguous(), c0.v[:, :, lo:hi].to(dev).contiguous()
        sl = pkg.sharding.local_seq_lens(c0.seq_lens.to(dev), lo, hi)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            pkg.sharding.decode_kv_sharded_fused(ext, sq, sk, sv, xa, sl, device_epoch=True)   # workspace of this stream
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                gout = pkg.sharding.decode_kv_sharded_fused(ext, sq, sk, sv, xa, sl, device_epoch=True)
            for step in range(3):
                c = inputs.decode_case(2, 32, 8, 128, 6000, seed=91 + step, ragged=True, min_len=100)
                sq.copy_(c.q.to(dev)); sk.copy_(c.k[:, :, lo:hi].to(dev)); sv.copy_(c.v[:, :, lo:hi].to(dev))
                sl.copy_(pkg.sharding.local_seq_lens(c.seq_lens.to(dev), lo, hi))
                graph.replay()
                torch.cuda.synchronize()
                compare.assert_close_attention(gout, attention.sdpa_reference(c.q, c.k, c.v, c.seq_lens))
        torch.cuda.current_stream(dev).wait_stream(side)
        assert xa.check() == 0
        # --- batch sharded by sequence: every rank computes its own sequences, nothing is exchanged
        batch = inputs.config2(seed=62)
        mine = pkg.sharding.partition_batch(batch.seq_lens.tolist(), world)[rank]
        idx = torch.tensor(mine)
        sub = inputs.DecodeCase(batch.q[idx], batch.k[idx], batch.v[idx], batch.seq_lens[idx]).to(dev)
        got = ext.flash_attention_decode(sub.q, sub.k, sub.v, seq_lens=sub.seq_lens)
        torch.cuda.synchronize()
        full = attention.sdpa_reference(batch.q, batch.k, batch.v, batch.seq_lens)
        compare.assert_close_attention(got, full[idx])
        assert ext.flash_decode_status(got) == 0
        q.put((rank, "ok"))
    except Exception as e:  # report instead of hanging the peer in a collective
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sequence_sharding_and_batch_sharding_over_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert results == {r: "ok" for r in range(world)}, results
