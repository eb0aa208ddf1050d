"""Bounded device-side waits that run out: the kernel gives up in order, reports L3CI_ERR_DEVICE_WAIT and the
context stays usable.

The failure is made on the host: a peer that never posts its flags, an arrival counter that can never reach its
target.  Nothing faults, traps or hangs; the waits are given a limit of a few milliseconds through
`l3ci_set_device_wait_limit_ns` (their defaults are 1 s and 2 s).  The wait on a bulk tensor copy's mbarrier is
not covered: making it run out would need a copy that never lands.
"""
import pytest
import torch

from oracle import attention, compare, inputs

pytestmark = pytest.mark.gpu
LIMIT_NS = 20_000_000  # 20 ms


def test_exchange_gives_up_when_a_peer_never_posts(capi, device):
    # "rank 0 of 2" on one GPU: both buffer pointers are local memory, and nothing ever plays rank 1, so the
    # flags [parity][1][row] of the local buffer keep their zeros
    B, Hq, D, ranks = 2, 8, 64, 2
    lib = capi.load()
    nbytes = lib.l3ci_lse_exchange_bytes(ranks, B, Hq, D)
    mine = torch.zeros(nbytes // 4, dtype=torch.float32, device=device)
    peer = torch.zeros_like(mine)
    bufs = torch.tensor([mine.data_ptr(), peer.data_ptr()], dtype=torch.int64, device=device)
    rows = B * Hq
    slot_floats = rows * D + ((rows + 3) & ~3)
    epoch = 1
    own = ((epoch & 1) * ranks + 0) * slot_floats            # rank 0's own slot of parity 1
    mine[own: own + rows * D] = torch.randn(rows * D, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    sentinel = 12352.0  # representable in bf16
    out = torch.full((B, 1, Hq, D), sentinel, dtype=torch.bfloat16, device=device).transpose(1, 2)
    with capi.device_wait_limit(LIMIT_NS):
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        capi.lse_exchange_merge(bufs, 0, ranks, epoch, out, B, Hq, D, status=status)
        t1.record()
        torch.cuda.synchronize()            # the kernel returns by itself
    assert 0.5 * LIMIT_NS * 1e-6 <= t0.elapsed_time(t1) < 1000.0
    assert int(status.item()) == capi.ERR_DEVICE_WAIT
    assert bool((out.float() == sentinel).all()), "rows whose peers never arrived must stay unwritten"
    # the push itself happened: the "peer" holds rank 0's rows and flags
    assert torch.equal(peer[own: own + rows * D], mine[own: own + rows * D])
    # and the context is intact: a complete exchange (both ranks' rows and flags in place) merges
    epoch = 2
    status.zero_()
    par = (epoch & 1) * ranks
    o = torch.randn(ranks, rows, D, device=device)
    lse = torch.randn(ranks, rows, device=device)
    flags_base = 2 * ranks * slot_floats
    for r in range(ranks):
        base = (par + r) * slot_floats
        mine[base: base + rows * D] = o[r].flatten()
        mine[base + rows * D: base + rows * D + rows] = lse[r]
    mine.view(torch.int32)[flags_base + (par + 1) * rows: flags_base + (par + 2) * rows] = epoch   # rank 1 "posted"
    capi.lse_exchange_merge(bufs, 0, ranks, epoch, out, B, Hq, D, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == capi.OK
    w = torch.softmax(lse, dim=0).unsqueeze(-1)
    want = (w * o).sum(0).view(B, Hq, 1, D)
    assert torch.allclose(out.float(), want, atol=2e-2, rtol=1e-2)


def test_arrival_counter_wait_runs_out_and_poll_reports_it(capi, device):
    # one long sequence through the persistent kernel: every (sequence, kv head) unit is shared by many CTAs, which
    # wait for each other's records on the unit's arrival counter.  Counters preset far below zero never reach
    # their target.
    case = inputs.decode_case(1, 32, 8, 128, 20000, seed=81)
    dc = case.to(device)
    scratch = capi.DecodeScratch(1, 32, 8, 128, device)
    header = 256
    scratch.buf[header: header + 4 * 8].view(torch.int32).fill_(-100000)
    with capi.device_wait_limit(LIMIT_NS):
        capi.flash_attention_decode(dc.q, dc.k, dc.v, scratch=scratch, max_ctas=148)
        torch.cuda.synchronize()
    assert scratch.poll() == capi.ERR_DEVICE_WAIT        # reported once ...
    assert "wait" in capi.load().l3ci_last_error().decode()
    assert scratch.poll() == capi.OK                     # ... and cleared, counters included
    assert int(scratch.buf[header: header + 4 * 8].view(torch.int32).abs().sum()) == 0
    out = capi.flash_attention_decode(dc.q, dc.k, dc.v, scratch=scratch, max_ctas=148)
    torch.cuda.synchronize()
    assert scratch.poll() == capi.OK
    compare.assert_close_attention(out, attention.sdpa_reference(case.q, case.k, case.v))
