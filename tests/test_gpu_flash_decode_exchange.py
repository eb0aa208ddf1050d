"""The sequence-sharded decode call with the cross-GPU exchange in the kernel's tail (`l3ci_flash_decode_exchange`)
on ONE GPU.  Kernels that wait for one another never run as separate launches on one GPU, so the peer is played by
the host: its words are put into the exchange buffer before the launch (the kernel then finds them at once), or
left out (the kernel's bounded wait runs out).  tests/test_gpu_multi.py runs real ranks on two GPUs.
"""
import pytest
import torch

from oracle import attention, compare, inputs

pytestmark = pytest.mark.gpu


def _buffers(capi, ranks, B, Hq, D, device):
    nbytes = capi.load().l3ci_flash_decode_exchange_bytes(ranks, B, Hq, D)
    bufs = [torch.zeros(nbytes // 8, dtype=torch.int64, device=device) for _ in range(ranks)]
    ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=device)
    return bufs, ptrs


def _post(buf, ranks, src, epoch, o, lse):
    """What rank `src` sends in call `epoch`: words {call number | value bits} at [parity][src][row * (D + 1) + col]."""
    rows, D = o.shape[0] * o.shape[1], o.shape[2]
    vals = torch.cat([o.reshape(rows, D), lse.reshape(rows, 1)], dim=1).contiguous().float()
    words = vals.view(torch.int32).to(torch.int64) & 0xFFFFFFFF | (epoch << 32)
    base = ((epoch & 1) * ranks + src) * rows * (D + 1)
    buf[base: base + rows * (D + 1)] = words.flatten()


@pytest.mark.parametrize("shape,max_ctas", [((1, 32, 8, 128, 9000), 0), ((1, 32, 8, 128, 9000), -(16 * 8 + 8)),
                                             ((3, 16, 4, 64, 700), -1), ((2, 8, 8, 64, 300), -(16 + 2)),
                                             ((40, 32, 8, 64, 200), 0)])
def test_two_ranks_with_the_peer_played_by_the_host(capi, device, shape, max_ctas):
    B, Hq, Hkv, D, S = shape
    case = inputs.decode_case(B, Hq, Hkv, D, S, seed=101, ragged=B > 1, min_len=1)
    dc = case.to(device)
    half = (S // 2 // 64) * 64
    lens = dc.seq_lens
    l0 = lens.clamp(max=half) if lens is not None else None
    l1 = (lens - half).clamp(min=0) if lens is not None else None
    bufs, ptrs = _buffers(capi, 2, B, Hq, D, device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    want = attention.sdpa_reference(case.q, case.k, case.v, case.seq_lens)
    for epoch in (1, 2, 3):       # both parities, and a slot used twice
        # "rank 1" holds the second half of the cache: its result goes into rank 0's buffer before rank 0 starts
        o1, lse1 = capi.flash_attention_decode_partial(dc.q, dc.k[:, :, half:], dc.v[:, :, half:], seq_lens=l1)
        _post(bufs[0], 2, 1, epoch, o1, lse1)
        torch.cuda.synchronize()
        out = capi.flash_decode_exchange(dc.q, dc.k[:, :, :half], dc.v[:, :, :half], ptrs, 0, 2, epoch, seq_lens=l0,
                                         status=status, max_ctas=max_ctas)
        torch.cuda.synchronize()
        assert int(status.item()) == capi.OK
        compare.assert_close_attention(out, want)
        # rank 0 sent its own result to "rank 1": the words of source 0 in the peer's buffer are this call's
        rows = B * Hq
        base = ((epoch & 1) * 2 + 0) * rows * (D + 1)
        sent = bufs[1][base: base + rows * (D + 1)]
        assert bool(((sent >> 32) == epoch).all())
        o0, lse0 = capi.flash_attention_decode_partial(dc.q, dc.k[:, :, :half], dc.v[:, :, :half], seq_lens=l0)
        got0 = (sent & 0xFFFFFFFF).to(torch.int32).view(torch.float32).view(rows, D + 1)
        # (the partial call may deal the tiles to warps differently: probabilities are rounded to bf16 per tile)
        assert torch.allclose(got0[:, :D], o0.view(rows, D), atol=5e-3, rtol=1e-2)
        assert torch.allclose(got0[:, D], lse0.view(rows), atol=1e-3, rtol=1e-4)


@pytest.mark.parametrize("ranks,me", [(8, 5), (4, 3), (3, 0)])
def test_many_ranks_with_the_peers_played_by_the_host(capi, device, ranks, me):
    # the widest exchange (8 ranks) and a rank that is not the first: every peer's words are in this rank's buffer
    # before it starts, and its own words must arrive in every peer's buffer
    B, Hq, Hkv, D, S = 1, 32, 8, 128, 16384
    case = inputs.decode_case(B, Hq, Hkv, D, S, seed=111)
    dc = case.to(device)
    step = (S // ranks // 64) * 64
    bounds = [(r * step, S if r == ranks - 1 else (r + 1) * step) for r in range(ranks)]
    bufs, ptrs = _buffers(capi, ranks, B, Hq, D, device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    want = attention.sdpa_reference(case.q, case.k, case.v)
    rows = B * Hq
    for epoch in (1, 2):
        for r, (lo, hi) in enumerate(bounds):
            if r != me:
                o, lse = capi.flash_attention_decode_partial(dc.q, dc.k[:, :, lo:hi], dc.v[:, :, lo:hi])
                _post(bufs[me], ranks, r, epoch, o, lse)
        torch.cuda.synchronize()
        lo, hi = bounds[me]
        out = capi.flash_decode_exchange(dc.q, dc.k[:, :, lo:hi], dc.v[:, :, lo:hi], ptrs, me, ranks, epoch, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == capi.OK
        compare.assert_close_attention(out, want)
        base = ((epoch & 1) * ranks + me) * rows * (D + 1)
        for r in range(ranks):
            if r != me:
                assert bool(((bufs[r][base: base + rows * (D + 1)] >> 32) == epoch).all()), r


def test_one_rank_and_the_call_number_kept_in_the_buffer(capi, device):
    # a "world" of one GPU: nothing to wait for; with epoch 0 the kernel numbers its calls itself
    case = inputs.decode_case(2, 32, 8, 128, 5000, seed=102)
    dc = case.to(device)
    bufs, ptrs = _buffers(capi, 1, 2, 32, 128, device)
    want = attention.sdpa_reference(case.q, case.k, case.v)
    words = 2 * 32 * 129
    for call in (1, 2, 3):
        out = capi.flash_decode_exchange(dc.q, dc.k, dc.v, ptrs, 0, 1, 0)
        torch.cuda.synchronize()
        compare.assert_close_attention(out, want)
        ctrl = bufs[0][2 * words: 2 * words + 2].view(torch.int32)
        assert int(ctrl[0]) == call and int(ctrl[2]) == 0     # call number advanced, finished-CTA count back to zero


def test_wait_runs_out_when_the_peer_never_sends(capi, device):
    case = inputs.decode_case(1, 32, 8, 128, 4096, seed=103)
    dc = case.to(device)
    bufs, ptrs = _buffers(capi, 2, 1, 32, 128, device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    out = torch.full_like(dc.q, 12352.0)
    with capi.device_wait_limit(20_000_000):
        capi.flash_decode_exchange(dc.q, dc.k, dc.v, ptrs, 0, 2, 1, out=out, status=status)
        torch.cuda.synchronize()       # the kernel returns by itself
    assert int(status.item()) == capi.ERR_DEVICE_WAIT
    assert bool((out.float() == 12352.0).all()), "elements whose peer values never arrived must stay unwritten"
    # the context is intact, and the next call on the same buffers works once the peer's words are there
    o1, lse1 = capi.flash_attention_decode_partial(dc.q, dc.k[:, :, :64], dc.v[:, :, :64])
    _post(bufs[0], 2, 1, 2, o1, lse1)
    status.zero_()
    out = capi.flash_decode_exchange(dc.q, dc.k[:, :, 64:], dc.v[:, :, 64:], ptrs, 0, 2, 2, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == capi.OK
    compare.assert_close_attention(out, attention.sdpa_reference(case.q, case.k, case.v))


def test_sizes_without_a_fused_exchange_are_refused(capi, device):
    case = inputs.decode_case(1, 32, 2, 64, 256, seed=104).to(device)      # 16 query heads per KV head
    bufs, ptrs = _buffers(capi, 2, 1, 32, 64, device)
    with pytest.raises(capi.L3ciError) as e:
        capi.flash_decode_exchange(case.q, case.k, case.v, ptrs, 0, 2, 1)
    assert e.value.status == capi.ERR_UNSUPPORTED
    case = inputs.decode_case(1, 32, 8, 64, 256, seed=105).to(device)
    with pytest.raises(capi.L3ciError) as e:
        capi.flash_decode_exchange(case.q, case.k, case.v, ptrs, 0, 2, 1, max_ctas=148)   # the persistent kernel
    assert e.value.status == capi.ERR_UNSUPPORTED
