"""The allocation-free entry point `l3ci_flash_decode_static` against the regular one.

Some hosts cannot hand this library a scratch buffer: a server that gave the whole card to its own memory
arena at start-up has nothing left to allocate from, and a decode loop that must never enter the driver's
allocator is not allowed to try.  For them the library carries a fixed scratch array in its own device
image.  This file is named so that pytest collects it last: if it fails under `-x`, every other test has
already run.  It must pass alone in a fresh process and after the rest of the suite, because the array is
shared by all calls of the process and keeps what the previous call left in it.
"""
import ctypes as C

import pytest
import torch

from oracle import inputs

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-2, 1e-2   # the attention tolerance used throughout tests/test_gpu_flash_decode.py


def _both(capi, case, device):
    """Output of the regular entry point (caller scratch) and of the static one for the same inputs."""
    dc = case.to(device)
    want = capi.flash_attention_decode(dc.q, dc.k, dc.v, seq_lens=dc.seq_lens)
    out = torch.full_like(dc.q, float("nan"))
    a = capi.flash_decode_args(dc.q, dc.k, dc.v, out=out, seq_lens=dc.seq_lens)   # scratch fields stay NULL / 0
    assert a.scratch is None and a.scratch_bytes == 0
    status = capi.load().l3ci_flash_decode_static(C.byref(a))
    assert status == capi.OK, capi.load().l3ci_last_error()
    torch.cuda.synchronize()
    return out, want


def test_two_calls_in_a_row_match_the_regular_entry_point(capi, device):
    # first call: one long sequence, every head shared by all CTAs (the merge scratch is used heavily);
    # second call: a ragged batch of another shape, which finds the first call's records in the array
    cases = [inputs.decode_case(1, 32, 8, 128, 20000, seed=71),
             inputs.decode_case(5, 32, 8, 64, 3000, seed=72, ragged=True, min_len=1)]
    for case in cases:
        out, want = _both(capi, case, device)
        assert torch.isfinite(out.float()).all()
        err = (out.float() - want.float()).abs()
        assert bool((err <= ATOL + RTOL * want.float().abs()).all()), f"max |diff| {err.max().item():.4g}"
    # and once more with the first shape: the array now holds the second call's leftovers
    out, want = _both(capi, cases[0], device)
    assert bool(((out.float() - want.float()).abs() <= ATOL + RTOL * want.float().abs()).all())


def test_shapes_beyond_the_built_in_area_are_rejected(capi, device):
    lib = capi.load()
    case = inputs.decode_case(1, 16, 1, 128, 64, seed=73).to(device)     # ratio 16 at D=128 needs ~20 MB
    assert lib.l3ci_flash_decode_scratch_bytes(1, 16, 1, 128) > capi.STATIC_SCRATCH_BYTES
    out = torch.empty_like(case.q)
    a = capi.flash_decode_args(case.q, case.k, case.v, out=out)
    assert lib.l3ci_flash_decode_static(C.byref(a)) == capi.ERR_SCRATCH
    msg = lib.l3ci_last_error().decode()
    assert str(capi.STATIC_SCRATCH_BYTES) in msg and "l3ci_flash_decode" in msg
    # the helper raises the same status
    with pytest.raises(capi.L3ciError) as e:
        capi.flash_attention_decode_static(case.q, case.k, case.v)
    assert e.value.status == capi.ERR_SCRATCH
