"""The allocation-free entry point `l3ci_flash_decode_static`.

Some hosts cannot hand this library a scratch buffer: a server that gave the whole card to its own memory
arena at start-up has nothing left to allocate from, and a decode loop that must never enter the driver's
allocator is not allowed to try.  For them the library carries a fixed scratch array in its own device
image.  This file is named so that pytest collects it last: if it fails under `-x`, every other test has
already run.  It must pass alone in a fresh process and after the rest of the suite, because the array is
shared by all calls of the process and keeps what the previous call left in it.

The array is only touched by the persistent kernel (the static-deal kernel merges in shared memory), so the
cases below ask for the persistent kernel with a positive `max_ctas`; results are checked against the regular
entry point (same kernel on caller scratch) and against the CPU oracle.
"""
import ctypes as C

import pytest
import torch

from oracle import attention, compare, inputs

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-2, 1e-2   # the attention tolerance used throughout tests/test_gpu_flash_decode.py


def _both(capi, case, device, max_ctas):
    """Output of the regular entry point (caller scratch) and of the static one for the same inputs, both through
    the persistent kernel capped at `max_ctas` CTAs."""
    dc = case.to(device)
    want = capi.flash_attention_decode(dc.q, dc.k, dc.v, seq_lens=dc.seq_lens, max_ctas=max_ctas)
    out = torch.full_like(dc.q, float("nan"))
    a = capi.flash_decode_args(dc.q, dc.k, dc.v, out=out, seq_lens=dc.seq_lens, max_ctas=max_ctas)   # scratch fields stay NULL / 0
    assert a.scratch is None and a.scratch_bytes == 0
    free_before = torch.cuda.mem_get_info(device)[0]
    status = capi.load().l3ci_flash_decode_static(C.byref(a))
    assert status == capi.OK, capi.load().l3ci_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(device)[0] >= free_before, "the call took device memory"
    return out, want


def _check(out, want, case):
    assert torch.isfinite(out.float()).all()
    err = (out.float() - want.float()).abs()
    assert bool((err <= ATOL + RTOL * want.float().abs()).all()), f"max |diff| {err.max().item():.4g}"
    # and against the CPU oracle, with the relative-L2 bound that an all-zero output cannot pass
    compare.assert_close_attention(out, attention.sdpa_reference(case.q, case.k, case.v, case.seq_lens))


@pytest.mark.parametrize("max_ctas", [1 << 20, 37])
def test_two_calls_in_a_row_match_the_regular_entry_point(capi, device, max_ctas):
    # first call: one long sequence, every head shared by all CTAs of the grid (merge records and arrival counters
    # of the built-in array are used heavily); second call: a ragged batch of another shape, which finds the first
    # call's records in the array.  37 CTAs cut the units at other places than the full grid does.
    cases = [inputs.decode_case(1, 32, 8, 128, 20000, seed=71),
             inputs.decode_case(5, 32, 8, 64, 3000, seed=72, ragged=True, min_len=1)]
    for case in cases:
        out, want = _both(capi, case, device, max_ctas)
        _check(out, want, case)
    # and once more with the first shape: the array now holds the second call's leftovers
    out, want = _both(capi, cases[0], device, max_ctas)
    _check(out, want, cases[0])


def test_library_choice_that_needs_no_scratch_is_not_limited_by_the_array(capi, device):
    # 8 query heads per KV head at head size 128 (the Llama-3 70B layout) would need 19 MB of records in the
    # persistent kernel; a short cache goes to the static-deal kernel, which needs none, and is accepted
    lib = capi.load()
    assert lib.l3ci_flash_decode_scratch_bytes(2, 64, 8, 128) > capi.STATIC_SCRATCH_BYTES
    assert lib.l3ci_flash_decode_kernel_choice(2, 64, 8, 128, 700, 0) != 0
    case = inputs.decode_case(2, 64, 8, 128, 700, seed=74)
    dc = case.to(device)
    out = capi.flash_attention_decode_static(dc.q, dc.k, dc.v)
    torch.cuda.synchronize()
    compare.assert_close_attention(out, attention.sdpa_reference(case.q, case.k, case.v))
    # the same shape through the persistent kernel does need the records, and is refused
    with pytest.raises(capi.L3ciError) as e:
        capi.flash_attention_decode_static(dc.q, dc.k, dc.v, max_ctas=148)
    assert e.value.status == capi.ERR_SCRATCH


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
