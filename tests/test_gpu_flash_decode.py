"""Flash-decode kernel through the C ABI against the fp32 oracle (the reference's PyTorch attention path).

Tolerance (stated for this path): |err| <= 2e-2 + 1e-2*|ref| against the fp32 reference, plus a relative-L2
bound of 1e-2 over the whole output so that long sequences (outputs ~1e-2) are not trivially accepted."""
import ctypes as C

import pytest
import torch

from oracle import attention, compare, inputs

pytestmark = pytest.mark.gpu
ATOL, RTOL, REL_L2 = 2e-2, 1e-2, 1e-2


def _run(capi, case, device, scratch=None, max_ctas=0, scale=0.0):
    dc = case.to(device)
    out = capi.flash_attention_decode(dc.q, dc.k, dc.v, seq_lens=dc.seq_lens, scratch=scratch, max_ctas=max_ctas,
                                      scale=scale)
    torch.cuda.synchronize()
    assert out.shape == dc.q.shape and out.stride() == dc.q.stride() and out.dtype == torch.bfloat16
    return out


def _check(capi, case, device, **kw):
    out = _run(capi, case, device, **kw)
    want = attention.sdpa_reference(case.q, case.k, case.v, case.seq_lens, scale=kw.get("scale") or None)
    compare.assert_close_attention(out, want, ATOL, RTOL, REL_L2)
    return out


# ---- the benchmark configurations ----------------------------------------------------------------

def test_config1_llama32_1b_decode_step(capi, device, golden):
    out = _check(capi, inputs.config1(), device)
    # and against what the reference's own bf16 SDPA call produced for these inputs
    compare.assert_close_attention(out, golden["sdpa_c1_bf16"].float(), ATOL, RTOL, 2e-2)


def test_config2_ragged_batch_ignores_padding(capi, device):
    case = inputs.config2()
    assert int(case.seq_lens.min()) >= 1024 and int(case.seq_lens.max()) <= 2048
    _check(capi, case, device)


def test_config3_long_context(capi, device):
    case = inputs.config3()
    out = _check(capi, case, device)
    assert out.float().abs().max().item() > 1e-3  # not the all-zeros answer the absolute bound would admit


# ---- shapes: head sizes, group ratios, lengths around the tile sizes -------------------------------

# max_ctas 0 lets the library choose between its two kernels; a positive value asks for the persistent grid,
# -1 for the kernel that deals units statically to warps, CTAs or clusters (with its own choice of split).
KERNELS = pytest.mark.parametrize("max_ctas", [0, 148, -1], ids=["auto", "persistent", "static"])
HEADS = [(4, 4), (4, 2), (6, 2), (32, 8), (8, 1), (12, 1), (16, 1), (24, 3), (32, 32), (10, 5)]
LENGTHS = [1, 15, 16, 17, 31, 32, 33, 63, 64, 65, 100, 255, 300, 1000]


@KERNELS
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("Hq,Hkv", HEADS)
def test_head_configurations(capi, device, D, Hq, Hkv, max_ctas):
    for i, S in enumerate([1, 33, 300]):
        _check(capi, inputs.decode_case(2, Hq, Hkv, D, S, seed=100 + i), device, max_ctas=max_ctas)


@KERNELS
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("S", LENGTHS)
def test_lengths_around_tile_boundaries(capi, device, D, S, max_ctas):
    _check(capi, inputs.decode_case(3, 8, 2, D, S, seed=S), device, max_ctas=max_ctas)


# -(16 * C + W): C CTAs (a cluster) per unit, W of a CTA's 8 warps per unit
SPLITS = {"w1": -17, "w2": -18, "w4": -20, "w8": -24, "c2": -40, "c4": -72, "c8": -136}


@pytest.mark.parametrize("split", list(SPLITS))
@pytest.mark.parametrize("D", [64, 128])
def test_every_static_split_agrees_with_the_oracle(capi, device, D, split):
    shapes = [(1, 32, 8, 700, False), (3, 9, 3, 333, True), (5, 8, 1, 40, True), (2, 16, 2, 2100, True), (11, 14, 7, 90, False)]
    for i, (B, Hq, Hkv, S, ragged) in enumerate(shapes):   # 9, 5 and 77 units: partly filled CTAs for W < 8
        case = inputs.decode_case(B, Hq, Hkv, D, S, seed=60 + i, ragged=ragged, min_len=0)
        a = _check(capi, case, device, max_ctas=SPLITS[split]).float()
        b = _run(capi, case, device, max_ctas=148).float()
        assert (a - b).abs().max().item() <= 2e-2


def test_kernel_choice_names_the_split_the_call_takes(capi, device):
    lib = capi.load()
    with torch.cuda.device(device):
        # the reference's own example and a batched step of 2048-token caches: static deal, one CTA per unit
        assert lib.l3ci_flash_decode_kernel_choice(1, 32, 8, 64, 256, 0) == 16 + 8
        assert lib.l3ci_flash_decode_kernel_choice(16, 32, 8, 128, 2048, 1) == 16 + 8
        # few long units: clusters; longer still or possibly lopsided ones, or 16 query heads per KV head: persistent grid
        assert lib.l3ci_flash_decode_kernel_choice(1, 32, 8, 128, 16384, 0) == 16 * 8 + 8
        assert lib.l3ci_flash_decode_kernel_choice(1, 32, 8, 128, 131072, 0) == 16 * 8 + 8
        assert lib.l3ci_flash_decode_kernel_choice(1, 32, 8, 128, 262144, 0) == 0
        assert lib.l3ci_flash_decode_kernel_choice(16, 32, 8, 128, 8192, 1) == 0
        assert lib.l3ci_flash_decode_kernel_choice(2, 32, 2, 128, 512, 0) == 0
        # many short units share CTAs
        assert lib.l3ci_flash_decode_kernel_choice(64, 32, 8, 64, 256, 0) == 16 + 2
    # the split it names, asked for explicitly, gives the same bits as the default call
    case = inputs.decode_case(1, 32, 8, 128, 16384, seed=5)
    a = _run(capi, case, device)
    b = _run(capi, case, device, max_ctas=-(16 * 8 + 8))
    assert torch.equal(a, b)


def test_static_kernel_refuses_a_malformed_split(capi, device):
    case = inputs.decode_case(1, 8, 2, 64, 50, seed=3).to(device)
    for code in (-(16 * 3 + 8), -(16 * 2 + 4), -(16 * 16 + 8), -(16 + 3)):
        with pytest.raises(capi.L3ciError, match="split code"):
            capi.flash_attention_decode(case.q, case.k, case.v, max_ctas=code)


def test_more_than_eight_query_heads_per_kv_head_take_the_persistent_kernel(capi, device):
    _check(capi, inputs.decode_case(2, 32, 2, 64, 100, seed=4), device, max_ctas=-1)


@pytest.mark.parametrize("name,shape", [("d128_r4_s300", (2, 8, 2, 128, 300, 7)), ("d64_r1_s65", (2, 4, 4, 64, 65, 8)),
                                        ("d128_r8_s1000", (1, 8, 1, 128, 1000, 9))])
def test_against_reference_produced_vectors(capi, device, golden, name, shape):
    B, Hq, Hkv, D, S, seed = shape
    out = _run(capi, inputs.decode_case(B, Hq, Hkv, D, S, seed=seed), device)
    compare.assert_close_attention(out, golden[f"sdpa_{name}_bf16"].float(), ATOL, RTOL, 2e-2)


def test_uniform01_inputs_as_the_reference_benchmark_draws_them(capi, device, golden):
    # benchmark_kernel.py:161-163 uses torch.rand inputs
    out = _check(capi, inputs.decode_case(1, 6, 2, 128, 130, seed=10, dist="uniform"), device)
    compare.assert_close_attention(out, golden["sdpa_d128_r3_s130_uniform01_bf16"].float(), ATOL, RTOL, 2e-2)


# ---- ragged batches ---------------------------------------------------------------------------------

@KERNELS
@pytest.mark.parametrize("D", [64, 128])
def test_ragged_lengths_including_empty_and_full(capi, device, D, max_ctas):
    case = inputs.decode_case(9, 12, 3, D, 200, seed=11, ragged=True)
    case.seq_lens[:] = torch.tensor([0, 1, 200, 16, 17, 199, 32, 33, 150], dtype=torch.int32)
    out = _check(capi, case, device, max_ctas=max_ctas)
    assert out[0].abs().max().item() == 0  # a sequence without cached tokens yields zeros


def test_lengths_are_clamped_to_the_cache(capi, device):
    case = inputs.decode_case(3, 8, 2, 128, 70, seed=12, ragged=True)
    case.seq_lens[:] = torch.tensor([500, -4, 70], dtype=torch.int32)
    out = _run(capi, case, device)
    clamped = inputs.DecodeCase(case.q, case.k, case.v, torch.tensor([70, 0, 70], dtype=torch.int32))
    compare.assert_close_attention(out, attention.sdpa_reference(clamped.q, clamped.k, clamped.v, clamped.seq_lens), ATOL, RTOL, REL_L2)


def test_many_short_sequences(capi, device):
    case = inputs.decode_case(300, 8, 8, 64, 40, seed=13, ragged=True)
    _check(capi, case, device)


# ---- the split structure: every grid size must give the same answer ---------------------------------

@pytest.mark.parametrize("max_ctas", [1, 2, 3, 5, 16, 147, 0])
def test_any_grid_size_gives_the_same_result(capi, device, max_ctas):
    for D, S in ((128, 1000), (64, 700)):
        case = inputs.decode_case(2, 16, 8, D, S, seed=21, ragged=True, min_len=S // 2)
        _check(capi, case, device, max_ctas=max_ctas)


def test_scratch_is_reusable_without_clearing(capi, device):
    # one scratch buffer, zeroed once, serves calls of different batch sizes, head counts and head sizes
    scratch = capi.DecodeScratch(4, 16, 2, 128, device)   # ratio 8 at D=128: the largest records used below
    shapes = [(1, 32, 8, 128, 3000), (4, 32, 8, 128, 40), (3, 16, 2, 128, 2000), (2, 8, 8, 64, 5000),
              (4, 32, 8, 64, 700), (1, 32, 8, 128, 3000)]
    for i, (B, Hq, Hkv, D, S) in enumerate(shapes):
        assert capi.load().l3ci_flash_decode_scratch_bytes(B, Hq, Hkv, D) <= scratch.bytes
        _check(capi, inputs.decode_case(B, Hq, Hkv, D, S, seed=30 + i, ragged=i % 2 == 1, min_len=S // 2), device,
               scratch=scratch)
    assert scratch.poll() == capi.OK
    counters = scratch.buf[256:256 + 65536 * 4].view(torch.int32)
    assert int(counters.abs().sum()) == 0  # arrival counters are left at zero


def test_custom_scale(capi, device):
    _check(capi, inputs.decode_case(2, 8, 2, 128, 100, seed=14), device, scale=0.05)


# ---- memory layouts -----------------------------------------------------------------------------------

def test_kv_cache_slice_layout_of_the_model(capi, device):
    # cache [maxB, maxLen, Hkv, D] sliced to [:B, :S] and transposed (model.py:89-90,107-111)
    max_b, max_len, Hkv, D, B, S, Hq = 5, 300, 8, 64, 3, 130, 32
    g = torch.Generator().manual_seed(15)
    ck = torch.randn(max_b, max_len, Hkv, D, generator=g).bfloat16()
    cv = torch.randn(max_b, max_len, Hkv, D, generator=g).bfloat16()
    q = torch.randn(B, 1, Hq, D, generator=g).bfloat16().transpose(1, 2)
    case = inputs.DecodeCase(q, ck[:B, :S].transpose(1, 2), cv[:B, :S].transpose(1, 2), None)
    dk, dv = ck.to(device)[:B, :S].transpose(1, 2), cv.to(device)[:B, :S].transpose(1, 2)
    out = capi.flash_attention_decode(q.to(device), dk, dv)
    torch.cuda.synchronize()
    compare.assert_close_attention(out, attention.sdpa_reference(case.q, case.k, case.v), ATOL, RTOL, REL_L2)


def test_contiguous_bhsd_layout_and_contiguous_query(capi, device):
    case = inputs.decode_case(2, 8, 4, 128, 77, seed=16)
    dq = case.q.contiguous().to(device)
    dk, dv = case.k.contiguous().to(device), case.v.contiguous().to(device)
    assert dk.stride() == (4 * 77 * 128, 77 * 128, 128, 1)
    out = capi.flash_attention_decode(dq, dk, dv)
    torch.cuda.synchronize()
    compare.assert_close_attention(out, attention.sdpa_reference(case.q, case.k, case.v), ATOL, RTOL, REL_L2)


# ---- shard results and their merge ----------------------------------------------------------------------

@pytest.mark.parametrize("D", [64, 128])
def test_partial_outputs_and_lse(capi, device, D):
    case = inputs.decode_case(3, 12, 4, D, 500, seed=17, ragged=True)
    case.seq_lens[0] = 0
    dc = case.to(device)
    o, lse = capi.flash_attention_decode_partial(dc.q, dc.k, dc.v, seq_lens=dc.seq_lens)
    torch.cuda.synchronize()
    want_o, want_lse = attention.attention_float64(case.q, case.k, case.v, case.seq_lens)
    assert (o.cpu().double() - torch.from_numpy(want_o[:, :, 0])).abs().max().item() < 2e-2
    got_lse = lse.cpu().double()
    want = torch.from_numpy(want_lse)
    finite = torch.isfinite(want)
    assert torch.equal(torch.isinf(got_lse) & (got_lse < 0), ~finite)
    assert (got_lse[finite] - want[finite]).abs().max().item() < 2e-3


@pytest.mark.parametrize("shards", [1, 2, 4, 8])
def test_sequence_shards_merge_to_full_attention(capi, pkg, device, shards):
    case = inputs.decode_case(2, 32, 8, 128, 1500, seed=18, ragged=True, min_len=100)
    dc = case.to(device)
    os_, ls_ = [], []
    for lo, hi in pkg.sharding.kv_shard_bounds(1500, shards):
        lens = pkg.sharding.local_seq_lens(dc.seq_lens, lo, hi)
        if hi > lo:
            o, l = capi.flash_attention_decode_partial(dc.q, dc.k[:, :, lo:hi], dc.v[:, :, lo:hi], seq_lens=lens)
        else:
            o = torch.zeros(2, 32, 128, device=device)
            l = torch.full((2, 32), float("-inf"), device=device)
        os_.append(o)
        ls_.append(l)
    out = capi.lse_merge(torch.stack(os_), torch.stack(ls_))
    torch.cuda.synchronize()
    assert out.shape == dc.q.shape and out.stride() == dc.q.stride()
    compare.assert_close_attention(out, attention.sdpa_reference(case.q, case.k, case.v, case.seq_lens), ATOL, RTOL, REL_L2)
    merged_ref = attention.lse_merge_reference(torch.stack(os_), torch.stack(ls_))
    assert (out.float().cpu()[:, :, 0] - merged_ref).abs().max().item() < 1e-2


# ---- errors --------------------------------------------------------------------------------------------

def test_error_statuses(capi, device):
    lib = capi.load()
    case = inputs.decode_case(1, 8, 2, 128, 64, seed=19).to(device)
    out = torch.empty_like(case.q)
    scratch = capi.DecodeScratch(1, 8, 2, 128, device)
    a = capi.flash_decode_args(case.q, case.k, case.v, out=out, scratch=scratch, max_ctas=148)
    a.scratch_bytes = 128     # the persistent kernel needs its scratch ...
    assert lib.l3ci_flash_decode(C.byref(a)) == capi.ERR_SCRATCH
    a = capi.flash_decode_args(case.q, case.k, case.v, out=out, max_ctas=-1)
    assert lib.l3ci_flash_decode(C.byref(a)) == capi.OK   # ... the static-deal kernel none at all
    a = capi.flash_decode_args(case.q, case.k[..., 8:], case.v, out=out, scratch=scratch)
    a.D = 128
    a.k = case.k.data_ptr() + 2
    assert lib.l3ci_flash_decode(C.byref(a)) == capi.ERR_ALIGNMENT
    a = capi.flash_decode_args(case.q, case.k, case.v, out=out, scratch=scratch)
    a.k_st = 129 * 2 + 1
    assert lib.l3ci_flash_decode(C.byref(a)) == capi.ERR_ALIGNMENT
    a = capi.flash_decode_args(case.q, case.k, case.v, scratch=scratch)  # no output at all
    assert lib.l3ci_flash_decode(C.byref(a)) == capi.ERR_INVALID
    torch.cuda.synchronize()
    assert scratch.poll() == capi.OK


def test_zero_length_cache(capi, device):
    q = torch.randn(2, 4, 1, 64).bfloat16().to(device)
    k = torch.empty(2, 2, 0, 64, dtype=torch.bfloat16, device=device)
    out = capi.flash_attention_decode(q, k, k)
    torch.cuda.synchronize()
    assert out.abs().max().item() == 0
