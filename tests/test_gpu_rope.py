"""Rotary-embedding kernels through the C ABI against the oracle, which is bit-equal to the reference's compiled
kernel (tests/test_oracle_reference_cuda.py).  The stated tolerance is 1 bf16 ulp; the kernel evaluates the same
fp32 expression with the same roundings, so the results are expected identical."""
import pytest
import torch

from oracle import compare, inputs
from oracle.rope import freqs_cis_reference, rot_embed_reference

pytestmark = pytest.mark.gpu
MAX_ULP = 1


def _table(D, S, start=0):
    return freqs_cis_reference(D, start + S, **inputs.ROPE_CONFIG4)[start:start + S].contiguous()


def test_config4_q_and_k_views(capi, device):
    _, _, _, qkv = inputs.config4()
    B, S, _ = qkv.shape
    Hq, Hkv, D = 32, 8, 64
    freq = _table(D, S)
    qkv_d, freq_d = qkv.to(device), freq.to(device)
    q, k, _ = qkv_d.split([Hq * D, Hkv * D, Hkv * D], dim=-1)   # strided views, as model.py:96-97
    for view, H in ((q, Hq), (k, Hkv)):
        x = view.view(B, S, H, D)
        got = capi.rot_embed(x, freq_d)
        torch.cuda.synchronize()
        want = rot_embed_reference(x, freq)
        assert got.is_contiguous() and got.shape == x.shape
        assert compare.max_bf16_ulp(got, want) <= MAX_ULP
        assert torch.equal(got.cpu(), want), "expected bit-identical results"


@pytest.mark.parametrize("B,S,H,D", [(1, 1, 1, 64), (2, 5, 3, 128), (64, 1, 32, 64), (1, 33, 8, 128), (3, 7, 2, 16), (2, 3, 5, 8)])
def test_shapes_dense_and_decode_offsets(capi, device, B, S, H, D):
    g = torch.Generator().manual_seed(B * 1000 + S * 10 + H)
    x = torch.randn(B, S, H, D, generator=g).bfloat16()
    freq = _table(D, S, start=777)
    got = capi.rot_embed(x.to(device), freq.to(device))
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), rot_embed_reference(x, freq))


def test_pair_fallback_for_rows_on_4_bytes(capi, device):
    # head size 6: rows start on 12-byte multiples, so the 16-byte path is not usable
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 4, 3, 6, generator=g).bfloat16()
    freq = torch.randn(4, 6, generator=g)
    got = capi.rot_embed(x.to(device), freq.to(device))
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), rot_embed_reference(x, freq))
    # a view that starts 4 bytes into a row
    y = torch.randn(1, 2, 2, 66, generator=g).bfloat16().to(device)[..., 2:]
    f2 = torch.randn(2, 64, generator=g)
    got = capi.rot_embed(y, f2.to(device))
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), rot_embed_reference(y, f2))


@pytest.mark.parametrize("B,T,start", [(2, 2048, 0), (64, 1, 300), (3, 5, 11)])
def test_fused_rope_kv_cache_write(capi, device, B, T, start):
    Hq, Hkv, D, max_b, max_len = 32, 8, 64, max(B, 4) + 1, start + T + 3
    g = torch.Generator().manual_seed(B + T + start)
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * D, generator=g).bfloat16()
    freq = _table(D, T, start=start)
    cache_k = torch.full((max_b, max_len, Hkv, D), 3.0, dtype=torch.bfloat16, device=device)
    cache_v = torch.full((max_b, max_len, Hkv, D), 5.0, dtype=torch.bfloat16, device=device)
    q_rot = capi.rot_embed_kv_cache(qkv.to(device), freq.to(device), cache_k, cache_v, start, Hq, Hkv)
    torch.cuda.synchronize()
    q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    assert torch.equal(q_rot.cpu(), rot_embed_reference(q.reshape(B, T, Hq, D), freq))
    assert torch.equal(cache_k[:B, start:start + T].cpu(), rot_embed_reference(k.reshape(B, T, Hkv, D), freq))
    assert torch.equal(cache_v[:B, start:start + T].cpu(), v.reshape(B, T, Hkv, D))
    # everything outside the written window is untouched
    ck, cv = cache_k.clone(), cache_v.clone()
    ck[:B, start:start + T] = 3.0
    cv[:B, start:start + T] = 5.0
    assert (ck == 3.0).all() and (cv == 5.0).all()


def test_fused_write_with_per_sequence_positions(capi, device):
    # every sequence at its own position; one is past the end of the cache and must be skipped untouched
    B, T, Hq, Hkv, D, max_len = 5, 1, 32, 8, 64, 50
    g = torch.Generator().manual_seed(9)
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * D, generator=g).bfloat16()
    table = _table(D, 64)
    pos = torch.tensor([0, 7, 49, 50, 31], dtype=torch.int32)
    cache_k = torch.full((B, max_len, Hkv, D), 3.0, dtype=torch.bfloat16, device=device)
    cache_v = torch.full((B, max_len, Hkv, D), 5.0, dtype=torch.bfloat16, device=device)
    q_rot = capi.rot_embed_kv_cache_at(qkv.to(device), table.to(device), cache_k, cache_v, pos.to(device), Hq, Hkv)
    torch.cuda.synchronize()
    q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    want_k = torch.full((B, max_len, Hkv, D), 3.0, dtype=torch.bfloat16)
    want_v = torch.full((B, max_len, Hkv, D), 5.0, dtype=torch.bfloat16)
    for b in range(B):
        p = int(pos[b])
        if p >= max_len:
            continue
        f = table[p:p + 1]
        assert torch.equal(q_rot[b:b + 1].cpu(), rot_embed_reference(q[b:b + 1].reshape(1, T, Hq, D), f))
        want_k[b, p] = rot_embed_reference(k[b:b + 1].reshape(1, T, Hkv, D), f)[0, 0]
        want_v[b, p] = v[b].reshape(T, Hkv, D)[0]
    assert torch.equal(cache_k.cpu(), want_k) and torch.equal(cache_v.cpu(), want_v)


def test_errors(capi, device):
    lib = capi.load()
    x = torch.zeros(64, dtype=torch.bfloat16, device=device)
    f = torch.zeros(64, device=device)
    assert lib.l3ci_rot_embed(x.data_ptr() + 2, f.data_ptr(), x.data_ptr(), 1, 1, 1, 8, 8, 8, 8, None) == capi.ERR_ALIGNMENT
    assert lib.l3ci_rot_embed(x.data_ptr(), f.data_ptr(), x.data_ptr(), 1, 1, 1, 7, 7, 7, 7, None) == capi.ERR_UNSUPPORTED


@pytest.mark.parametrize("which", ["q", "k"])
def test_config4_is_bit_equal_to_the_reference_kernels_output(capi, device, ref_cuda, which):
    """Directly against what the reference's own CUDA kernel wrote for configuration 4 on a B200 (every element)."""
    from test_oracle_reference_cuda import c4_rope_full

    t, freq, full = c4_rope_full(ref_cuda, which)
    got = capi.rot_embed(t.to(device), freq.to(device))
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), full)


@pytest.mark.parametrize("name", sorted(inputs.ROPE_GOLDEN_CASES))
def test_small_shapes_are_bit_equal_to_the_reference_kernels_output(capi, device, ref_cuda, name):
    B, S, H, D, seed, extra = inputs.ROPE_GOLDEN_CASES[name]
    x = inputs.rope_case(B, S, H, D, seed, extra)
    freq = freqs_cis_reference(D, S, theta=500000.0, use_scaled=True, scale_factor=8)
    got = capi.rot_embed(x.to(device), freq.to(device))
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), ref_cuda["rope/" + name])
