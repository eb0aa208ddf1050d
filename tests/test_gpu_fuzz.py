"""Seeded random shapes for the two attention entry points against the oracle: head sizes, head ratios, batch sizes,
cache lengths, ragged lengths (empty sequences included), both cache layouts, restricted grids, chunk offsets."""
import random

import pytest
import torch

from oracle import attention, compare

pytestmark = pytest.mark.gpu
ATOL, RTOL, REL_L2 = 2e-2, 1e-2, 1e-2


@pytest.mark.parametrize("seed", range(10))
def test_decode_random_shapes(capi, device, seed):
    rnd = random.Random(1000 + seed)
    for it in range(12):
        D = rnd.choice([64, 128])
        Hkv = rnd.choice([1, 2, 3, 4, 8, 16])
        R = rnd.choice([1, 2, 3, 4, 8, 12, 16])
        B = rnd.choice([1, 2, 3, 5, 16, 37, 70])
        S = rnd.choice([1, 7, 31, 32, 33, 100, 256, 700, 1500, 3000])
        S = max(1, min(S, int(3e6 // (B * Hkv * D))))
        g = torch.Generator().manual_seed(seed * 100 + it)
        q = torch.randn(B, 1, Hkv * R, D, generator=g).bfloat16().transpose(1, 2)
        if rnd.random() < 0.5:
            k = torch.randn(B, S, Hkv, D, generator=g).bfloat16().transpose(1, 2)
            v = torch.randn(B, S, Hkv, D, generator=g).bfloat16().transpose(1, 2)
        else:
            k = torch.randn(B, Hkv, S, D, generator=g).bfloat16()
            v = torch.randn(B, Hkv, S, D, generator=g).bfloat16()
        lens = None
        if rnd.random() < 0.5:
            lens = torch.tensor([rnd.randint(0 if rnd.random() < 0.15 else 1, S) for _ in range(B)], dtype=torch.int32)
        # 0: the library's choice of kernel; > 0: persistent grid of that size; < 0: the static deal, its own split
        # or one of -(16 * C + W) (units over warps: 17, 18, 20, 24; clusters: 40, 72, 136); it takes R <= 8 only
        mc = rnd.choice([0, 0, 0, 1, 7, 100, -1, -1, -17, -18, -20, -24, -40, -72, -136])
        if mc < 0 and R > 8:
            mc = 0
        got = capi.flash_attention_decode(q.to(device), k.to(device), v.to(device),
                                          seq_lens=lens.to(device) if lens is not None else None, max_ctas=mc)
        torch.cuda.synchronize()
        want = attention.sdpa_reference(q, k, v, lens)
        try:
            compare.assert_close_attention(got, want, ATOL, RTOL, REL_L2)
        except AssertionError as e:
            raise AssertionError(f"B={B} Hq={Hkv * R} Hkv={Hkv} D={D} S={S} lens={lens} max_ctas={mc}: {e}") from e


@pytest.mark.parametrize("seed", range(4))
def test_prefill_random_shapes(capi, device, seed):
    rnd = random.Random(2000 + seed)
    for it in range(8):
        D = rnd.choice([64, 128])
        Hkv = rnd.choice([1, 2, 4, 8])
        R = rnd.choice([1, 2, 4, 8])
        B = rnd.choice([1, 2, 3])
        T = rnd.choice([2, 5, 63, 64, 65, 127, 128, 129, 255, 300, 700])
        start = rnd.choice([0, 0, 1, 50, 128, 333])
        extra = rnd.choice([0, 0, 17])
        S = start + T + extra
        variant = rnd.choice([1, 2])
        g = torch.Generator().manual_seed(seed * 100 + it)
        q = torch.randn(B, T, Hkv * R, D, generator=g).bfloat16().transpose(1, 2)
        k = torch.randn(B, S, Hkv, D, generator=g).bfloat16().transpose(1, 2)
        v = torch.randn(B, S, Hkv, D, generator=g).bfloat16().transpose(1, 2)
        got = capi.prefill_attention(q.to(device), k.to(device), v.to(device), start_pos=start, variant=variant)
        torch.cuda.synchronize()
        want = attention.prefill_reference(q, k[:, :, :start + T], v[:, :, :start + T], start)
        try:
            compare.assert_close_attention(got, want, ATOL, RTOL, REL_L2)
        except AssertionError as e:
            raise AssertionError(f"B={B} Hq={Hkv * R} Hkv={Hkv} D={D} T={T} start={start} S={S} variant={variant}: {e}") from e
