"""Causal GQA prefill attention through the C ABI and the extension against the reference's PyTorch call
(model.py:114-116) in fp32 on the CPU.  Tolerance: the attention tolerance of the decode tests."""
import pytest
import torch

from oracle import attention, compare

pytestmark = pytest.mark.gpu
ATOL, RTOL, REL_L2 = 2e-2, 1e-2, 1e-2


def _case(B, Hq, Hkv, D, T, S, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, Hq, D, generator=g).bfloat16().transpose(1, 2)        # the model's layout, model.py:96-112
    k = torch.randn(B, S, Hkv, D, generator=g).bfloat16().transpose(1, 2)
    v = torch.randn(B, S, Hkv, D, generator=g).bfloat16().transpose(1, 2)
    return q, k, v


def _check(capi, device, B, Hq, Hkv, D, T, S=None, start_pos=0, seed=0, scale=0.0, variant=0):
    S = T + start_pos if S is None else S
    q, k, v = _case(B, Hq, Hkv, D, T, S, seed)
    got = capi.prefill_attention(q.to(device), k.to(device), v.to(device), start_pos=start_pos, scale=scale,
                                 variant=variant)
    torch.cuda.synchronize()
    assert got.shape == q.shape and got.stride() == q.stride() and got.dtype == torch.bfloat16
    want = attention.prefill_reference(q, k[:, :, :start_pos + T], v[:, :, :start_pos + T], start_pos,
                                       scale=scale if scale > 0 else None)
    compare.assert_close_attention(got, want, ATOL, RTOL, REL_L2)


@pytest.mark.parametrize("variant", [1, 2])      # 1: tcgen05 / tensor-memory kernel, 2: mma.sync kernel
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("T", [2, 17, 64, 65, 128, 129, 200, 256, 513])
def test_prompt_lengths_around_the_block_sizes(capi, device, D, T, variant):
    _check(capi, device, 2, 8, 2, D, T, seed=T + D, variant=variant)


@pytest.mark.parametrize("Hq,Hkv", [(32, 8), (8, 8), (6, 2), (16, 1), (24, 8)])
def test_head_ratios(capi, device, Hq, Hkv):
    _check(capi, device, 1, Hq, Hkv, 64, 150, seed=Hq)


# The tcgen05 kernel comes in two forms: two query heads of a KV head per CTA when the head ratio is even, one head
# per CTA otherwise (ratios 1 and 3 here).
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("Hq,Hkv", [(8, 8), (6, 2), (8, 4), (16, 2), (2, 1)])
@pytest.mark.parametrize("T", [128, 300, 640])
def test_head_ratios_on_the_tensor_memory_kernel(capi, device, Hq, Hkv, D, T):
    _check(capi, device, 2, Hq, Hkv, D, T, seed=Hq * 7 + T + D, variant=1)


def test_model_prefill_shape(capi, device):
    # benchmark_model.py's first scenario at a smaller batch: 128-token prompts of the 1B shape
    _check(capi, device, 4, 32, 8, 64, 128, seed=5)


@pytest.mark.parametrize("variant", [1, 2])
def test_long_prompt(capi, device, variant):
    _check(capi, device, 1, 32, 8, 128, 2048, seed=6, variant=variant)
    _check(capi, device, 2, 32, 8, 64, 1000, seed=7, variant=variant)


@pytest.mark.parametrize("D", [64, 128])
def test_more_query_blocks_than_sms(capi, device, D):
    # the persistent form of the head-pair kernel: a CTA per SM walks several (head pair, query block) items, with a
    # ragged last block, and as a later chunk of a longer cache
    _check(capi, device, 3, 32, 8, D, 1111, seed=21 + D)
    _check(capi, device, 2, 32, 8, D, 700, S=1500, start_pos=800, seed=22 + D)
    _check(capi, device, 5, 16, 8, D, 640, seed=23 + D, scale=0.11)


def test_very_long_prompt_on_the_default_kernel(capi, device):
    # 32 query blocks per head: every CTA of the head-pair kernel walks up to 32 key tiles
    _check(capi, device, 1, 8, 2, 128, 4096, seed=8)
    _check(capi, device, 1, 4, 4, 64, 4000, seed=9)      # head ratio 1: one head per CTA, ragged last block


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("start_pos,T,S", [(100, 60, 160), (64, 64, 200), (1, 1, 2), (300, 5, 305), (7, 130, 137),
                                           (200, 300, 640), (128, 128, 256)])
def test_later_chunk_and_longer_cache(capi, device, start_pos, T, S, variant):
    # a chunk that starts at start_pos; rows beyond start_pos + T of the cache must not be seen
    q, k, v = _case(2, 8, 4, 128, T, S, seed=start_pos)
    k2, v2 = k.clone(), v.clone()
    k2[:, :, start_pos + T:] = 1e4                       # poison what lies beyond the causal limit
    v2[:, :, start_pos + T:] = 1e4
    got = capi.prefill_attention(q.to(device), k2.to(device), v2.to(device), start_pos=start_pos, variant=variant)
    want = attention.prefill_reference(q, k[:, :, :start_pos + T], v[:, :, :start_pos + T], start_pos)
    compare.assert_close_attention(got, want, ATOL, RTOL, REL_L2)


def test_custom_scale_and_decode_agreement(capi, device):
    _check(capi, device, 2, 8, 2, 64, 90, seed=9, scale=0.07)
    # the last row of a prefill is a decode step over the same cache
    q, k, v = _case(2, 16, 4, 128, 70, 70, seed=10)
    pre = capi.prefill_attention(q.to(device), k.to(device), v.to(device))
    dec = capi.flash_attention_decode(q[:, :, -1:].to(device), k.to(device), v.to(device))
    compare.assert_close_attention(pre[:, :, -1:], dec.float().cpu(), 1e-2, 1e-2, REL_L2)


def test_extension_call_form_and_errors(ext, device):
    q, k, v = _case(2, 8, 2, 64, 40, 40, seed=12)
    got = ext.prefill_attention(q.to(device), k.to(device), v.to(device))
    compare.assert_close_attention(got, attention.prefill_reference(q, k, v), ATOL, RTOL, REL_L2)
    got = ext.prefill_attention(q.to(device)[:, :, :10], k.to(device), v.to(device), start_pos=30)
    compare.assert_close_attention(got, attention.prefill_reference(q[:, :, :10], k, v, 30), ATOL, RTOL, REL_L2)
    with pytest.raises(RuntimeError):
        ext.prefill_attention(q.to(device), k.to(device), v.to(device), start_pos=1)      # start_pos + T > keys
    with pytest.raises(RuntimeError):
        ext.prefill_attention(q.to(device)[..., :32], k.to(device)[..., :32], v.to(device)[..., :32])  # head size 32
