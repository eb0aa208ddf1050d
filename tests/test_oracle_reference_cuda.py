"""The RMSNorm and rotary-rotation oracles against outputs of the reference's own CUDA kernels
(tests/golden/reference_cuda_vectors.pt, written on a B200 by tests/golden/make_reference_cuda_golden.py from the
reference's unmodified custom_kernels.cu compiled for sm_100).  CPU only.

What is pinned, and how tightly:
  rms_norm_reference_rounding   bit-equal to the reference kernel (its three bf16 roundings restated)
  rms_norm_reference            the fp32, one-rounding form the product kernel is held to: within 2 bf16 ulp of the
                                reference kernel (the reference's extra roundings), more than 99 % within 1
  rot_embed_reference           bit-equal to the reference kernel (the compiler's fused multiply-add form)
  rot_embed_reference_unfused   the source as written: differs from the compiled kernel in ~1e-5 of the elements
"""
import pytest
import torch

from oracle import compare, inputs
from oracle.rms_norm import rms_norm_reference, rms_norm_reference_rounding
from oracle.rope import freqs_cis_reference, rot_embed_reference, rot_embed_reference_fma, rot_embed_reference_unfused

SMALL_ROPE_TABLE = dict(theta=500000.0, use_scaled=True, scale_factor=8)


def c4_rope_full(ref_cuda, which):
    """(input view, table, the reference kernel's whole output on configuration 4's q or k), the output rebuilt
    from the unfused restatement and the held list of all elements where the kernel differs from it."""
    _, _, _, qkv = inputs.config4(seed=42)
    Hq, Hkv, D = 32, 8, 64
    B, S = qkv.shape[:2]
    freq = freqs_cis_reference(D, S, **inputs.ROPE_CONFIG4)
    t = qkv[..., : Hq * D].view(B, S, Hq, D) if which == "q" else qkv[..., Hq * D: (Hq + Hkv) * D].view(B, S, Hkv, D)
    full = rot_embed_reference_unfused(t, freq).contiguous()
    flat = full.view(-1)
    flat[ref_cuda[f"rope/c4_{which}_diff_idx"].long()] = ref_cuda[f"rope/c4_{which}_diff_val"]
    # the rows held verbatim agree with the rebuilt output
    assert torch.equal(full[:, :: inputs.C4_GOLDEN_ROW_STEP], ref_cuda[f"rope/c4_{which}"])
    return t, freq, full


@pytest.mark.parametrize("name", sorted(inputs.RMS_GOLDEN_CASES))
def test_rms_norm_oracles_against_the_reference_kernel(ref_cuda, name):
    B, S, E, seed = inputs.RMS_GOLDEN_CASES[name]
    x, w = inputs.rms_case(B, S, E, seed)
    want = ref_cuda["rms/" + name]
    assert torch.equal(rms_norm_reference_rounding(x, w, 1e-5), want)
    d = compare.bf16_ulp_distance(rms_norm_reference(x, w, 1e-5), want)
    assert int(d.max()) <= 2 and float((d > 1).float().mean()) < 0.01


def test_rms_norm_oracles_against_the_reference_kernel_config4(ref_cuda):
    x, w, eps, _ = inputs.config4(seed=42)
    rows = slice(None, None, inputs.C4_GOLDEN_ROW_STEP)
    want = ref_cuda["rms/c4_rows"]
    assert torch.equal(rms_norm_reference_rounding(x, w, eps).view(-1, x.shape[-1])[rows], want)
    d = compare.bf16_ulp_distance(rms_norm_reference(x, w, eps).view(-1, x.shape[-1])[rows].contiguous(), want)
    assert int(d.max()) <= 2 and float((d > 1).float().mean()) < 0.01


@pytest.mark.parametrize("name", sorted(inputs.ROPE_GOLDEN_CASES))
def test_rotation_oracle_is_bit_equal_to_the_reference_kernel(ref_cuda, name):
    B, S, H, D, seed, extra = inputs.ROPE_GOLDEN_CASES[name]
    x = inputs.rope_case(B, S, H, D, seed, extra)
    freq = freqs_cis_reference(D, S, **SMALL_ROPE_TABLE)
    assert torch.equal(rot_embed_reference(x, freq), ref_cuda["rope/" + name])


@pytest.mark.parametrize("which", ["q", "k"])
def test_rotation_oracle_is_bit_equal_on_all_of_config4(ref_cuda, which):
    t, freq, full = c4_rope_full(ref_cuda, which)
    assert torch.equal(rot_embed_reference(t, freq), full)
    # the other three ways a compiler could have contracted the two expressions are NOT the reference's
    for form in ("aa", "ab", "ba"):
        assert not torch.equal(rot_embed_reference_fma(t, freq, form), full)
    # and the uncontracted source differs in a handful of elements, by more than one ulp in places
    n_diff = ref_cuda[f"rope/c4_{which}_diff_idx"].numel()
    assert 0 < n_diff < 1e-4 * full.numel()
