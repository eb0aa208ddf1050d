"""The oracle and the product's host-side rotary table against vectors the reference itself produced
(tests/golden/make_golden.py).  CPU only."""
import hashlib

import pytest
import torch

from oracle import attention, compare, inputs, rope

CASES = {
    "c1": lambda: inputs.config1(),
    "d128_r4_s300": lambda: inputs.decode_case(2, 8, 2, 128, 300, seed=7),
    "d64_r1_s65": lambda: inputs.decode_case(2, 4, 4, 64, 65, seed=8),
    "d128_r8_s1000": lambda: inputs.decode_case(1, 8, 1, 128, 1000, seed=9),
    "d128_r3_s130_uniform01": lambda: inputs.decode_case(1, 6, 2, 128, 130, seed=10, dist="uniform"),
}


def _sha(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


@pytest.mark.parametrize("dim", [64, 128])
def test_oracle_rope_table_matches_reference_rows(golden, dim):
    rows = golden["freq_rows"].tolist()
    scaled = rope.freqs_cis_reference(dim, 16384, 500000.0, True)
    plain = rope.freqs_cis_reference(dim, 16384, 10000.0, False)
    assert torch.equal(scaled[rows], golden[f"freqs_cis_scaled_d{dim}"])
    assert torch.equal(plain[rows], golden[f"freqs_cis_plain_d{dim}"])
    base = 1.0 / (500000.0 ** (torch.arange(0, dim, 2)[: dim // 2].float() / dim))
    assert torch.equal(rope.apply_scaling_reference(base), golden[f"apply_scaling_d{dim}"])


@pytest.mark.parametrize("dim", [64, 128])
def test_product_rope_table_is_bit_identical_to_reference(pkg, golden, dim):
    rt = pkg.rope_table
    rows = golden["freq_rows"].tolist()
    assert torch.equal(rt.precompute_freqs_cis(dim, 16384, 500000.0, True)[rows], golden[f"freqs_cis_scaled_d{dim}"])
    assert torch.equal(rt.precompute_freqs_cis(dim, 16384, 10000.0, False)[rows], golden[f"freqs_cis_plain_d{dim}"])
    assert _sha(rt.precompute_freqs_cis(dim, 2048, 500000.0, True)) == golden[f"freqs_cis_scaled_d{dim}_sha256_2048"]
    base = 1.0 / (500000.0 ** (torch.arange(0, dim, 2)[: dim // 2].float() / dim))
    assert torch.equal(rt.apply_scaling(base), golden[f"apply_scaling_d{dim}"])


@pytest.mark.parametrize("factor", [8, 32])
def test_product_rope_scaling_parameters_match_oracle(pkg, factor):
    kw = dict(scale_factor=factor, low_freq_factor=1, high_freq_factor=4, old_context_len=8192)
    for dim in (64, 128):
        a = pkg.rope_table.precompute_freqs_cis(dim, 2048, 500000.0, True, **kw)
        b = rope.freqs_cis_reference(dim, 2048, 500000.0, True, **kw)
        assert torch.equal(a, b)
    with pytest.raises(ValueError):
        pkg.rope_table.apply_scaling(torch.ones(4), low_freq_factor=2, high_freq_factor=2)


@pytest.mark.parametrize("name", sorted(CASES))
def test_attention_oracle_matches_reference_sdpa(golden, name):
    case = CASES[name]()
    assert _sha(case.q) + _sha(case.k) + _sha(case.v) == golden[f"sdpa_{name}_inputs_sha256"], "input generator drifted"
    ref_bf16 = golden[f"sdpa_{name}_bf16"]
    ours = attention.sdpa_reference(case.q, case.k, case.v)
    # The reference call computes in bf16; the oracle is the same call in fp32.
    compare.assert_close_attention(ref_bf16, ours, atol=2e-2, rtol=1e-2, max_rel_l2=2e-2)
    # and the bf16 evaluation of the oracle function is the reference call itself, bit for bit
    again = attention.sdpa_reference(case.q, case.k, case.v, dtype=torch.bfloat16)
    assert torch.equal(again, ref_bf16)


PREFILL_CASES = {"d64_r4_t40": (2, 8, 2, 64, 40, 21), "d128_r2_t150": (1, 4, 2, 128, 150, 22)}


@pytest.mark.parametrize("name", sorted(PREFILL_CASES))
def test_prefill_oracle_matches_reference_sdpa(golden, name):
    """The golden tensors are outputs of the reference's prefill call (model.py:114-116) on these inputs."""
    q, k, v = inputs.prefill_case(*PREFILL_CASES[name])
    assert _sha(q) + _sha(k) + _sha(v) == golden[f"prefill_{name}_inputs_sha256"], "input generator drifted"
    ref_bf16 = golden[f"prefill_{name}_bf16"]
    compare.assert_close_attention(ref_bf16, attention.prefill_reference(q, k, v), atol=2e-2, rtol=1e-2, max_rel_l2=2e-2)
    assert torch.equal(attention.prefill_reference(q, k, v, dtype=torch.bfloat16), ref_bf16)
    # the explicit-mask form used for later chunks is the same function at start_pos = 0
    T = q.shape[2]
    chunk = attention.prefill_reference(q[:, :, T // 2:], k, v, start_pos=T // 2)
    compare.assert_close_attention(chunk, attention.prefill_reference(q, k, v)[:, :, T // 2:], atol=1e-5, rtol=1e-5, max_rel_l2=1e-5)


@pytest.mark.parametrize("ragged", [False, True])
def test_attention_oracle_matches_float64_restatement(ragged):
    case = inputs.decode_case(3, 12, 4, 64, 150, seed=3, ragged=ragged)
    if ragged:
        case.seq_lens[1] = 0  # an empty sequence yields zeros
    a = attention.sdpa_reference(case.q, case.k, case.v, case.seq_lens)
    b, lse = attention.attention_float64(case.q, case.k, case.v, case.seq_lens)
    assert (a.double() - torch.from_numpy(b)).abs().max().item() < 2e-6
    if ragged:
        assert a[1].abs().max().item() == 0 and lse[1].max() == float("-inf")


def test_lse_merge_reference_reassembles_attention():
    case = inputs.decode_case(2, 8, 2, 64, 200, seed=5)
    full, _ = attention.attention_float64(case.q, case.k, case.v)
    parts_o, parts_l = [], []
    for lo, hi in [(0, 64), (64, 192), (192, 200)]:
        o, l = attention.attention_float64(case.q, case.k[:, :, lo:hi], case.v[:, :, lo:hi])
        parts_o.append(torch.from_numpy(o[:, :, 0]))
        parts_l.append(torch.from_numpy(l))
    merged = attention.lse_merge_reference(torch.stack(parts_o), torch.stack(parts_l))
    assert (merged.double() - torch.from_numpy(full[:, :, 0])).abs().max().item() < 1e-6


def test_bf16_ulp_distance():
    a = torch.tensor([1.0, -1.0, 0.0, 2.0]).bfloat16()
    b = torch.tensor([1.0078125, -1.0, -0.0, 1.9921875]).bfloat16()
    assert compare.bf16_ulp_distance(a, b).tolist() == [1, 0, 0, 1]


TOP_P_CASES = {"flat": (3, 500, 1.0, 0.9, 11), "peaked": (2, 2000, 6.0, 0.9, 12), "half": (4, 300, 2.0, 0.5, 13)}


@pytest.mark.parametrize("name", sorted(TOP_P_CASES))
def test_top_p_oracle_matches_the_references_sampler(golden, name):
    """The golden draws are what the reference's own sample_top_p (model.py:400-423) returned for these seeded
    distributions under torch.manual_seed(seed): the restatement must return the same tokens, and every one of them
    must lie in the nucleus the oracle describes."""
    from oracle import sampling

    rows, vocab, scale, p, seed = TOP_P_CASES[name]
    g = torch.Generator().manual_seed(seed)
    probs = torch.softmax(torch.randn(rows, vocab, generator=g) * scale, dim=-1)
    want = golden[f"top_p_{name}_draws"]
    torch.manual_seed(seed)
    got = torch.cat([sampling.sample_top_p_reference(probs.clone(), p) for _ in range(want.shape[1])], dim=1)
    assert torch.equal(got, want)
    kept, renorm, before = sampling.nucleus_reference(probs, p)
    assert bool(torch.gather(kept, 1, want).all())
    assert torch.allclose(renorm.sum(-1), torch.ones(rows, dtype=torch.float64))
    # the nucleus is the shortest descending prefix whose mass exceeds p
    mass = (probs.double() * kept).sum(-1)
    smallest_kept = torch.where(kept, probs.double(), torch.ones_like(probs.double())).min(-1).values
    assert bool((mass > p).all()) and bool((mass - smallest_kept <= p + 1e-12).all())
