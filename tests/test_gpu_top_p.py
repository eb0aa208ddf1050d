"""The nucleus-sampling step (`l3ci_top_p_step`) against the restatement of the reference's `sample_top_p`
(oracle/sampling.py, pinned to the reference's own draws in tests/test_oracle_golden.py).

A sampler is checked at the level of its distribution: the nucleus it draws from must be the oracle's (exactly,
except for entries whose preceding mass is within fp32 rounding of top_p), every token it returns must lie in it,
and the frequencies of many draws must fit the renormalised probabilities (chi-square).  The nucleus is taken from
the float64 value of the reference's formula: torch's own fp32 softmax is up to 1e-4 off in its normalisation on
adversarial rows (see oracle/sampling.py), more than this kernel's error."""
import pytest
import torch

from oracle import sampling

pytestmark = pytest.mark.gpu
BAND = 5e-6   # fp32 sums of up to 128 256 probabilities: entries this close to the boundary may fall on either side


def _state(B, G, device):
    return (torch.zeros(B, G, dtype=torch.int64, device=device), torch.zeros(B, dtype=torch.int64, device=device),
            torch.zeros(B, dtype=torch.int64, device=device), torch.zeros(B, dtype=torch.int32, device=device),
            torch.zeros(B, dtype=torch.int32, device=device))


def _logits(kind, rows, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    if kind == "normal":
        x = torch.randn(rows, vocab, generator=g)
    elif kind == "peaked":
        x = torch.randn(rows, vocab, generator=g) * 6
    elif kind == "flat":
        x = torch.zeros(rows, vocab)                       # every entry ties with every other
    elif kind == "two_levels":
        x = torch.where(torch.rand(rows, vocab, generator=g) < 0.01, torch.tensor(4.0), torch.tensor(0.0))
    elif kind == "one_hot":
        x = torch.full((rows, vocab), -30.0)
        x[torch.arange(rows), torch.randint(0, vocab, (rows,), generator=g)] = 20.0
    return x.bfloat16()


@pytest.mark.parametrize("kind", ["normal", "peaked", "flat", "two_levels", "one_hot"])
@pytest.mark.parametrize("vocab,temperature,top_p", [(1000, 0.6, 0.9), (128256, 0.6, 0.9), (32003, 1.0, 0.5), (4096, 0.3, 0.99)])
def test_nucleus_is_the_references(capi, device, kind, vocab, temperature, top_p):
    rows = 4
    logits = _logits(kind, rows, vocab, seed=vocab + len(kind))
    probs = sampling.softmax_with_temperature(logits, temperature, torch.float64)
    kept, renorm, before = sampling.nucleus_reference(probs, top_p)
    lo = (before <= top_p - BAND).sum(-1)       # entries that are in beyond doubt
    hi = (before <= top_p + BAND).sum(-1)       # ... and those that may be
    out, steps, cur, pos, lens = _state(rows, 1, device)
    count = torch.zeros(rows, dtype=torch.int32, device=device)
    mass = torch.zeros(rows, dtype=torch.float32, device=device)
    capi.top_p_step(logits.to(device), temperature, top_p, 1234, out, steps, cur, pos, lens, count, mass)
    torch.cuda.synchronize()
    count, mass, tok = count.cpu(), mass.cpu().double(), cur.cpu()
    assert bool((count >= lo).all()) and bool((count <= hi).all()), (count, lo, hi)
    mass_lo = (probs.double() * (before <= top_p - BAND)).sum(-1)
    mass_hi = (probs.double() * (before <= top_p + BAND)).sum(-1)
    assert bool((mass >= mass_lo - 1e-5).all()) and bool((mass <= mass_hi + 1e-5).all())
    assert bool(torch.gather(before <= top_p + BAND, 1, tok.view(-1, 1)).all()), "token outside the nucleus"
    assert torch.equal(out[:, 0].cpu(), tok) and bool((steps == 1).all()) and bool((pos == 1).all()) and bool((lens == 1).all())


def test_frequencies_follow_the_renormalised_nucleus(capi, device):
    vocab, temperature, top_p, rows, steps_n = 1000, 0.8, 0.9, 4096, 12
    row = _logits("normal", 1, vocab, seed=5) * 2
    probs = sampling.softmax_with_temperature(row, temperature, torch.float64)
    kept, renorm, before = sampling.nucleus_reference(probs, top_p)
    logits = row.expand(rows, vocab).contiguous().to(device)           # the same distribution in every row
    out, steps, cur, pos, lens = _state(rows, steps_n, device)
    for _ in range(steps_n):                                            # (row, step) index the random stream
        capi.top_p_step(logits, temperature, top_p, 99, out, steps, cur, pos, lens)
    torch.cuda.synchronize()
    draws = out.cpu().flatten()
    n = draws.numel()
    freq = torch.bincount(draws, minlength=vocab).double()
    assert float(freq[~kept[0]].sum()) <= n * 1e-4                      # (boundary band only)
    expected = renorm[0] * n
    sel = expected >= 5                                                 # pool the thin tail into one cell
    chi2 = float((((freq[sel] - expected[sel]) ** 2) / expected[sel]).sum())
    tail_e, tail_o = float(expected[~sel].sum()), float(freq[~sel].sum())
    dof = int(sel.sum()) - 1
    if tail_e > 0:
        chi2 += (tail_o - tail_e) ** 2 / tail_e
        dof += 1
    assert chi2 < dof + 6 * (2 * dof) ** 0.5, (chi2, dof)
    # consecutive steps of a row are not the same draw repeated, and rows differ
    assert len(set(out[0].tolist())) > 1 and len(set(out[:, 0].tolist())) > 10


def test_draws_are_reproducible_and_keyed_by_seed_row_and_step(capi, device):
    rows, vocab = 64, 128256
    logits = _logits("normal", rows, vocab, seed=9).to(device)

    def run(seed, start_step):
        out, steps, cur, pos, lens = _state(rows, 4, device)
        steps.fill_(start_step)
        capi.top_p_step(logits, 0.6, 0.9, seed, out, steps, cur, pos, lens)
        torch.cuda.synchronize()
        return cur.cpu()

    a, b, c, d = run(7, 0), run(7, 0), run(8, 0), run(7, 1)
    assert torch.equal(a, b)
    assert not torch.equal(a, c) and not torch.equal(a, d)


def test_limits_greedy_and_whole_vocabulary(capi, device):
    rows, vocab = 8, 5000
    logits = _logits("normal", rows, vocab, seed=3)
    out, steps, cur, pos, lens = _state(rows, 1, device)
    count = torch.zeros(rows, dtype=torch.int32, device=device)
    # a tiny nucleus: only the most probable entry is ever kept (its preceding mass is 0 <= p)
    capi.top_p_step(logits.to(device), 0.05, 1e-6, 1, out, steps, cur, pos, lens, count)
    torch.cuda.synchronize()
    assert torch.equal(cur.cpu(), logits.float().argmax(-1)) and bool((count == 1).all())
    # top_p = 1: nothing is cut
    capi.top_p_step(logits.to(device), 1.0, 1.0, 1, out, steps, cur, pos, lens, count)
    torch.cuda.synchronize()
    assert bool((count.cpu() >= vocab - 2).all())
    with pytest.raises(capi.L3ciError):
        capi.top_p_step(logits.to(device), 0.0, 0.9, 1, out, steps, cur, pos, lens)


@pytest.mark.parametrize("kind,vocab", [("normal", 128256), ("flat", 32003), ("two_levels", 128256), ("peaked", 1001),
                                        ("one_hot", 4096), ("normal", 37), ("flat", 8)])
def test_several_ctas_per_row_change_no_bit(capi, device, kind, vocab):
    """Small batches run as a cluster of 8, 4 or 2 CTAs per row (up to 15, 33, 74 rows), larger ones with one CTA per
    row.  The draw is keyed by (seed, row, step) and all sums are integers, so the same rows give the same tokens,
    nucleus sizes and masses either way: the first rows of a batch of 80 (one CTA each) against batches of 10, 30 and
    40 of them."""
    large = 80
    logits = _logits(kind, large, vocab, seed=17 + vocab)

    def run(rows):
        out, steps, cur, pos, lens = _state(rows, 3, device)
        count = torch.zeros(rows, dtype=torch.int32, device=device)
        mass = torch.zeros(rows, dtype=torch.float32, device=device)
        for _ in range(3):
            capi.top_p_step(logits[:rows].to(device), 0.7, 0.9, 4242, out, steps, cur, pos, lens, count, mass)
        torch.cuda.synchronize()
        return out.cpu(), count.cpu(), mass.cpu(), pos.cpu()

    ref = run(large)
    for small in (10, 30, 40):
        got = run(small)
        for a, b in zip(got, ref):
            assert torch.equal(a, b[:small]), small
        assert bool((got[3] == 3).all())
