"""The drop-in boundary: `custom_kernels_extension` called exactly as the reference's model.py and
benchmark_kernel.py call it, checked against the oracle."""
import pytest
import torch
import torch.nn.functional as F

from oracle import attention, compare, inputs
from oracle.rms_norm import rms_norm_reference
from oracle.rope import freqs_cis_reference, rot_embed_reference

pytestmark = pytest.mark.gpu


def test_benchmark_kernel_call_form(ext, device):
    # benchmark_kernel.py:161-173: rand inputs reshaped to (B,1,Hq,D)/(B,S,Hkv,D), moved to cuda, transposed
    case = inputs.decode_case(1, 32, 8, 128, 8192, seed=42, dist="uniform")
    q, k, v = (t.to(device) for t in (case.q, case.k, case.v))
    out = ext.flash_attention_decode(q, k, v)
    torch.cuda.synchronize()
    assert out.shape == q.shape and out.stride() == q.stride()
    compare.assert_close_attention(out, attention.sdpa_reference(case.q, case.k, case.v))
    assert ext.flash_decode_status(q) == 0


def test_attention_layer_decode_step_like_the_model(ext, pkg, device):
    """One decode step of CausalSelfAttention.forward (model.py:92-122) with T == 1, written with the same
    extension calls and tensor views, against the same step computed by the oracle on the CPU."""
    B, Hq, Hkv, D, max_len, start = 4, 32, 8, 64, 64, 37
    C = Hq * D
    g = torch.Generator().manual_seed(5)
    x = torch.randn(B, 1, C, generator=g).bfloat16()
    ln_w = (1 + 0.02 * torch.randn(C, generator=g)).bfloat16()
    w_attn = (0.02 * torch.randn((Hq + 2 * Hkv) * D, C, generator=g)).bfloat16()
    cache_k = torch.randn(B, max_len, Hkv, D, generator=g).bfloat16()
    cache_v = torch.randn(B, max_len, Hkv, D, generator=g).bfloat16()
    table = pkg.rope_table.precompute_freqs_cis(D, 128, 500000.0, True)
    freqs = table[start:start + 1]

    # --- GPU, through the extension, mirroring model.py line by line
    dx, dw, dwa = x.to(device), ln_w.to(device), w_attn.to(device)
    dck, dcv, dfreqs = cache_k.to(device), cache_v.to(device), freqs.to(device)
    h = ext.rms_norm(dx, dw, 1e-5)                                         # model.py:71
    qkv = F.linear(h, dwa)                                                 # model.py:95
    q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)                # model.py:96
    q, k, v = map(lambda t: t.view(B, 1, -1, D), (q, k, v))                # model.py:97
    q = ext.rot_embed(q, dfreqs)                                           # model.py:100
    k = ext.rot_embed(k, dfreqs)                                           # model.py:101
    dck[:B, start:start + 1] = k                                           # model.py:105
    dcv[:B, start:start + 1] = v                                           # model.py:106
    kk, vv = dck[:B, :start + 1], dcv[:B, :start + 1]                      # model.py:107-108
    q, kk, vv = map(lambda t: t.transpose(1, 2), (q, kk, vv))              # model.py:111
    y = ext.flash_attention_decode(q, kk, vv)                              # model.py:118
    y = y.transpose(1, 2).contiguous().view(B, 1, C)                       # model.py:120
    torch.cuda.synchronize()

    # --- the fused entry point gives the same q and the same cache rows
    dck2, dcv2 = cache_k.to(device), cache_v.to(device)
    q2 = ext.rot_embed_kv_cache(qkv, dfreqs, dck2, dcv2, start, Hq, Hkv)
    torch.cuda.synchronize()
    assert torch.equal(q2.transpose(1, 2), q) and torch.equal(dck2, dck) and torch.equal(dcv2, dcv)

    # --- CPU oracle on the same intermediate (qkv is taken from the GPU so that the GEMM is not under test)
    h_ref = rms_norm_reference(x, ln_w, 1e-5)
    assert compare.max_bf16_ulp(h, h_ref) <= 1
    qkv_c = qkv.cpu()
    qc, kc, vc = qkv_c.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    qc, kc, vc = map(lambda t: t.reshape(B, 1, -1, D), (qc, kc, vc))
    qc, kc = rot_embed_reference(qc, freqs), rot_embed_reference(kc, freqs)
    ck, cv = cache_k.clone(), cache_v.clone()
    ck[:B, start:start + 1] = kc
    cv[:B, start:start + 1] = vc
    want = attention.sdpa_reference(qc.transpose(1, 2), ck[:B, :start + 1].transpose(1, 2), cv[:B, :start + 1].transpose(1, 2))
    compare.assert_close_attention(y.view(B, 1, Hq, D).transpose(1, 2), want)


def test_keyword_extras_and_non_default_stream(ext, device):
    case = inputs.config2().to(device)
    ref = attention.sdpa_reference(case.q.cpu(), case.k.cpu(), case.v.cpu(), case.seq_lens.cpu())
    s = torch.cuda.Stream(device)
    s.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(s):
        out = torch.empty_like(case.q)
        ret = ext.flash_attention_decode(case.q, case.k, case.v, seq_lens=case.seq_lens, out=out)
        assert ret.data_ptr() == out.data_ptr()
        o, lse = ext.flash_attention_decode_partial(case.q, case.k, case.v, seq_lens=case.seq_lens)
        merged = ext.lse_merge(o.unsqueeze(0), lse.unsqueeze(0))
    s.synchronize()
    compare.assert_close_attention(out, ref)
    compare.assert_close_attention(merged, ref)
    with torch.cuda.stream(s):
        assert ext.flash_decode_status(case.q) == 0


def test_rms_norm_and_rot_embed_call_forms(ext, device):
    x, w, eps, qkv = inputs.config4(B=1, S=64)
    got = ext.rms_norm(x.to(device), w.to(device), eps)
    assert compare.max_bf16_ulp(got, rms_norm_reference(x, w, eps)) <= 1
    freq = freqs_cis_reference(64, 64, **inputs.ROPE_CONFIG4)
    q = qkv[..., : 32 * 64].view(1, 64, 32, 64)
    got = ext.rot_embed(q.to(device), freq.to(device))
    assert torch.equal(got.cpu(), rot_embed_reference(q, freq))


def test_errors_are_runtime_errors(ext, device):
    q = torch.zeros(1, 8, 1, 96, dtype=torch.bfloat16, device=device)
    k = torch.zeros(1, 2, 4, 96, dtype=torch.bfloat16, device=device)
    with pytest.raises(RuntimeError, match="Unsupported head size"):   # custom_kernels.cu:318 wording
        ext.flash_attention_decode(q, k, k)
    q = torch.zeros(1, 34, 1, 64, dtype=torch.bfloat16, device=device)
    k = torch.zeros(1, 2, 4, 64, dtype=torch.bfloat16, device=device)
    with pytest.raises(RuntimeError, match="Unsupported QKV head ratio"):  # custom_kernels.cu:290,313
        ext.flash_attention_decode(q, k, k)
    with pytest.raises(RuntimeError, match="bfloat16"):
        ext.rms_norm(torch.zeros(1, 1, 8, device=device), torch.zeros(8, device=device), 1e-5)


def test_fused_elementwise_call_forms(ext, device):
    """add_rms_norm and silu_mul on [B, T, *] tensors, silu_mul on the two halves of one GEMM result."""
    from oracle.rms_norm import add_rms_norm_reference, silu_mul_reference

    g = torch.Generator().manual_seed(5)
    x = torch.randn(4, 3, 256, generator=g).bfloat16().to(device)
    r = torch.randn(4, 3, 256, generator=g).bfloat16().to(device)
    w = torch.randn(256, generator=g).bfloat16().to(device)
    s, h = ext.add_rms_norm(x, r, w, 1e-5)
    s_want, h_want = add_rms_norm_reference(x, r, w, 1e-5)
    assert s.shape == x.shape and torch.equal(s.cpu(), s_want)
    assert compare.max_bf16_ulp(h, h_want) <= 1
    gu = torch.randn(4, 3, 512, generator=g).bfloat16().to(device)
    got = ext.silu_mul(gu[..., :256], gu[..., 256:])
    assert got.shape == (4, 3, 256) and got.is_contiguous()
    assert compare.max_bf16_ulp(got, silu_mul_reference(gu[..., :256], gu[..., 256:])) <= 1
    with pytest.raises(RuntimeError):
        ext.silu_mul(gu[..., :256], gu[..., 250:])


def test_greedy_step_matches_torch_argmax_and_keeps_the_books(ext, device):
    """model.py:370-381 as one call: argmax (first index on ties), token into the output and the next input,
    per-sequence counters advanced."""
    g = torch.Generator().manual_seed(11)
    B, V, G = 7, 128256, 5
    logits = (torch.randn(B, V, generator=g) * 3).bfloat16()
    logits[1, 77] = logits[1].max()            # a tie further left than the maximum's first place?
    logits[2, :] = 0.5                         # all equal: index 0
    logits[3, V - 1] = 100.0                   # the last element, reached by the scalar tail when V % 8 != 0
    logits[4, 12345] = float("nan")            # torch.argmax treats NaN as the maximum
    want = logits.float().argmax(dim=-1)
    d = logits.to(device)
    out = torch.full((B, G), -1, dtype=torch.int64, device=device)
    steps = torch.tensor([0, 1, 2, 3, 4, 5, 0], dtype=torch.int64, device=device)   # row 5: output already full
    cur = torch.zeros(B, dtype=torch.int64, device=device)
    pos = torch.arange(B, dtype=torch.int32, device=device)
    lens = pos + 1
    ext.greedy_step(d, out, steps, cur, pos, lens)
    assert torch.equal(cur.cpu(), want)
    for b in range(B):
        s0 = [0, 1, 2, 3, 4, 5, 0][b]
        row = out[b].cpu()
        if s0 < G:
            assert int(row[s0]) == int(want[b]) and int((row != -1).sum()) == 1
        else:
            assert bool((row == -1).all())
    assert steps.cpu().tolist() == [1, 2, 3, 4, 5, 6, 1]
    assert pos.cpu().tolist() == list(range(1, B + 1)) and lens.cpu().tolist() == list(range(2, B + 2))
    # a strided view (rows of a wider buffer, vocabulary not a multiple of 8, rows not 16-byte aligned)
    wide = (torch.randn(3, 1003, generator=g)).bfloat16().to(device)
    view = wide[:, 1:1000]
    out2 = torch.zeros(3, 1, dtype=torch.int64, device=device)
    st2 = torch.zeros(3, dtype=torch.int64, device=device)
    cur2 = torch.zeros(3, dtype=torch.int64, device=device)
    ext.greedy_step(view, out2, st2, cur2, torch.zeros(3, dtype=torch.int32, device=device),
                    torch.zeros(3, dtype=torch.int32, device=device))
    assert torch.equal(cur2.cpu(), view.float().argmax(dim=-1).cpu())
