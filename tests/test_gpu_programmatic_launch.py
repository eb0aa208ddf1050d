"""Programmatic stream serialization (l3ci_set_programmatic_launch): the kernels launched that way give the same
bits as plain launches, back to back on one stream where each reads what the one before wrote, eagerly and from a
captured CUDA graph."""
import pytest
import torch

from oracle import inputs
from oracle.rope import freqs_cis_reference

pytestmark = pytest.mark.gpu


def _step(capi, x, w, qkv_w, freq, ck, cv, pos, n_head, n_kv_head):
    """A chain of dependent launches: norm -> (a projection by torch) -> rotary + cache write at position `pos` ->
    decode attention over pos + 1 tokens -> SiLU * mul on the result -> norm again.  Caches are [B, S, Hkv, D]."""
    h = capi.rms_norm(x, w, 1e-5)
    qkv = (h @ qkv_w).view(x.shape[0], 1, -1)
    q = capi.rot_embed_kv_cache(qkv, freq, ck, cv, pos, n_head, n_kv_head)
    o = capi.flash_attention_decode(q.transpose(1, 2), ck[:, :pos + 1].transpose(1, 2), cv[:, :pos + 1].transpose(1, 2))
    flat = o.transpose(1, 2).reshape(x.shape[0], -1)
    g = capi.silu_mul(flat, flat)
    return capi.rms_norm(g, w[: g.shape[-1]].contiguous(), 1e-5)


@pytest.mark.parametrize("graph", [False, True])
def test_same_bits_as_plain_launches(capi, device, graph):
    torch.manual_seed(3)
    B, n_head, n_kv_head, D, S = 4, 8, 2, 64, 700
    E = n_head * D
    x = torch.randn(B, E, device=device).bfloat16()
    w = (1 + 0.1 * torch.randn(E, device=device)).bfloat16()
    qkv_w = (torch.randn(E, (n_head + 2 * n_kv_head) * D, device=device) / E ** 0.5).bfloat16()
    pos = S - 1
    freq = freqs_cis_reference(D, S, **inputs.ROPE_CONFIG4)[pos:pos + 1].contiguous().to(device)
    results = {}
    for on in (False, True):
        ck = torch.randn(B, S, n_kv_head, D, device=device, generator=torch.Generator(device=device).manual_seed(5)).bfloat16()
        cv = torch.randn(B, S, n_kv_head, D, device=device, generator=torch.Generator(device=device).manual_seed(6)).bfloat16()
        with capi.programmatic_launch(on):
            if graph:
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    _step(capi, x, w, qkv_w, freq, ck, cv, pos, n_head, n_kv_head)      # warm-up outside capture
                torch.cuda.current_stream().wait_stream(s)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    out = _step(capi, x, w, qkv_w, freq, ck, cv, pos, n_head, n_kv_head)
                for _ in range(3):
                    g.replay()
            else:
                for _ in range(3):
                    out = _step(capi, x, w, qkv_w, freq, ck, cv, pos, n_head, n_kv_head)
            torch.cuda.synchronize()
        results[on] = (out.clone(), ck.clone(), cv.clone())
    for a, b in zip(results[False], results[True]):
        assert torch.equal(a, b)
    assert bool(torch.isfinite(results[True][0].float()).all())
