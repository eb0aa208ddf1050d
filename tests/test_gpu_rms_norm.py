"""RMSNorm kernel through the C ABI against the fp32 oracle: at most 1 bf16 ulp; and against the outputs of the
reference's own CUDA kernel, which rounds three times in bf16: at most 2 bf16 ulp."""
import pytest
import torch

from oracle import compare, inputs
from oracle.rms_norm import add_rms_norm_reference, rms_norm_reference, silu_mul_reference

pytestmark = pytest.mark.gpu
MAX_ULP = 1  # stated tolerance for RMSNorm


def _check(capi, x, w, eps):
    got = capi.rms_norm(x, w, eps)
    torch.cuda.synchronize()
    want = rms_norm_reference(x, w, eps)
    assert got.shape == x.shape and got.dtype == torch.bfloat16
    ulp = compare.bf16_ulp_distance(got.cpu(), want)
    assert int(ulp.max()) <= MAX_ULP, f"max ulp {int(ulp.max())}, {(ulp > MAX_ULP).float().mean().item():.2%} beyond tolerance"
    return float((ulp > 0).float().mean())


def test_config4_token_batch(capi, device):
    x, w, eps, _ = inputs.config4()
    frac = _check(capi, x.to(device), w.to(device), eps)
    assert frac < 0.05  # almost every element is the identical bf16 value


@pytest.mark.parametrize("rows,embed", [(1, 2048), (64, 2048), (7, 8), (5, 64), (3, 256), (33, 1000), (9, 4096),
                                        (4, 8192), (3, 16384), (2, 5120), (130, 2056), (2, 65536),
                                        # many rows: the warp-per-row persistent kernel, 1, 2, 4 and 8 vectors per lane,
                                        # full and ragged last vectors, more rows than one pass of the grid
                                        (3000, 64), (2500, 512), (2400, 1000), (2368, 2048), (20011, 8), (9000, 776),
                                        (2400, 2056)])
def test_shapes(capi, device, rows, embed):
    g = torch.Generator().manual_seed(rows * 131 + embed)
    x = (torch.randn(rows, 1, embed, generator=g) * 3).bfloat16().to(device)
    w = (1 + 0.1 * torch.randn(embed, generator=g)).bfloat16().to(device)
    _check(capi, x, w, 1e-5)


def test_zero_row_and_large_values(capi, device):
    x = torch.zeros(4, 1, 2048, dtype=torch.bfloat16, device=device)
    x[1] = 1e4
    x[2, 0, ::2] = -3e-3
    w = torch.ones(2048, dtype=torch.bfloat16, device=device)
    _check(capi, x, w, 1e-5)
    _check(capi, x, w, 1e-6)


def test_strided_rows_and_untouched_padding(capi, device):
    rows, embed, pitch = 10, 512, 640
    g = torch.Generator().manual_seed(1)
    xbuf = torch.randn(rows, pitch, generator=g).bfloat16().to(device)
    w = torch.randn(embed, generator=g).bfloat16().to(device)
    obuf = torch.full((rows, pitch), 7.0, dtype=torch.bfloat16, device=device)
    st = capi.load().l3ci_rms_norm(xbuf.data_ptr(), w.data_ptr(), obuf.data_ptr(), rows, embed, pitch, pitch, 1e-5,
                                   torch.cuda.current_stream().cuda_stream)
    assert st == capi.OK
    torch.cuda.synchronize()
    want = rms_norm_reference(xbuf[:, :embed], w, 1e-5)
    assert compare.max_bf16_ulp(obuf[:, :embed].contiguous(), want) <= MAX_ULP
    assert (obuf[:, embed:] == 7.0).all()


def test_strided_rows_of_a_token_batch(capi, device):
    # enough rows for the warp-per-row kernel, rows 640 elements apart, padding must stay untouched
    rows, embed, pitch = 2500, 512, 640
    g = torch.Generator().manual_seed(2)
    xbuf = torch.randn(rows, pitch, generator=g).bfloat16().to(device)
    w = torch.randn(embed, generator=g).bfloat16().to(device)
    obuf = torch.full((rows, pitch), 7.0, dtype=torch.bfloat16, device=device)
    st = capi.load().l3ci_rms_norm(xbuf.data_ptr(), w.data_ptr(), obuf.data_ptr(), rows, embed, pitch, pitch, 1e-5,
                                   torch.cuda.current_stream().cuda_stream)
    assert st == capi.OK
    torch.cuda.synchronize()
    assert compare.max_bf16_ulp(obuf[:, :embed].contiguous(), rms_norm_reference(xbuf[:, :embed], w, 1e-5)) <= MAX_ULP
    assert (obuf[:, embed:] == 7.0).all()


def test_errors(capi, device):
    lib = capi.load()
    x = torch.zeros(2, 16, dtype=torch.bfloat16, device=device)
    assert lib.l3ci_rms_norm(x.data_ptr() + 2, x.data_ptr(), x.data_ptr(), 1, 8, 8, 8, 1e-5, None) == capi.ERR_ALIGNMENT
    assert lib.l3ci_rms_norm(x.data_ptr(), x.data_ptr(), x.data_ptr(), 1, 12, 12, 12, 1e-5, None) == capi.ERR_UNSUPPORTED


# ---- residual add fused into the norm, and the SwiGLU gate (the elementwise passes either side of the norm) ----

@pytest.mark.parametrize("rows,embed", [(64, 2048), (1, 2048), (7, 8), (33, 1000), (9, 4096), (3, 16384), (130, 2056),
                                        (8192, 2048), (2400, 512), (2500, 1000), (3000, 64)])
def test_add_rms_norm(capi, device, rows, embed):
    g = torch.Generator().manual_seed(rows * 17 + embed)
    x = (torch.randn(rows, embed, generator=g) * 2).bfloat16().to(device)
    r = (torch.randn(rows, embed, generator=g) * 3).bfloat16().to(device)
    w = (1 + 0.1 * torch.randn(embed, generator=g)).bfloat16().to(device)
    s, out = capi.add_rms_norm(x, r, w, 1e-5)
    torch.cuda.synchronize()
    s_want, out_want = add_rms_norm_reference(x, r, w, 1e-5)
    assert torch.equal(s.cpu().view(torch.int16), s_want.view(torch.int16))  # the sum is bit-exact
    assert compare.max_bf16_ulp(out, out_want) <= MAX_ULP
    # and the norm of the fused call is the plain kernel applied to that sum
    assert torch.equal(out, capi.rms_norm(s, w, 1e-5))


@pytest.mark.parametrize("rows,cols", [(64, 8192), (1, 8), (5, 1000), (3, 65536)])
def test_silu_mul(capi, device, rows, cols):
    g = torch.Generator().manual_seed(rows + cols)
    gu = (torch.randn(rows, 2 * cols, generator=g) * 4).bfloat16().to(device)
    gu[0, :8] = torch.tensor([0.0, -0.0, 30.0, -30.0, 100.0, -100.0, 1e-3, -1e-3], dtype=torch.bfloat16)
    gate, up = gu[:, :cols], gu[:, cols:]          # halves of one GEMM result: strided rows
    got = capi.silu_mul(gate, up)
    torch.cuda.synchronize()
    want = silu_mul_reference(gate, up)
    assert torch.isfinite(got.float()).all()
    assert compare.max_bf16_ulp(got, want) <= MAX_ULP
    assert float((compare.bf16_ulp_distance(got.cpu(), want) > 0).float().mean()) < 0.01
    assert torch.equal(got, capi.silu_mul(gate.contiguous(), up.contiguous()))


def test_fused_errors(capi, device):
    lib = capi.load()
    x = torch.zeros(2, 16, dtype=torch.bfloat16, device=device)
    p = x.data_ptr()
    assert lib.l3ci_add_rms_norm(p, None, p, p, p, 1, 8, 1e-5, None) == capi.ERR_INVALID
    assert lib.l3ci_add_rms_norm(p, p + 2, p, p, p, 1, 8, 1e-5, None) == capi.ERR_ALIGNMENT
    assert lib.l3ci_silu_mul(p, p, p, 1, 12, 12, 12, None) == capi.ERR_ALIGNMENT
    assert lib.l3ci_silu_mul(p, p, p, 0, 8, 8, 8, None) == capi.OK


@pytest.mark.parametrize("name", sorted(inputs.RMS_GOLDEN_CASES) + ["c4_rows"])
def test_within_two_ulp_of_the_reference_kernels_output(capi, device, ref_cuda, name):
    """The reference kernel rounds the inverse RMS, its product with the weight and the final product to bf16
    (custom_kernels/custom_kernels.cu:362,365); this kernel rounds once.  Measured on the held vectors: the two
    differ by at most 2 ulp, in under 1 % of the elements by more than 1."""
    if name == "c4_rows":
        x, w, eps, _ = inputs.config4(seed=42)
        got = capi.rms_norm(x.to(device), w.to(device), eps).view(-1, x.shape[-1])[:: inputs.C4_GOLDEN_ROW_STEP].contiguous()
    else:
        x, w = inputs.rms_case(*inputs.RMS_GOLDEN_CASES[name])
        got = capi.rms_norm(x.to(device), w.to(device), 1e-5)
    torch.cuda.synchronize()
    d = compare.bf16_ulp_distance(got.cpu(), ref_cuda["rms/" + name])
    assert int(d.max()) <= 2 and float((d > 1).float().mean()) < 0.01
