"""Generates tests/golden/reference_vectors.pt by RUNNING the reference's own Python code.

Needs a checkout of the reference (its path as argv[1]); the produced file is committed, so the tests
never read the checkout.  What is executed from the reference:

  * model.precompute_freqs_cis / model.apply_scaling (model.py:27-60), imported from the reference's
    model.py with its compiled extension replaced by an empty stub module (model.py:23 imports it at
    module level; neither function touches it);
  * model.sample_top_p (model.py:400-423) on seeded probability rows under torch.manual_seed;
  * the attention call of model.py:115-116 / benchmark_kernel.py:27-28,
    `sdpa_kernel(SDPBackend.FLASH_ATTENTION)` + `F.scaled_dot_product_attention(q, k, v, enable_gqa=True)`,
    on the bf16 CPU tensors of oracle.inputs (the reference has no other CPU-runnable attention path).

The reference ships no golden vectors or tests of its own, so these outputs are the pin.
"""
from __future__ import annotations

import hashlib
import sys
import types
from pathlib import Path

import torch
import torch.nn.functional as F
from torch.nn.attention import SDPBackend, sdpa_kernel

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))
from oracle import inputs  # noqa: E402


# name -> (B, Hq, Hkv, D, T, seed) of oracle.inputs.prefill_case
# name -> (rows, vocab, scale of the N(0,1) logits, top_p, seed) for the reference's sample_top_p; TOP_P_DRAWS calls each
TOP_P_CASES = {"flat": (3, 500, 1.0, 0.9, 11), "peaked": (2, 2000, 6.0, 0.9, 12), "half": (4, 300, 2.0, 0.5, 13)}
TOP_P_DRAWS = 64

PREFILL_CASES = {"d64_r4_t40": (2, 8, 2, 64, 40, 21), "d128_r2_t150": (1, 4, 2, 128, 150, 22)}


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def import_reference_model(ref: Path):
    stub_pkg = types.ModuleType("custom_kernels")
    stub_ext = types.ModuleType("custom_kernels.custom_kernels_extension")
    stub_pkg.custom_kernels_extension = stub_ext
    sys.modules["custom_kernels"] = stub_pkg
    sys.modules["custom_kernels.custom_kernels_extension"] = stub_ext
    sys.path.insert(0, str(ref))
    import model  # the reference's model.py

    return model


def reference_attention(case) -> torch.Tensor:
    with sdpa_kernel(SDPBackend.FLASH_ATTENTION):
        return F.scaled_dot_product_attention(case.q, case.k, case.v, enable_gqa=True)


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path of the reference checkout>")
    ref = Path(sys.argv[1])
    model = import_reference_model(ref)
    out = {}
    rows = [0, 1, 2, 3, 17, 127, 511, 2047, 8191, 16383]
    out["freq_rows"] = torch.tensor(rows)
    for dim in (64, 128):
        base = 1.0 / (500000.0 ** (torch.arange(0, dim, 2)[: dim // 2].float() / dim))
        out[f"apply_scaling_d{dim}"] = model.apply_scaling(base).clone()
        table = model.precompute_freqs_cis(dim, 16384, 500000.0, True)
        out[f"freqs_cis_scaled_d{dim}"] = table[rows].clone()
        table = model.precompute_freqs_cis(dim, 16384, 10000.0, False)
        out[f"freqs_cis_plain_d{dim}"] = table[rows].clone()
        out[f"freqs_cis_scaled_d{dim}_sha256_2048"] = sha(model.precompute_freqs_cis(dim, 2048, 500000.0, True))
    cases = {
        "c1": inputs.config1(),
        "d128_r4_s300": inputs.decode_case(2, 8, 2, 128, 300, seed=7),
        "d64_r1_s65": inputs.decode_case(2, 4, 4, 64, 65, seed=8),
        "d128_r8_s1000": inputs.decode_case(1, 8, 1, 128, 1000, seed=9),
        "d128_r3_s130_uniform01": inputs.decode_case(1, 6, 2, 128, 130, seed=10, dist="uniform"),
    }
    for name, case in cases.items():
        out[f"sdpa_{name}_bf16"] = reference_attention(case).contiguous()
        out[f"sdpa_{name}_inputs_sha256"] = sha(case.q) + sha(case.k) + sha(case.v)
    # the prefill call of model.py:114-116, same backend selection, on bf16 CPU tensors
    for name, shape in PREFILL_CASES.items():
        q, k, v = inputs.prefill_case(*shape)
        with sdpa_kernel(SDPBackend.FLASH_ATTENTION):
            out[f"prefill_{name}_bf16"] = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True).contiguous()
        out[f"prefill_{name}_inputs_sha256"] = sha(q) + sha(k) + sha(v)
    # the reference's nucleus sampler (model.py:400-423) on seeded distributions, under a known RNG state
    for name, (rows, vocab, scale, p, seed) in TOP_P_CASES.items():
        g = torch.Generator().manual_seed(seed)
        probs = torch.softmax(torch.randn(rows, vocab, generator=g) * scale, dim=-1)
        torch.manual_seed(seed)
        draws = torch.cat([model.sample_top_p(probs.clone(), p) for _ in range(TOP_P_DRAWS)], dim=1)
        out[f"top_p_{name}_draws"] = draws.clone()
    out["torch_version"] = str(torch.__version__)
    dst = Path(__file__).with_name("reference_vectors.pt")
    torch.save(out, dst)
    print("wrote", dst, dst.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
