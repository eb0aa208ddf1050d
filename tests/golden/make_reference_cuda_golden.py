"""Generates tests/golden/reference_cuda_vectors.pt by RUNNING the reference's own CUDA kernels on a GPU.

    python tests/golden/make_reference_cuda_golden.py <output .pt> [<summary .json>]

Needs a CUDA device and oracle/_ref/reference_kernels_sm100.so (the reference's unmodified
custom_kernels/custom_kernels.cu + main.cpp compiled for sm_100 by oracle/build_ref.py).  The reference has no
CPU implementation, no test and no vector for RMSNorm and for the rotary rotation; its CUDA kernels
(custom_kernels/custom_kernels.cu:340-367, 391-416) are its only statement of them, so their outputs on seeded
inputs are the pin for oracle/rms_norm.py and oracle/rope.py.  The produced file is committed; the tests never
need the reference or this script again.

Held in the file (inputs are regenerated from their seeds by oracle.inputs):
  rms/<name>      whole output of `rms_norm` for the small shapes of inputs.RMS_GOLDEN_CASES
  rms/c4_rows     every 64th row of the output on configuration 4 (4096 x 2048), in row order
  rope/<name>     whole output of `rot_embed` for inputs.ROPE_GOLDEN_CASES (table: theta 5e5, scaling factor 8)
  rope/c4_q, c4_k every 64th position of the rotated q / k of configuration 4 (table: scaling factor 32)
  rope/c4_q_diff_idx, _diff_val (and c4_k)  flat indices and values of ALL elements of the full output that differ
                  from the unfused restatement oracle.rope.rot_embed_reference (a few dozen), so that a test can
                  rebuild the whole 17 MB output from the restatement and check another restatement against it
The reference's `flash_attention_decode` output is NOT held: it is not an oracle (its combine kernel weighs
every split with the statistics of split 0, custom_kernels.cu:184,201,209); the summary only records how far
it is from softmax attention on N(0,1) inputs.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))
from oracle import attention, build_ref, compare, inputs  # noqa: E402
from oracle.rms_norm import rms_norm_reference, rms_norm_reference_rounding  # noqa: E402
from oracle.rope import freqs_cis_reference, rot_embed_reference, rot_embed_reference_fma  # noqa: E402

SMALL_ROPE_TABLE = dict(theta=500000.0, use_scaled=True, scale_factor=8)


def ulp_stats(a: torch.Tensor, b: torch.Tensor) -> dict:
    d = compare.bf16_ulp_distance(a.cpu(), b.cpu())
    return {"max_ulp": int(d.max()), "frac_exact": float((d == 0).float().mean()), "frac_gt1": float((d > 1).float().mean())}


def main() -> None:
    out_path = Path(sys.argv[1])
    ref = build_ref.load()
    if ref is None:
        raise SystemExit("oracle/_ref/reference_kernels_sm100.so is missing: run oracle/build_ref.py where the "
                         "reference checkout is")
    dev = torch.device("cuda", 0)
    vec, summary = {}, {}

    # ---- RMSNorm -------------------------------------------------------------------------------------------
    for name, (B, S, E, seed) in inputs.RMS_GOLDEN_CASES.items():
        x, w = inputs.rms_case(B, S, E, seed)
        got = ref.rms_norm(x.to(dev), w.to(dev), 1e-5).cpu()
        vec["rms/" + name] = got
        summary["rms/" + name] = {"vs_one_rounding_oracle": ulp_stats(got, rms_norm_reference(x, w, 1e-5)),
                                  "vs_three_rounding_emulation": ulp_stats(got, rms_norm_reference_rounding(x, w, 1e-5))}
    x, w, eps, qkv = inputs.config4(seed=42)
    got = ref.rms_norm(x.to(dev), w.to(dev), eps).cpu()
    vec["rms/c4_rows"] = got.view(-1, x.shape[-1])[:: inputs.C4_GOLDEN_ROW_STEP].clone()
    summary["rms/c4"] = {"vs_one_rounding_oracle": ulp_stats(got, rms_norm_reference(x, w, eps)),
                         "vs_three_rounding_emulation": ulp_stats(got, rms_norm_reference_rounding(x, w, eps))}

    # ---- rotary rotation -----------------------------------------------------------------------------------
    for name, (B, S, H, D, seed, extra) in inputs.ROPE_GOLDEN_CASES.items():
        xr = inputs.rope_case(B, S, H, D, seed, extra)
        freq = freqs_cis_reference(D, S, **SMALL_ROPE_TABLE)
        got = ref.rot_embed(xr.to(dev), freq.to(dev)).cpu().contiguous()
        vec["rope/" + name] = got
        summary["rope/" + name] = {"vs_unfused_oracle": ulp_stats(got, rot_embed_reference(xr, freq))}
    Hq, Hkv, D = 32, 8, 64
    B, S = qkv.shape[:2]
    freq = freqs_cis_reference(D, S, **inputs.ROPE_CONFIG4)
    dq = qkv.to(dev)
    q_in = dq[..., : Hq * D].view(B, S, Hq, D)
    k_in = dq[..., Hq * D: (Hq + Hkv) * D].view(B, S, Hkv, D)
    for name, t in (("c4_q", q_in), ("c4_k", k_in)):
        got = ref.rot_embed(t, freq.to(dev)).cpu().contiguous()
        vec["rope/" + name] = got[:, :: inputs.C4_GOLDEN_ROW_STEP].clone()
        unfused = rot_embed_reference(t.cpu(), freq)
        diff = (got.view(torch.int16) != unfused.view(torch.int16)).flatten().nonzero().flatten()
        vec["rope/" + name + "_diff_idx"] = diff.to(torch.int32)
        vec["rope/" + name + "_diff_val"] = got.flatten()[diff].clone()
        summary["rope/" + name] = {"vs_unfused_oracle": ulp_stats(got, unfused)}
        for form in ("aa", "ab", "ba", "bb"):
            summary["rope/" + name]["vs_fma_form_" + form] = ulp_stats(got, rot_embed_reference_fma(t.cpu(), freq, form))

    # ---- attention: recorded distance from softmax attention, nothing held -----------------------------------
    for name, case in (("c1_normal", inputs.config1()), ("c1_uniform01", inputs.decode_case(1, 32, 8, 64, 256, 42, dist="uniform")),
                       ("s64_normal", inputs.decode_case(1, 32, 8, 64, 64, 42))):
        got = ref.flash_attention_decode(case.q.to(dev), case.k.to(dev), case.v.to(dev)).float().cpu()
        want = attention.sdpa_reference(case.q, case.k, case.v)
        err = (got - want).abs()
        summary["attention/" + name] = {"max_abs_err_vs_sdpa_fp32": float(err.max()),
                                        "within_2e-2_1e-2": bool((err <= 2e-2 + 1e-2 * want.abs()).all())}
    torch.cuda.synchronize()

    vec["meta"] = {"gpu": torch.cuda.get_device_name(0), "torch": str(torch.__version__),
                   "source": "custom_kernels/custom_kernels.cu + main.cpp of the reference, unmodified, compiled for sm_100"}
    torch.save(vec, out_path)
    print(json.dumps(summary, indent=1))
    if len(sys.argv) > 2:
        Path(sys.argv[2]).write_text(json.dumps(summary, indent=1))


if __name__ == "__main__":
    main()
