"""CPU oracle for the decode hot path.  TEST INFRASTRUCTURE, not product code.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / `--impl reference` legs may import
this package, and only as the checker or as the timed CPU baseline.  Nothing under the product
package (llama3-custom-inference_b200/) imports it, and it never runs on the GPU.

What it restates, and how each part is pinned:

  attention.py   The reference's own PyTorch attention path
                 `F.scaled_dot_product_attention(q, k, v, enable_gqa=True)` (model.py:115-116,
                 benchmark_kernel.py:27-28) evaluated in fp32, plus a boolean length mask for ragged
                 batches, plus an independent float64 numpy restatement.  PINNED: tests/golden holds
                 outputs of that very call made in the reference's dtype (bf16) by
                 tests/golden/make_golden.py.  The reference's CUDA kernels are NOT the oracle: their
                 combine step indexes every split with blockIdx.z == 0
                 (custom_kernels/custom_kernels.cu:184,201,209) and so does not compute softmax
                 attention for more than 64 tokens.
  rope.py        `precompute_freqs_cis` / `apply_scaling` (model.py:27-60) with the scaling constants
                 as parameters.  PINNED: golden rows produced by importing the reference's model.py.
                 The rotation restates custom_rot_embed_kernel (custom_kernels/custom_kernels.cu:400-412)
                 with the multiply-add contraction the compiler gives it (x' = fma(x, c, -rn(y*s)),
                 y' = fma(x, s, rn(y*c))).  PINNED bit for bit: tests/golden/reference_cuda_vectors.pt
                 holds outputs of the reference's own kernel, compiled for sm_100 by build_ref.py and run
                 on a B200 by tests/golden/make_reference_cuda_golden.py.
  rms_norm.py    Restates custom_rms_norm_kernel (custom_kernels/custom_kernels.cu:343-365) twice: with
                 its three bf16 roundings (`rms_norm_reference_rounding`, PINNED bit for bit by the same
                 fixture) and in fp32 with one final rounding (`rms_norm_reference`, what the product
                 computes: within 2 bf16 ulp of the reference kernel, checked against the fixture too).
  sampling.py    `sample_top_p` and the temperature softmax in front of it (model.py:400-423,
                 model.py:368-369).  PINNED: draws of the reference's own function on seeded
                 generators, made by tests/golden/make_golden.py.
  build_ref.py   Compiles the reference's custom_kernels.cu + main.cpp, where they lie in a checkout of
                 the reference, into _ref/reference_kernels_sm100.so (not tracked): the source of the
                 fixture above and the same-box comparator of bench.py.
  inputs.py      Seeded synthetic inputs with the shapes and distributions of the five benchmark
                 configurations.
  compare.py     bf16 ulp distance and absolute/relative tolerance checks.
"""
