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
                 The rotation itself restates custom_rot_embed_kernel
                 (custom_kernels/custom_kernels.cu:400-412) in unfused fp32: PARITY UNPINNED, the
                 reference has no CPU implementation and no test vector for it.
  rms_norm.py    Restates custom_rms_norm_kernel (custom_kernels/custom_kernels.cu:343-365) in fp32
                 with one final rounding: PARITY UNPINNED for the same reason (and the reference kernel
                 itself rounds three times in bf16, so it is within 2 bf16 ulp of this, not equal).
  inputs.py      Seeded synthetic inputs with the shapes and distributions of the five benchmark
                 configurations.
  compare.py     bf16 ulp distance and absolute/relative tolerance checks.
"""
