// Log-sum-exp merge of per-shard attention results (KV sequence sharded across GPUs).
//
// Each shard p delivers, per query row r, a softmax-normalised fp32 output o[p, r, :] and the
// natural-log sum-exp lse[p, r] of its scaled scores.  The exact attention over the union is
//     out[r, :] = sum_p exp(lse[p, r] - L) * o[p, r, :],   L = log sum_p exp(lse[p, r]).
// This is what the reference's combine kernel is meant to do for its 64-token steps
// (custom_kernels/custom_kernels.cu:198-222), here with the weights indexed per shard and
// with fp32 partial outputs.  One warp per row; a shard with lse = -inf (no tokens) has weight 0.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include "bf16x8.cuh"
#include "host_common.h"
#include "warp_reduce.cuh"

namespace l3ci {
namespace {

constexpr int kMergeBlock = 128;

__global__ void __launch_bounds__(kMergeBlock)
lse_merge_kernel(const float* __restrict__ o, const float* __restrict__ lse, __nv_bfloat16* __restrict__ out,
                 int parts, long long rows, int Hq, int D, long long o_sb, long long o_sh) {
  const long long row = (long long)blockIdx.x * (kMergeBlock / kWarp) + threadIdx.x / kWarp;
  const int lane = threadIdx.x % kWarp;
  if (row >= rows) return;
  float M = -INFINITY;
  for (int p = 0; p < parts; ++p) M = fmaxf(M, __ldg(lse + p * rows + row));
  const float Mu = M == -INFINITY ? 0.f : M;
  float L = 0.f;
  for (int p = 0; p < parts; ++p) L += __expf(__ldg(lse + p * rows + row) - Mu);
  const float invL = L > 0.f ? 1.f / L : 0.f;
  const long long b = row / Hq;
  const int h = (int)(row % Hq);
  __nv_bfloat16* orow = out + b * o_sb + h * o_sh;
  for (int d = lane * 2; d < D; d += 2 * kWarp) {
    float ax = 0.f, ay = 0.f;
    for (int p = 0; p < parts; ++p) {
      const float w = __expf(__ldg(lse + p * rows + row) - Mu) * invL;
      const float2 v = __ldg(reinterpret_cast<const float2*>(o + (p * rows + row) * D + d));
      ax = fmaf(v.x, w, ax);
      ay = fmaf(v.y, w, ay);
    }
    *reinterpret_cast<uint32_t*>(orow + d) = pack_bf16x2(ax, ay);
  }
}

}  // namespace
}  // namespace l3ci

extern "C" int l3ci_lse_merge(const float* o, const float* lse, void* out, int32_t parts, int32_t B,
                              int32_t Hq, int32_t D, int64_t o_sb, int64_t o_sh, l3ci_stream_t stream_) {
  using namespace l3ci;
  clear_error();
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (parts <= 0 || B < 0 || Hq <= 0 || D <= 0) return fail(L3CI_ERR_INVALID, "lse_merge: bad size");
  if (B == 0) return L3CI_OK;
  if (!o || !lse || !out) return fail(L3CI_ERR_INVALID, "lse_merge: null pointer");
  if (D % 2) return fail(L3CI_ERR_UNSUPPORTED, "lse_merge: head size %d is odd", D);
  if ((reinterpret_cast<uintptr_t>(o) & 7) || (reinterpret_cast<uintptr_t>(out) & 3) || (o_sb & 1) || (o_sh & 1))
    return fail(L3CI_ERR_ALIGNMENT, "lse_merge: rows must start on 8 bytes (fp32) / 4 bytes (bf16)");
  const long long rows = (long long)B * Hq;
  const long long ctas = (rows + kMergeBlock / kWarp - 1) / (kMergeBlock / kWarp);
  lse_merge_kernel<<<(unsigned)ctas, kMergeBlock, 0, stream>>>(o, lse, static_cast<__nv_bfloat16*>(out), parts,
                                                               rows, Hq, D, o_sb, o_sh);
  L3CI_CHECK_LAUNCH("lse_merge_kernel");
  return L3CI_OK;
}
