// RMSNorm for sm_100a: each row is read from HBM exactly once, held in registers as 16-byte
// bf16 vectors, reduced in fp32 and written once.
//
// Replaces custom_rms_norm_kernel / rms_norm (custom_kernels/custom_kernels.cu:340-389),
// which walks every row twice with 2-byte loads and rounds three times in bf16.  The
// arithmetic here is fp32 with one final rounding:
//     out = bf16( (float(x) * rsqrt(sum(x^2)/E + eps)) * float(w) )
//
// Work split: a row of up to 2048 elements belongs to one warp (8 vectors per lane, no
// shared memory, no barrier); longer rows get one CTA of 64..1024 threads.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "bf16x8.cuh"
#include "host_common.h"
#include "warp_reduce.cuh"

namespace l3ci {
namespace {

template <int TPR>
struct RmsCfg {
  static constexpr int kBlock = TPR <= 32 ? 128 : TPR;
  static constexpr int kRowsPerCta = kBlock / TPR;
};

template <int TPR, int VPT>
__global__ void __launch_bounds__(RmsCfg<TPR>::kBlock)
rms_norm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                __nv_bfloat16* __restrict__ out, long long rows, int nvec, long long x_stride,
                long long out_stride, float embed_f, float eps) {
  constexpr int kRows = RmsCfg<TPR>::kRowsPerCta;
  __shared__ float red[32];
  const int t = threadIdx.x % TPR;
  const long long row = (long long)blockIdx.x * kRows + threadIdx.x / TPR;
  const bool row_ok = row < rows;
  const __nv_bfloat16* xr = x + (row_ok ? row : 0) * x_stride;

  uint4 v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = t + i * TPR;
    if (row_ok && idx < nvec) {
      v[i] = ld_stream16(xr + (long long)idx * kVecElems);
    } else {
      v[i] = make_uint4(0, 0, 0, 0);
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    float f[8];
    unpack8(v[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
  }
  if constexpr (TPR <= 32) {
    ss = group_sum<TPR>(ss);
  } else {
    ss = cta_sum(ss, red, TPR / kWarp);
  }
  const float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, embed_f), eps));
  if (!row_ok) return;
  __nv_bfloat16* orow = out + row * out_stride;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = t + i * TPR;
    if (idx < nvec) {
      const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w) + idx);
      float f[8], g[8];
      unpack8(v[i], f);
      unpack8(wv, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __fmul_rn(__fmul_rn(f[j], inv), g[j]);
      st_stream16(orow + (long long)idx * kVecElems, pack8(f));
    }
  }
}

template <int TPR, int VPT>
int launch(const void* x, const void* w, void* out, long long rows, int nvec, long long xs,
           long long os, float eps, cudaStream_t stream) {
  constexpr int kRows = RmsCfg<TPR>::kRowsPerCta;
  const long long ctas = (rows + kRows - 1) / kRows;
  if (ctas > 0x7fffffffLL) return fail(L3CI_ERR_INVALID, "rms_norm: too many rows (%lld)", rows);
  rms_norm_kernel<TPR, VPT><<<(unsigned)ctas, RmsCfg<TPR>::kBlock, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<__nv_bfloat16*>(out), rows, nvec, xs, os, (float)(nvec * kVecElems), eps);
  L3CI_CHECK_LAUNCH("rms_norm_kernel");
  return L3CI_OK;
}

template <int TPR>
int launch_vpt(int vpt, const void* x, const void* w, void* out, long long rows, int nvec,
               long long xs, long long os, float eps, cudaStream_t stream) {
  if (vpt <= 1) return launch<TPR, 1>(x, w, out, rows, nvec, xs, os, eps, stream);
  if (vpt <= 2) return launch<TPR, 2>(x, w, out, rows, nvec, xs, os, eps, stream);
  if (vpt <= 4) return launch<TPR, 4>(x, w, out, rows, nvec, xs, os, eps, stream);
  return launch<TPR, 8>(x, w, out, rows, nvec, xs, os, eps, stream);
}

}  // namespace
}  // namespace l3ci

extern "C" int l3ci_rms_norm(const void* x, const void* weight, void* out, int64_t rows,
                             int64_t embed, int64_t x_row_stride, int64_t out_row_stride,
                             float eps, l3ci_stream_t stream_) {
  using namespace l3ci;
  clear_error();
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (rows < 0 || embed <= 0) return fail(L3CI_ERR_INVALID, "rms_norm: rows=%lld embed=%lld", (long long)rows, (long long)embed);
  if (rows == 0) return L3CI_OK;
  if (!x || !weight || !out) return fail(L3CI_ERR_INVALID, "rms_norm: null pointer");
  if (embed % kVecElems != 0 || embed > 65536)
    return fail(L3CI_ERR_UNSUPPORTED, "rms_norm: embed=%lld must be a multiple of 8 and <= 65536", (long long)embed);
  if (!aligned16(x) || !aligned16(weight) || !aligned16(out) || x_row_stride % kVecElems ||
      out_row_stride % kVecElems)
    return fail(L3CI_ERR_ALIGNMENT, "rms_norm: rows must start on 16 bytes");
  const int nvec = (int)(embed / kVecElems);
  // Smallest thread group whose lanes hold the row in <= 8 vectors each.
  int tpr = 32;
  while (tpr * 8 < nvec) tpr *= 2;
  const int vpt = (nvec + tpr - 1) / tpr;
  switch (tpr) {
    case 32: return launch_vpt<32>(vpt, x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream);
    case 64: return launch_vpt<64>(vpt, x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream);
    case 128: return launch_vpt<128>(vpt, x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream);
    case 256: return launch_vpt<256>(vpt, x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream);
    case 512: return launch_vpt<512>(vpt, x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream);
    default: return launch_vpt<1024>(vpt, x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream);
  }
}
