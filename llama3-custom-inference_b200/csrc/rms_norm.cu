// RMSNorm for sm_100a: each row is read from HBM exactly once, held in registers as 16-byte
// bf16 vectors, reduced in fp32 and written once.
//
// Replaces custom_rms_norm_kernel / rms_norm (custom_kernels/custom_kernels.cu:340-389),
// which walks every row twice with 2-byte loads and rounds three times in bf16.  The
// arithmetic here is fp32 with one final rounding:
//     out = bf16( (float(x) * rsqrt(sum(x^2)/E + eps)) * float(w) )
//
// Work split: a row of up to 512 elements belongs to one warp (no shared memory, no barrier);
// longer rows get one CTA of 64..1024 threads with two vectors per thread (up to eight beyond
// 16384 elements).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "bf16x8.cuh"
#include "host_common.h"
#include "ptx_sm100.cuh"
#include "warp_reduce.cuh"

namespace l3ci {
namespace {

template <int TPR>
struct RmsCfg {
  static constexpr int kBlock = TPR <= 32 ? 128 : TPR;
  static constexpr int kRowsPerCta = kBlock / TPR;
};

// With `res` the row that is normalised is s = bf16(x + res) (what a bf16 tensor add produces); s is also
// written to `sum_out`, which is the residual stream of the next layer (model.py:147-148 do the add and the
// norm as separate kernels).
template <int TPR, int VPT>
__global__ void __launch_bounds__(RmsCfg<TPR>::kBlock)
rms_norm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                __nv_bfloat16* __restrict__ out, long long rows, int nvec, long long x_stride,
                long long out_stride, float embed_f, float eps, const __nv_bfloat16* __restrict__ res,
                __nv_bfloat16* __restrict__ sum_out) {
  constexpr int kRows = RmsCfg<TPR>::kRowsPerCta;
  __shared__ float red[32];
  pdl_wait();               // the previous kernel of the stream has completed; its writes are visible
  pdl_launch_dependents();  // the next one may be set up while this one runs
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
      if (res) {
        // rows of res and sum_out are dense (stride = row length)
        const long long off = row * ((long long)nvec * kVecElems) + (long long)idx * kVecElems;
        const uint4 rv = ld_stream16(res + off);
        float a[8], b[8];
        unpack8(v[i], a);
        unpack8(rv, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = __fadd_rn(a[j], b[j]);
        v[i] = pack8(a);
        *reinterpret_cast<uint4*>(sum_out + off) = v[i];
      }
    } else {
      v[i] = make_uint4(0, 0, 0, 0);
    }
  }
  // the weight does not depend on the reduction: fetch it while the row is in flight
  // (unless row + weight would not fit the registers a thread of this CTA size can have)
  constexpr bool kEarlyW = VPT * RmsCfg<TPR>::kBlock <= 2048;
  uint4 wv[VPT];
  if constexpr (kEarlyW) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = t + i * TPR;
      wv[i] = idx < nvec ? __ldg(reinterpret_cast<const uint4*>(w) + idx) : make_uint4(0, 0, 0, 0);
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
      if constexpr (!kEarlyW) wv[i] = __ldg(reinterpret_cast<const uint4*>(w) + idx);
      float f[8], g[8];
      unpack8(v[i], f);
      unpack8(wv[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __fmul_rn(__fmul_rn(f[j], inv), g[j]);
      st_stream16(orow + (long long)idx * kVecElems, pack8(f));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Many rows (a prefill or a token batch): a persistent grid in which every WARP owns a stream of rows.
//
// The kernel above spends a CTA per row: 4096 rows of 2048 columns are 4096 CTAs of 128 threads that each load two
// vectors, meet at two barriers and leave — the launch ramp, the CTA turnover and ~15 instructions per element
// pair keep it at two thirds of the copy bandwidth.  Here a warp keeps the weight row in registers for its whole
// life, holds a row as VPL 16-byte vectors per lane, has the NEXT row's loads in flight while it reduces and
// writes the current one, reduces with shuffles only (no shared memory, no barrier), and does the fp32 arithmetic
// two lanes at a time (fma.rn.f32x2 / mul.rn.f32x2, exact per component), which halves the arithmetic issue slots.
// Same values as the kernel above except for the order of the fp32 sum of squares.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long mul_f32x2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// The two bf16 of a packed word widened to an fp32 pair.
__device__ __forceinline__ unsigned long long bf16x2_to_f32x2(uint32_t w) {
  return pack_f32x2(bf16lo_to_f32(w), bf16hi_to_f32(w));
}

constexpr int kRowsBlock = 256;  // 8 warps, each on its own rows

// (Two CTAs per SM, i.e. 128 registers per thread; the widest rows with a residual need more and run one per SM.
// With eight vectors per lane the weight row is re-read from L1 for every row instead of held in registers.)
template <int VPL, bool kRes>
__global__ void __launch_bounds__(kRowsBlock, (VPL >= 8 && kRes) ? 1 : 2)
rms_norm_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                     __nv_bfloat16* __restrict__ out, long long rows, int nvec, long long x_stride, long long out_stride,
                     float embed_f, float eps, const __nv_bfloat16* __restrict__ res, __nv_bfloat16* __restrict__ sum_out) {
  pdl_wait();               // the previous kernel of the stream has completed; its writes are visible
  pdl_launch_dependents();  // the next one may be set up while this one runs
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (kRowsBlock / 32);
  long long row = (long long)blockIdx.x * (kRowsBlock / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;
  constexpr bool kKeepW = VPL < 8;
  uint4 wv[kKeepW ? VPL : 1];
  if constexpr (kKeepW) {
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int idx = lane + 32 * i;
      wv[i] = idx < nvec ? __ldg(reinterpret_cast<const uint4*>(w) + idx) : make_uint4(0, 0, 0, 0);
    }
  }
  const long long dense = (long long)nvec * kVecElems;  // row length of res / sum_out
  uint4 cur[VPL], nxt[VPL], rcur[kRes ? VPL : 1], rnxt[kRes ? VPL : 1];
  auto fetch = [&](long long r, uint4 (&v)[VPL], uint4 (&rv)[kRes ? VPL : 1]) {
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int idx = lane + 32 * i;
      const bool ok = idx < nvec;
      v[i] = ok ? ld_stream16(x + r * x_stride + (long long)idx * kVecElems) : make_uint4(0, 0, 0, 0);
      if constexpr (kRes) rv[i] = ok ? ld_stream16(res + r * dense + (long long)idx * kVecElems) : make_uint4(0, 0, 0, 0);
    }
  };
  fetch(row, cur, rcur);
  while (true) {
    const long long next = row + warps;
    const bool more = next < rows;
    if (more) fetch(next, nxt, rnxt);
    if constexpr (kRes) {  // s = bf16(x + residual), written out and normalised
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        float a[8], b[8];
        unpack8(cur[i], a);
        unpack8(rcur[i], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = __fadd_rn(a[j], b[j]);
        cur[i] = pack8(a);
        const int idx = lane + 32 * i;
        if (idx < nvec) *reinterpret_cast<uint4*>(sum_out + row * dense + (long long)idx * kVecElems) = cur[i];
      }
    }
    unsigned long long acc0 = 0ull, acc1 = 0ull;  // two fp32 pairs of partial sums
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const unsigned long long p0 = bf16x2_to_f32x2(cur[i].x), p1 = bf16x2_to_f32x2(cur[i].y);
      const unsigned long long p2 = bf16x2_to_f32x2(cur[i].z), p3 = bf16x2_to_f32x2(cur[i].w);
      acc0 = fma_f32x2(p0, p0, acc0);
      acc1 = fma_f32x2(p1, p1, acc1);
      acc0 = fma_f32x2(p2, p2, acc0);
      acc1 = fma_f32x2(p3, p3, acc1);
    }
    float s0, s1, s2, s3;
    unpack_f32x2(acc0, s0, s1);
    unpack_f32x2(acc1, s2, s3);
    const float ss = group_sum<32>((s0 + s1) + (s2 + s3));
    const float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, embed_f), eps));
    const unsigned long long inv2 = pack_f32x2(inv, inv);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int idx = lane + 32 * i;
      if (idx < nvec) {
        const uint32_t xs[4] = {cur[i].x, cur[i].y, cur[i].z, cur[i].w};
        const uint4 wi = kKeepW ? wv[kKeepW ? i : 0] : __ldg(reinterpret_cast<const uint4*>(w) + idx);
        const uint32_t ws[4] = {wi.x, wi.y, wi.z, wi.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float lo, hi;
          unpack_f32x2(mul_f32x2(mul_f32x2(bf16x2_to_f32x2(xs[j]), inv2), bf16x2_to_f32x2(ws[j])), lo, hi);
          o[j] = pack_bf16x2(lo, hi);
        }
        st_stream16(out + row * out_stride + (long long)idx * kVecElems, make_uint4(o[0], o[1], o[2], o[3]));
      }
    }
    if (!more) break;
    row = next;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      cur[i] = nxt[i];
      if constexpr (kRes) rcur[i] = rnxt[i];
    }
  }
}

template <int VPL>
int launch_rows(const void* x, const void* w, void* out, long long rows, int nvec, long long xs, long long os, float eps,
                cudaStream_t stream, const void* res, void* sum_out) {
  const int sms = sm_count();
  if (sms <= 0) return fail(L3CI_ERR_CUDA, "rms_norm: no CUDA device");
  const long long want = (rows + kRowsBlock / 32 - 1) / (kRowsBlock / 32);
  const long long per_sm = (VPL >= 8 && res) ? 1 : 2;  // CTAs an SM holds (see the launch bounds); all resident for the whole launch
  const unsigned grid = (unsigned)(want < per_sm * sms ? want : per_sm * sms);
  const auto xb = static_cast<const __nv_bfloat16*>(x), wb = static_cast<const __nv_bfloat16*>(w), rb = static_cast<const __nv_bfloat16*>(res);
  const auto ob = static_cast<__nv_bfloat16*>(out), sb = static_cast<__nv_bfloat16*>(sum_out);
  if (res) L3CI_LAUNCH("rms_norm_rows_kernel", rms_norm_rows_kernel<VPL, true>, dim3(grid), dim3(kRowsBlock), 0, stream, xb, wb, ob, rows, nvec, xs, os, (float)(nvec * kVecElems), eps, rb, sb);
  else L3CI_LAUNCH("rms_norm_rows_kernel", rms_norm_rows_kernel<VPL, false>, dim3(grid), dim3(kRowsBlock), 0, stream, xb, wb, ob, rows, nvec, xs, os, (float)(nvec * kVecElems), eps, rb, sb);
  return L3CI_OK;
}

template <int TPR, int VPT>
int launch(const void* x, const void* w, void* out, long long rows, int nvec, long long xs,
           long long os, float eps, cudaStream_t stream, const void* res, void* sum_out) {
  constexpr int kRows = RmsCfg<TPR>::kRowsPerCta;
  const long long ctas = (rows + kRows - 1) / kRows;
  if (ctas > 0x7fffffffLL) return fail(L3CI_ERR_INVALID, "rms_norm: too many rows (%lld)", rows);
  L3CI_LAUNCH("rms_norm_kernel", rms_norm_kernel<TPR, VPT>, dim3((unsigned)ctas), dim3(RmsCfg<TPR>::kBlock), 0, stream,
              static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
              static_cast<__nv_bfloat16*>(out), rows, nvec, xs, os, (float)(nvec * kVecElems), eps,
              static_cast<const __nv_bfloat16*>(res), static_cast<__nv_bfloat16*>(sum_out));
  return L3CI_OK;
}

template <int TPR>
int launch_vpt(int vpt, const void* x, const void* w, void* out, long long rows, int nvec,
               long long xs, long long os, float eps, cudaStream_t stream, const void* res, void* sum_out) {
  if (vpt <= 1) return launch<TPR, 1>(x, w, out, rows, nvec, xs, os, eps, stream, res, sum_out);
  if (vpt <= 2) return launch<TPR, 2>(x, w, out, rows, nvec, xs, os, eps, stream, res, sum_out);
  if (vpt <= 4) return launch<TPR, 4>(x, w, out, rows, nvec, xs, os, eps, stream, res, sum_out);
  return launch<TPR, 8>(x, w, out, rows, nvec, xs, os, eps, stream, res, sum_out);
}

int rms_norm_dispatch(const void* x, const void* weight, void* out, int64_t rows, int64_t embed, int64_t x_row_stride,
                      int64_t out_row_stride, float eps, cudaStream_t stream, const void* res, void* sum_out,
                      const char* what) {
  if (rows < 0 || embed <= 0) return fail(L3CI_ERR_INVALID, "%s: rows=%lld embed=%lld", what, (long long)rows, (long long)embed);
  if (rows == 0) return L3CI_OK;
  if (!x || !weight || !out) return fail(L3CI_ERR_INVALID, "%s: null pointer", what);
  if (embed % kVecElems != 0 || embed > 65536)
    return fail(L3CI_ERR_UNSUPPORTED, "%s: embed=%lld must be a multiple of 8 and <= 65536", what, (long long)embed);
  if (!aligned16(x) || !aligned16(weight) || !aligned16(out) || x_row_stride % kVecElems ||
      out_row_stride % kVecElems || (res && !aligned16(res)) || (sum_out && !aligned16(sum_out)))
    return fail(L3CI_ERR_ALIGNMENT, "%s: rows must start on 16 bytes", what);
  const int nvec = (int)(embed / kVecElems);
  // Many rows of up to 2048 columns: a warp per row in a persistent grid (from a few rows per warp of the device on;
  // below that the rows-in-flight of the one-CTA-per-row kernel win).
  if (nvec <= 256 && rows >= 16LL * sm_count()) {
    const int vpl = (nvec + 31) / 32;
    if (vpl <= 1) return launch_rows<1>(x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream, res, sum_out);
    if (vpl <= 2) return launch_rows<2>(x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream, res, sum_out);
    if (vpl <= 4) return launch_rows<4>(x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream, res, sum_out);
    return launch_rows<8>(x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream, res, sum_out);
  }
  // Thread group per row: two vectors per thread where the row allows it (measured on B200 at 2048 columns:
  // 128 threads x 2 vectors beat 32 x 8 by 1 us of 13 at 4096 rows and by 2 us of 8 at 64 rows: the loads of a
  // row are one or two deep instead of eight), up to eight per thread for the longest rows.
  int tpr = 32;
  while (tpr < 1024 && tpr * 2 < nvec) tpr *= 2;
  const int vpt = (nvec + tpr - 1) / tpr;
  switch (tpr) {
    case 32: return launch_vpt<32>(vpt, x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream, res, sum_out);
    case 64: return launch_vpt<64>(vpt, x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream, res, sum_out);
    case 128: return launch_vpt<128>(vpt, x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream, res, sum_out);
    case 256: return launch_vpt<256>(vpt, x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream, res, sum_out);
    case 512: return launch_vpt<512>(vpt, x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream, res, sum_out);
    default: return launch_vpt<1024>(vpt, x, weight, out, rows, nvec, x_row_stride, out_row_stride, eps, stream, res, sum_out);
  }
}

// out = bf16( bf16(silu(gate)) * up ): the two roundings of F.silu(gate) * up on bf16 tensors (model.py:134).
__global__ void __launch_bounds__(256)
silu_mul_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                __nv_bfloat16* __restrict__ out, long long nvec, int row_vecs, long long gate_stride,
                long long up_stride) {
  pdl_wait();               // the previous kernel of the stream has completed; its writes are visible
  pdl_launch_dependents();  // the next one may be set up while this one runs
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= nvec) return;
  const long long r = i / row_vecs, c = (i % row_vecs) * kVecElems;
  const uint4 g = ld_stream16(gate + r * gate_stride + c), u = ld_stream16(up + r * up_stride + c);
  float a[8], b[8];
  unpack8(g, a);
  unpack8(u, b);
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = __fdiv_rn(a[j], __fadd_rn(1.0f, expf(-a[j])));
  const uint4 s = pack8(a);  // first rounding: silu(gate) as a bf16 tensor
  unpack8(s, a);
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = __fmul_rn(a[j], b[j]);
  st_stream16(out + i * kVecElems, pack8(a));
}

}  // namespace
}  // namespace l3ci

extern "C" int l3ci_rms_norm(const void* x, const void* weight, void* out, int64_t rows,
                             int64_t embed, int64_t x_row_stride, int64_t out_row_stride,
                             float eps, l3ci_stream_t stream_) {
  l3ci::clear_error();
  return l3ci::rms_norm_dispatch(x, weight, out, rows, embed, x_row_stride, out_row_stride, eps,
                                 reinterpret_cast<cudaStream_t>(stream_), nullptr, nullptr, "rms_norm");
}

extern "C" int l3ci_add_rms_norm(const void* x, const void* residual, const void* weight, void* sum_out, void* out,
                                 int64_t rows, int64_t embed, float eps, l3ci_stream_t stream_) {
  l3ci::clear_error();
  if (!residual || !sum_out) return l3ci::fail(L3CI_ERR_INVALID, "add_rms_norm: null pointer");
  return l3ci::rms_norm_dispatch(x, weight, out, rows, embed, embed, embed, eps, reinterpret_cast<cudaStream_t>(stream_),
                                 residual, sum_out, "add_rms_norm");
}

extern "C" int l3ci_silu_mul(const void* gate, const void* up, void* out, int64_t rows, int64_t cols,
                             int64_t gate_row_stride, int64_t up_row_stride, l3ci_stream_t stream_) {
  using namespace l3ci;
  clear_error();
  if (rows < 0 || cols < 0) return fail(L3CI_ERR_INVALID, "silu_mul: negative size");
  if (rows == 0 || cols == 0) return L3CI_OK;
  if (!gate || !up || !out) return fail(L3CI_ERR_INVALID, "silu_mul: null pointer");
  if (cols % kVecElems || cols / kVecElems > 0x7fffffffLL || gate_row_stride % kVecElems || up_row_stride % kVecElems ||
      !aligned16(gate) || !aligned16(up) || !aligned16(out))
    return fail(L3CI_ERR_ALIGNMENT, "silu_mul: rows must start on 16 bytes and cols be a multiple of 8");
  const long long nvec = rows * (cols / kVecElems);
  const long long ctas = (nvec + 255) / 256;
  if (ctas > 0x7fffffffLL) return fail(L3CI_ERR_INVALID, "silu_mul: tensor too large");
  L3CI_LAUNCH("silu_mul_kernel", silu_mul_kernel, dim3((unsigned)ctas), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream_),
              static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up), static_cast<__nv_bfloat16*>(out), nvec,
              (int)(cols / kVecElems), gate_row_stride, up_row_stride);
  return L3CI_OK;
}
