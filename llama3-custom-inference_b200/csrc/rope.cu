// Rotary embedding (interleaved pairs) for sm_100a, alone and fused with the KV-cache write.
//
// Replaces custom_rot_embed_kernel / rot_embed (custom_kernels/custom_kernels.cu:391-442),
// which launches one 32/64-thread CTA per (batch, token, head) and moves 4 bytes per thread.
// Here one thread owns 8 consecutive bf16 (four rotation pairs, one 16-byte load and store)
// and the two fp32 table vectors that go with them; one CTA walks one token's heads.
// The fused variant walks the projection output q|k|v once and writes rotated q to a dense
// buffer, rotated k and untouched v straight into the cache rows of this step, which is what
// CausalSelfAttention.forward does with two kernel calls and two copies (model.py:100-108).
//
// Arithmetic: (x*c - y*s, x*s + y*c) in fp32 with each product and the sum rounded
// separately (no fused multiply-add), then one rounding to bf16, so results are
// bit-identical to the same formula evaluated with unfused fp32 operations on a CPU.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "bf16x8.cuh"
#include "host_common.h"
#include "ptx_sm100.cuh"

namespace l3ci {
namespace {

constexpr int kRopeBlock = 256;   // pair kernel: one thread per rotation pair
constexpr int kTokenBlock = 128;  // token kernels: threads stride over one token's vectors
constexpr int kTokenBatch = 4;    // 16-byte loads a thread has in flight

// One rotation, rounded exactly as the reference's compiled kernel rounds it: nvcc contracts each of
// `x*c - y*s` and `x*s + y*c` (custom_kernels/custom_kernels.cu:408,410) into a rounded product of the second
// term and a fused multiply-add of the first.  Written with explicit intrinsics so that the form does not depend
// on this file's compiler flags; outputs are bit-identical to the reference kernel's on the same inputs.
__device__ __forceinline__ void rotate_pair(float x, float y, float c, float s, float& xo, float& yo) {
  xo = __fmaf_rn(x, c, -__fmul_rn(y, s));
  yo = __fmaf_rn(x, s, __fmul_rn(y, c));
}

// Rotates the 8 bf16 of `v` with the table entries (f0, f1) = (c0,s0,c1,s1 | c2,s2,c3,s3).
__device__ __forceinline__ uint4 rotate8(const uint4& v, const float4& f0, const float4& f1) {
  float a[8], r[8];
  unpack8(v, a);
  rotate_pair(a[0], a[1], f0.x, f0.y, r[0], r[1]);
  rotate_pair(a[2], a[3], f0.z, f0.w, r[2], r[3]);
  rotate_pair(a[4], a[5], f1.x, f1.y, r[4], r[5]);
  rotate_pair(a[6], a[7], f1.z, f1.w, r[6], r[7]);
  return pack8(r);
}
__device__ __forceinline__ uint4 rotate8(const uint4& v, const float* __restrict__ freq8) {
  return rotate8(v, __ldg(reinterpret_cast<const float4*>(freq8)), __ldg(reinterpret_cast<const float4*>(freq8) + 1));
}

// x [B,S,H,D] strided, out dense.  One CTA per token: (batch, position) is decoded once per CTA and the
// threads stride over the token's H * D/8 vectors, so no thread does 64-bit index arithmetic.  VPH = vectors per
// head when that is 8 or 16 (head size 64 or 128; 0 = any): the CTA size is a multiple of it, so all vectors of a
// thread sit at the same place of their heads and share ONE pair of table loads, and head / vector indices are
// shifts (at 15 instructions per element pair the first version of this kernel was bound by instruction issue,
// not by memory: two table loads per vector and two integer divisions were most of them).
template <int VPH>
__global__ void __launch_bounds__(kTokenBlock)
rot_embed_vec8_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ freq,
                      __nv_bfloat16* __restrict__ out, int S, int H, int vec_per_head_rt, long long sb, long long ss,
                      long long sh) {
  pdl_wait();               // the previous kernel of the stream has completed; its writes are visible
  pdl_launch_dependents();  // the next one may be set up while this one runs
  const int vec_per_head = VPH ? VPH : vec_per_head_rt;
  const long long token = blockIdx.x;
  const int s = (int)(token % S);
  const long long b = token / S;
  const int D = vec_per_head * kVecElems;
  const int row_vecs = H * vec_per_head;
  const __nv_bfloat16* xin = x + b * sb + s * ss;
  __nv_bfloat16* xout = out + token * (long long)row_vecs * kVecElems;
  const float* f = freq + (long long)s * D;
  float4 f0 = make_float4(0, 0, 0, 0), f1 = f0;
  if constexpr (VPH != 0) {
    const float* fv = f + (threadIdx.x % VPH) * kVecElems;
    f0 = __ldg(reinterpret_cast<const float4*>(fv));
    f1 = __ldg(reinterpret_cast<const float4*>(fv) + 1);
  }
  for (int i0 = threadIdx.x; i0 < row_vecs; i0 += kTokenBlock * kTokenBatch) {
    uint4 v[kTokenBatch];
#pragma unroll
    for (int u = 0; u < kTokenBatch; ++u) {
      const int i = i0 + u * kTokenBlock;
      if (i < row_vecs) {
        const int h = i / vec_per_head, vec = i - h * vec_per_head;
        v[u] = ld_stream16(xin + h * sh + vec * kVecElems);
      }
    }
#pragma unroll
    for (int u = 0; u < kTokenBatch; ++u) {
      const int i = i0 + u * kTokenBlock;
      if (i >= row_vecs) continue;
      if constexpr (VPH != 0) st_stream16(xout + i * kVecElems, rotate8(v[u], f0, f1));
      else st_stream16(xout + i * kVecElems, rotate8(v[u], f + (i % vec_per_head) * kVecElems));
    }
  }
}

// Fallback for rows that only start on 4 bytes: one thread per rotation pair.
__global__ void __launch_bounds__(kRopeBlock)
rot_embed_pair_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ freq,
                      __nv_bfloat16* __restrict__ out, long long total, int S, int H, int pairs_per_head,
                      long long sb, long long ss, long long sh) {
  const long long idx = (long long)blockIdx.x * kRopeBlock + threadIdx.x;
  if (idx >= total) return;
  const int p = (int)(idx % pairs_per_head);
  long long rest = idx / pairs_per_head;
  const int h = (int)(rest % H);
  rest /= H;
  const int s = (int)(rest % S);
  const long long b = rest / S;
  const int D = pairs_per_head * 2;
  const uint32_t w = *reinterpret_cast<const uint32_t*>(x + b * sb + s * ss + h * sh + 2 * p);
  const float2 cs = __ldg(reinterpret_cast<const float2*>(freq + (long long)s * D) + p);
  float xo, yo;
  rotate_pair(bf16lo_to_f32(w), bf16hi_to_f32(w), cs.x, cs.y, xo, yo);
  *reinterpret_cast<uint32_t*>(out + idx * 2) = pack_bf16x2(xo, yo);
}

// qkv [B,T,(Hq+2Hkv)*D] -> q_out dense [B,T,Hq,D], cache_k/v[b, pos, h, :].  One CTA per token; VPH as above.
template <int VPH>
__global__ void __launch_bounds__(kTokenBlock)
rot_embed_kv_cache_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ freq,
                          __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ cache_k,
                          __nv_bfloat16* __restrict__ cache_v, int T, int Hq, int Hkv, int vec_per_head_rt,
                          long long qkv_sb, long long qkv_st, long long cache_sb, long long cache_st,
                          long long start_pos, const int* __restrict__ positions, long long freq_rows,
                          long long cache_len) {
  pdl_wait();               // the previous kernel of the stream has completed; its writes are visible
  pdl_launch_dependents();  // the next one may be set up while this one runs
  const int vec_per_head = VPH ? VPH : vec_per_head_rt;
  const long long token = blockIdx.x;
  const int t = (int)(token % T);
  const long long b = token / T;
  const int D = vec_per_head * kVecElems;
  // Position of this token: start_pos + t for the whole batch, or positions[b] + t per sequence (then
  // `freq` is the whole table and a position outside the table or the cache is skipped, not written).
  long long pos = start_pos + t, frow = t;
  if (positions) {
    pos = (long long)__ldg(positions + b) + t;
    frow = pos;
    if (pos < 0 || pos >= freq_rows || pos >= cache_len) return;
  }
  const __nv_bfloat16* in = qkv + b * qkv_sb + t * qkv_st;
  const float* f = freq + frow * D;
  __nv_bfloat16* qo = q_out + token * (long long)Hq * D;
  __nv_bfloat16* ko = cache_k + b * cache_sb + pos * cache_st;
  __nv_bfloat16* vo = cache_v + b * cache_sb + pos * cache_st;
  const int q_vecs = Hq * vec_per_head, k_vecs = Hkv * vec_per_head;
  const int row_vecs = q_vecs + 2 * k_vecs;
  float4 f0 = make_float4(0, 0, 0, 0), f1 = f0;
  if constexpr (VPH != 0) {
    const float* fv = f + (threadIdx.x % VPH) * kVecElems;
    f0 = __ldg(reinterpret_cast<const float4*>(fv));
    f1 = __ldg(reinterpret_cast<const float4*>(fv) + 1);
  }
  for (int i0 = threadIdx.x; i0 < row_vecs; i0 += kTokenBlock * kTokenBatch) {
    uint4 v[kTokenBatch];
#pragma unroll
    for (int u = 0; u < kTokenBatch; ++u) {
      const int i = i0 + u * kTokenBlock;
      if (i < row_vecs) v[u] = ld_stream16(in + i * kVecElems);
    }
#pragma unroll
    for (int u = 0; u < kTokenBatch; ++u) {
      const int i = i0 + u * kTokenBlock;
      if (i >= row_vecs) continue;
      if (i < q_vecs + k_vecs) {
        uint4 r;
        if constexpr (VPH != 0) r = rotate8(v[u], f0, f1);
        else r = rotate8(v[u], f + (i % vec_per_head) * kVecElems);
        if (i < q_vecs) st_stream16(qo + i * kVecElems, r);
        // Cache rows are read again by the attention kernel of the same step: plain store.
        else *reinterpret_cast<uint4*>(ko + (i - q_vecs) * kVecElems) = r;
      } else {
        *reinterpret_cast<uint4*>(vo + (i - q_vecs - k_vecs) * kVecElems) = v[u];
      }
    }
  }
}

// Launch of the instance for this head size (8 or 16 vectors per head: shifts and shared table loads; else generic).
template <typename... Args>
cudaError_t launch_kv_cache(int vec_per_head, unsigned grid, cudaStream_t stream, Args... args) {
  if (vec_per_head == 8) return launch_kernel(rot_embed_kv_cache_kernel<8>, dim3(grid), dim3(kTokenBlock), 0, stream, args...);
  if (vec_per_head == 16) return launch_kernel(rot_embed_kv_cache_kernel<16>, dim3(grid), dim3(kTokenBlock), 0, stream, args...);
  return launch_kernel(rot_embed_kv_cache_kernel<0>, dim3(grid), dim3(kTokenBlock), 0, stream, args...);
}

int grid_for(long long total, unsigned* grid) {
  const long long ctas = (total + kRopeBlock - 1) / kRopeBlock;
  if (ctas > 0x7fffffffLL) return fail(L3CI_ERR_INVALID, "rot_embed: tensor too large");
  *grid = (unsigned)ctas;
  return L3CI_OK;
}

}  // namespace
}  // namespace l3ci

extern "C" int l3ci_rot_embed(const void* x, const float* freq, void* out, int64_t B, int64_t S,
                              int64_t H, int64_t D, int64_t sb, int64_t ss, int64_t sh,
                              l3ci_stream_t stream_) {
  using namespace l3ci;
  clear_error();
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (B < 0 || S < 0 || H < 0 || D <= 0) return fail(L3CI_ERR_INVALID, "rot_embed: negative size");
  if (B == 0 || S == 0 || H == 0) return L3CI_OK;
  if (!x || !freq || !out) return fail(L3CI_ERR_INVALID, "rot_embed: null pointer");
  if (D % 2) return fail(L3CI_ERR_UNSUPPORTED, "rot_embed: head size %lld is odd", (long long)D);
  if (S > 0x7fffffff || H > 0x7fffffff || D > 0x7fffffff) return fail(L3CI_ERR_INVALID, "rot_embed: size overflow");
  const auto xp = static_cast<const __nv_bfloat16*>(x);
  const auto op = static_cast<__nv_bfloat16*>(out);
  const bool vec8 = D % kVecElems == 0 && aligned16(x) && aligned16(out) && aligned16(freq) &&
                    sb % kVecElems == 0 && ss % kVecElems == 0 && sh % kVecElems == 0;
  unsigned grid = 0;
  if (vec8) {
    if (B * S > 0x7fffffffLL || H * (D / kVecElems) > 0x7fffffffLL) return fail(L3CI_ERR_INVALID, "rot_embed: tensor too large");
    grid = (unsigned)(B * S);
    const int vph = (int)(D / kVecElems);
    if (vph == 8) L3CI_LAUNCH("rot_embed_vec8_kernel", rot_embed_vec8_kernel<8>, dim3(grid), dim3(kTokenBlock), 0, stream, xp, freq, op, (int)S, (int)H, vph, sb, ss, sh);
    else if (vph == 16) L3CI_LAUNCH("rot_embed_vec8_kernel", rot_embed_vec8_kernel<16>, dim3(grid), dim3(kTokenBlock), 0, stream, xp, freq, op, (int)S, (int)H, vph, sb, ss, sh);
    else L3CI_LAUNCH("rot_embed_vec8_kernel", rot_embed_vec8_kernel<0>, dim3(grid), dim3(kTokenBlock), 0, stream, xp, freq, op, (int)S, (int)H, vph, sb, ss, sh);
    return L3CI_OK;
  }
  if ((reinterpret_cast<uintptr_t>(x) & 3) || (reinterpret_cast<uintptr_t>(out) & 3) ||
      (reinterpret_cast<uintptr_t>(freq) & 7) || (sb & 1) || (ss & 1) || (sh & 1))
    return fail(L3CI_ERR_ALIGNMENT, "rot_embed: rotation pairs must start on 4 bytes");
  const long long total = B * S * H * (D / 2);
  if (int st = grid_for(total, &grid)) return st;
  rot_embed_pair_kernel<<<grid, kRopeBlock, 0, stream>>>(xp, freq, op, total, (int)S, (int)H,
                                                         (int)(D / 2), sb, ss, sh);
  L3CI_CHECK_LAUNCH("rot_embed_pair_kernel");
  return L3CI_OK;
}

extern "C" int l3ci_rot_embed_kv_cache(const void* qkv, const float* freq, void* q_out, void* cache_k,
                                       void* cache_v, int64_t B, int64_t T, int64_t Hq, int64_t Hkv,
                                       int64_t D, int64_t qkv_sb, int64_t qkv_st, int64_t cache_sb,
                                       int64_t cache_st, int64_t start_pos, l3ci_stream_t stream_) {
  using namespace l3ci;
  clear_error();
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (B < 0 || T < 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || start_pos < 0)
    return fail(L3CI_ERR_INVALID, "rot_embed_kv_cache: bad size");
  if (B == 0 || T == 0) return L3CI_OK;
  if (!qkv || !freq || !q_out || !cache_k || !cache_v)
    return fail(L3CI_ERR_INVALID, "rot_embed_kv_cache: null pointer");
  if (D % kVecElems) return fail(L3CI_ERR_UNSUPPORTED, "rot_embed_kv_cache: head size %lld not a multiple of 8", (long long)D);
  if (!aligned16(qkv) || !aligned16(freq) || !aligned16(q_out) || !aligned16(cache_k) ||
      !aligned16(cache_v) || qkv_sb % kVecElems || qkv_st % kVecElems || cache_sb % kVecElems ||
      cache_st % kVecElems)
    return fail(L3CI_ERR_ALIGNMENT, "rot_embed_kv_cache: rows must start on 16 bytes");
  if (B * T > 0x7fffffffLL || (Hq + 2 * Hkv) * (D / kVecElems) > 0x7fffffffLL)
    return fail(L3CI_ERR_INVALID, "rot_embed_kv_cache: tensor too large");
  const cudaError_t le = launch_kv_cache((int)(D / kVecElems), (unsigned)(B * T), stream,
      static_cast<const __nv_bfloat16*>(qkv), freq, static_cast<__nv_bfloat16*>(q_out),
      static_cast<__nv_bfloat16*>(cache_k), static_cast<__nv_bfloat16*>(cache_v), (int)T,
      (int)Hq, (int)Hkv, (int)(D / kVecElems), (long long)qkv_sb, (long long)qkv_st, (long long)cache_sb, (long long)cache_st,
      (long long)start_pos, (const int*)nullptr, 0LL, 0LL);
  if (le != cudaSuccess) return fail(L3CI_ERR_CUDA, "launch of rot_embed_kv_cache_kernel failed: %s", cudaGetErrorString(le));
  return L3CI_OK;
}

extern "C" int l3ci_rot_embed_kv_cache_at(const void* qkv, const float* freq_table, int64_t freq_rows, void* q_out,
                                          void* cache_k, void* cache_v, const int32_t* positions, int64_t B,
                                          int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t qkv_sb,
                                          int64_t qkv_st, int64_t cache_sb, int64_t cache_st, int64_t cache_len,
                                          l3ci_stream_t stream_) {
  using namespace l3ci;
  clear_error();
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (B < 0 || T < 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || freq_rows < 0 || cache_len < 0)
    return fail(L3CI_ERR_INVALID, "rot_embed_kv_cache_at: bad size");
  if (B == 0 || T == 0) return L3CI_OK;
  if (!qkv || !freq_table || !q_out || !cache_k || !cache_v || !positions)
    return fail(L3CI_ERR_INVALID, "rot_embed_kv_cache_at: null pointer");
  if (D % kVecElems) return fail(L3CI_ERR_UNSUPPORTED, "rot_embed_kv_cache_at: head size %lld not a multiple of 8", (long long)D);
  if (!aligned16(qkv) || !aligned16(freq_table) || !aligned16(q_out) || !aligned16(cache_k) || !aligned16(cache_v) ||
      (reinterpret_cast<uintptr_t>(positions) & 3) || qkv_sb % kVecElems || qkv_st % kVecElems ||
      cache_sb % kVecElems || cache_st % kVecElems)
    return fail(L3CI_ERR_ALIGNMENT, "rot_embed_kv_cache_at: rows must start on 16 bytes");
  if (B * T > 0x7fffffffLL || (Hq + 2 * Hkv) * (D / kVecElems) > 0x7fffffffLL)
    return fail(L3CI_ERR_INVALID, "rot_embed_kv_cache_at: tensor too large");
  const cudaError_t le = launch_kv_cache((int)(D / kVecElems), (unsigned)(B * T), stream,
      static_cast<const __nv_bfloat16*>(qkv), freq_table, static_cast<__nv_bfloat16*>(q_out),
      static_cast<__nv_bfloat16*>(cache_k), static_cast<__nv_bfloat16*>(cache_v), (int)T, (int)Hq, (int)Hkv,
      (int)(D / kVecElems), (long long)qkv_sb, (long long)qkv_st, (long long)cache_sb, (long long)cache_st, 0LL,
      (const int*)positions, (long long)freq_rows, (long long)cache_len);
  if (le != cudaSuccess) return fail(L3CI_ERR_CUDA, "launch of rot_embed_kv_cache_kernel failed: %s", cudaGetErrorString(le));
  return L3CI_OK;
}
