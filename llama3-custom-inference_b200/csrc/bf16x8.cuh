// 16-byte bf16 vectors and bf16 <-> fp32 conversion for the decode kernels.
//
// Role of the reference's custom_kernels/dtype_bfloat16.cuh:6-54 (Precision, VEC_SIZE,
// Vec<>, bf16_8_t, float2p, p2float): the storage type is bf16, the widest access is
// 8 elements = 16 bytes, and all arithmetic happens in fp32 after unpacking.
// Here the 16-byte vector is a plain uint4 so that it maps to one LDG.128 / STG.128, and
// unpacking uses the fact that a bf16 is the high half of an fp32.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace l3ci {

constexpr int kVecElems = 8;  // bf16 per 16-byte access

// Low / high bf16 of a packed 32-bit word, widened to fp32 (exact).
__device__ __forceinline__ float bf16lo_to_f32(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Round two fp32 to bf16 (nearest-even) and pack: `lo` lands in the low half.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf16lo_to_f32(v.x); f[1] = bf16hi_to_f32(v.x);
  f[2] = bf16lo_to_f32(v.y); f[3] = bf16hi_to_f32(v.y);
  f[4] = bf16lo_to_f32(v.z); f[5] = bf16hi_to_f32(v.z);
  f[6] = bf16lo_to_f32(v.w); f[7] = bf16hi_to_f32(v.w);
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  v.x = pack_bf16x2(f[0], f[1]);
  v.y = pack_bf16x2(f[2], f[3]);
  v.z = pack_bf16x2(f[4], f[5]);
  v.w = pack_bf16x2(f[6], f[7]);
  return v;
}

// Streaming 16-byte accesses: data touched once should not displace what other kernels keep
// in L1/L2 (weights, rotary table).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  return __ldcs(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void st_stream16(void* p, const uint4& v) {
  __stcs(reinterpret_cast<uint4*>(p), v);
}

}  // namespace l3ci
