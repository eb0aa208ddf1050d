// Shuffle reductions for the online softmax and RMSNorm.
//
// Role of the reference's custom_kernels/reduce_kernels.cuh:8-64 (block_sum / block_max:
// xor-butterfly inside a warp, one shared-memory hop between warps, result broadcast).
// Differences: the butterfly width is a template parameter because the attention kernel
// only ever reduces across the 4 lanes that share an MMA row, and the cross-warp step
// barriers on BOTH sides of the shared-memory hop, so back-to-back calls on the same
// scratch cannot overtake one another.
#pragma once

#include <cuda_runtime.h>

namespace l3ci {

constexpr int kWarp = 32;
constexpr unsigned kFullMask = 0xffffffffu;

// Sum over groups of WIDTH consecutive lanes (WIDTH a power of two <= 32); every lane of a
// group ends with the group's total.
template <int WIDTH>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int m = WIDTH / 2; m >= 1; m >>= 1) v += __shfl_xor_sync(kFullMask, v, m);
  return v;
}

template <int WIDTH>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
  for (int m = WIDTH / 2; m >= 1; m >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, m));
  return v;
}

// Sum over the first `warps` warps of the CTA (each contributes one value per thread);
// `smem` holds >= 32 floats.  All threads of those warps must call it.
__device__ __forceinline__ float cta_sum(float v, float* smem, int warps) {
  v = group_sum<kWarp>(v);
  if (warps == 1) return v;
  const int lane = threadIdx.x & (kWarp - 1);
  const int warp = threadIdx.x / kWarp;
  __syncthreads();  // previous readers of smem are done
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float t = lane < warps ? smem[lane] : 0.f;
  return group_sum<kWarp>(t);
}

}  // namespace l3ci
