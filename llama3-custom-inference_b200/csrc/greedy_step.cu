// Greedy next-token step of a decode loop as one kernel: per sequence, the argmax of its logits row and the
// bookkeeping that follows it.
//
// The reference's greedy branch (model.py:370-371 `torch.argmax(logits[:, -1], dim=-1)`, then model.py:373-381:
// write the token into the output, make it the next input, advance the position) is an argmax kernel plus a
// handful of tiny elementwise launches per generated token, and a host sync for the end-of-sequence test.  Here
// row b's CTA scans the row once with 16-byte loads, reduces (value, first index) and then, as one thread,
//     tok = argmax            (ties: the smallest index, like torch.argmax; a NaN counts as the maximum)
//     out_tokens[b, steps[b]] = tok;  next_input[b] = tok;  steps[b] += 1;  positions[b] += 1;  seq_lens[b] += 1
// Everything the next decode step reads stays in device memory, so the step can sit in a CUDA graph.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include "bf16x8.cuh"
#include "host_common.h"
#include "ptx_sm100.cuh"
#include "warp_reduce.cuh"

namespace l3ci {
namespace {

constexpr int kGreedyBlock = 1024;

// Is candidate (v, i) better than the best so far (bv, bi)?  Larger value wins, NaN beats every number, equal
// values (and NaN against NaN) go to the smaller index.
__device__ __forceinline__ bool better(float v, long long i, float bv, long long bi) {
  const bool vn = v != v, bn = bv != bv;
  if (vn != bn) return vn;
  if (!vn && v != bv) return v > bv;
  return i < bi;
}
// Maximum that is NaN as soon as one input is.
__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float vec_max(uint4 x) {
  float f[8];
  unpack8(x, f);
  return max_nan(max_nan(max_nan(f[0], f[1]), max_nan(f[2], f[3])), max_nan(max_nan(f[4], f[5]), max_nan(f[6], f[7])));
}

__global__ void __launch_bounds__(kGreedyBlock)
greedy_step_kernel(const __nv_bfloat16* __restrict__ logits, long long vocab, long long row_stride,
                   long long* __restrict__ out_tokens, long long out_stride, long long out_cols,
                   long long* __restrict__ steps, long long* __restrict__ next_input, int* __restrict__ positions,
                   int* __restrict__ seq_lens) {
  __shared__ float s_val[kGreedyBlock / kWarp];
  __shared__ long long s_idx[kGreedyBlock / kWarp];
  pdl_wait();               // the previous kernel of the stream has completed; its writes are visible
  pdl_launch_dependents();  // the next one may be set up while this one runs
  const long long b = blockIdx.x;
  const __nv_bfloat16* row = logits + b * row_stride;
  float best = -INFINITY;
  long long best_i = 0x7fffffffffffffffLL;
  // 16-byte vectors where the row allows it (row start 16-byte aligned), four in flight per thread; scalars for
  // the rest.  Per vector only its maximum is compared (a thread meets its vectors in increasing order, so
  // "strictly larger" keeps the first); the element is looked up once, in the winning vector.
  const bool vec_ok = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
  const long long nvec = vec_ok ? vocab / kVecElems : 0;
  constexpr int kInFlight = 4;
  long long best_v = -1;
  for (long long v0 = threadIdx.x; v0 < nvec; v0 += kInFlight * kGreedyBlock) {
    uint4 x[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const long long v = v0 + (long long)u * kGreedyBlock;
      if (v < nvec) x[u] = __ldg(reinterpret_cast<const uint4*>(row) + v);
    }
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const long long v = v0 + (long long)u * kGreedyBlock;
      if (v >= nvec) continue;
      const float m = vec_max(x[u]);
      if (best_v < 0 || m > best || (m != m && best == best)) { best = m; best_v = v; }
    }
  }
  if (best_v >= 0) {
    float f[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(row) + best_v), f);
    int j = 7;
#pragma unroll
    for (int t = 6; t >= 0; --t)
      if (best != best ? f[t] != f[t] : f[t] == best) j = t;
    best_i = best_v * kVecElems + j;
  }
  for (long long i = nvec * kVecElems + threadIdx.x; i < vocab; i += kGreedyBlock) {
    const float x = __bfloat162float(row[i]);
    if (better(x, i, best, best_i)) { best = x; best_i = i; }
  }
#pragma unroll
  for (int m = kWarp / 2; m >= 1; m >>= 1) {
    const float ov = __shfl_xor_sync(kFullMask, best, m);
    const long long oi = __shfl_xor_sync(kFullMask, best_i, m);
    if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
  }
  const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = s_val[lane];
    best_i = s_idx[lane];
#pragma unroll
    for (int m = kWarp / 2; m >= 1; m >>= 1) {
      const float ov = __shfl_xor_sync(kFullMask, best, m);
      const long long oi = __shfl_xor_sync(kFullMask, best_i, m);
      if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) {
      if (out_tokens && steps) {
        const long long s = steps[b];
        if (s >= 0 && s < out_cols) out_tokens[b * out_stride + s] = best_i;  // a full output row is left alone
        steps[b] = s + 1;
      } else if (out_tokens) {
        out_tokens[b * out_stride] = best_i;
      }
      if (next_input) next_input[b] = best_i;
      if (positions) positions[b] += 1;
      if (seq_lens) seq_lens[b] += 1;
    }
  }
}

}  // namespace
}  // namespace l3ci

extern "C" int l3ci_greedy_step(const void* logits, int64_t rows, int64_t vocab, int64_t row_stride,
                                int64_t* out_tokens, int64_t out_stride, int64_t out_cols, int64_t* steps,
                                int64_t* next_input, int32_t* positions, int32_t* seq_lens, l3ci_stream_t stream_) {
  using namespace l3ci;
  clear_error();
  if (rows < 0 || vocab <= 0 || row_stride < vocab) return fail(L3CI_ERR_INVALID, "greedy_step: bad size");
  if (rows == 0) return L3CI_OK;
  if (!logits || (!out_tokens && !next_input)) return fail(L3CI_ERR_INVALID, "greedy_step: null logits or no output");
  if (rows > 0x7fffffffLL) return fail(L3CI_ERR_INVALID, "greedy_step: too many rows");
  if (steps && (!out_tokens || out_cols <= 0)) return fail(L3CI_ERR_INVALID, "greedy_step: steps needs out_tokens and its width");
  L3CI_LAUNCH("greedy_step_kernel", greedy_step_kernel, dim3((unsigned)rows), dim3(kGreedyBlock), 0, reinterpret_cast<cudaStream_t>(stream_),
              static_cast<const __nv_bfloat16*>(logits), vocab, row_stride, reinterpret_cast<long long*>(out_tokens), out_stride,
              out_cols, reinterpret_cast<long long*>(steps), reinterpret_cast<long long*>(next_input), positions, seq_lens);
  return L3CI_OK;
}
