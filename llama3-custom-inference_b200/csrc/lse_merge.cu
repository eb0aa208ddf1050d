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

// ---------------------------------------------------------------------------------------------
// Exchange + merge over peer memory (NVLink), one launch per rank, no collective library.
//
// Every rank owns a buffer of the same layout that all ranks can address (peer mapping set up by the caller):
//   data  [2 parities][W source ranks][rows * D outputs | rows lse, padded to a multiple of 4]   fp32
//   flags [2 parities][W source ranks][rows]                          uint32 (after the data)
// A call uses parity = epoch & 1.  Rank r has put its shard result into its own slot [parity][r] (the decode
// kernel writes there directly).  One warp per query row then
//   1. copies the row of the local slot into slot [parity][r] of every peer with plain stores,
//   2. fences at system scope and stores `epoch` into flag [parity][r][row] of every peer,
//   3. waits, bounded, until the local flags [parity][s][row] of all sources s show `epoch`,
//   4. merges the W rows by log-sum-exp from LOCAL memory and writes bf16.
// Two parities make the slots safe to reuse: a rank can only start call e + 2 after its call e + 1 finished,
// which needed every peer's call-(e+1) rows, which a peer sends only after its own call e has finished reading.
//
// The call number can live on the device (epoch argument 0): behind the flags every buffer has a staging slot and
// two control words.  The rank's own result is then expected in the staging slot (a fixed address, whatever the
// call number), the call number is control word 0 plus one, and the last warp of the launch to finish stores it
// back (control word 1 counts the finished warps).  A launch sequence without any host-side state can be
// captured in a CUDA graph and replayed.
// ---------------------------------------------------------------------------------------------
constexpr unsigned long long kXchgWaitNs = 1000000000ull;  // default bound of the wait for the peers' rows

__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long xchg_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__global__ void __launch_bounds__(kMergeBlock)
lse_exchange_merge_kernel(float* const* __restrict__ bufs, int rank, int W, unsigned epoch_arg, long long rows, int Hq,
                          int D, __nv_bfloat16* __restrict__ out, long long o_sb, long long o_sh, int* status,
                          unsigned long long wait_ns) {
  const long long row = (long long)blockIdx.x * (kMergeBlock / kWarp) + threadIdx.x / kWarp;
  const int lane = threadIdx.x % kWarp;
  if (row >= rows) return;
  const long long slot_floats = rows * D + ((rows + 3) & ~3LL);
  const long long data_floats = 2LL * W * slot_floats;
  const long long flag_words = (2LL * W * rows + 3) & ~3LL;
  float* local = bufs[rank];
  float* staging = local + data_floats + flag_words;
  unsigned* ctrl = reinterpret_cast<unsigned*>(staging + slot_floats);
  const bool auto_epoch = epoch_arg == 0u;
  // every warp of the launch reads the call number before the last of them to finish can advance it
  const unsigned epoch = auto_epoch ? __ldcg(ctrl) + 1u : epoch_arg;
  auto leave = [&]() {
    if (auto_epoch && lane == 0) {
      if (atomicAdd(ctrl + 1, 1u) == (unsigned)rows - 1u) {
        ctrl[1] = 0u;
        __threadfence();
        ctrl[0] = epoch;
      }
    }
  };
  const int parity = epoch & 1u;
  auto slot = [&](float* base, int src) { return base + ((long long)parity * W + src) * slot_floats; };
  auto flag = [&](float* base, int src) {
    return reinterpret_cast<unsigned*>(base + data_floats) + ((long long)parity * W + src) * rows + row;
  };
  // 1. push this rank's row to every peer
  const float* mine = auto_epoch ? staging : slot(local, rank);
  const float my_lse = mine[rows * D + row];
  for (int p = 0; p < W; ++p) {
    if (p == rank) continue;
    float* dst = slot(bufs[p], rank);
    for (int d = lane * 4; d < D; d += 4 * kWarp)
      *reinterpret_cast<float4*>(dst + row * D + d) = *reinterpret_cast<const float4*>(mine + row * D + d);
    if (lane == 0) dst[rows * D + row] = my_lse;
  }
  // 2. publish
  __threadfence_system();
  __syncwarp();
  if (lane < W && lane != rank) st_release_sys_u32(flag(bufs[lane], rank), epoch);
  for (int p = kWarp + lane; p < W; p += kWarp)
    if (p != rank) st_release_sys_u32(flag(bufs[p], rank), epoch);
  // 3. wait for the peers' rows (lane s watches source s; more than 32 ranks: strided)
  {
    const unsigned long long t0 = xchg_ns();
    bool late = false;
    for (unsigned it = 0;; ++it) {
      bool there = true;
      for (int s = lane; s < W; s += kWarp)
        if (s != rank && ld_acquire_sys_u32(flag(local, s)) != epoch) there = false;
      if (__all_sync(kFullMask, there)) break;
      __nanosleep(64);
      if ((it & 15u) == 15u && __any_sync(kFullMask, xchg_ns() - t0 > wait_ns)) { late = true; break; }
    }
    if (late) {
      if (lane == 0 && status) atomicExch(status, (int)L3CI_ERR_DEVICE_WAIT);
      leave();
      return;
    }
  }
  // 4. merge from local memory
  auto src = [&](int s) { return s == rank ? mine : slot(local, s); };
  float M = -INFINITY;
  for (int s = 0; s < W; ++s) M = fmaxf(M, __ldcg(src(s) + rows * D + row));
  const float Mu = M == -INFINITY ? 0.f : M;
  float L = 0.f;
  for (int s = 0; s < W; ++s) L += __expf(__ldcg(src(s) + rows * D + row) - Mu);
  const float invL = L > 0.f ? 1.f / L : 0.f;
  const long long b = row / Hq;
  const int h = (int)(row % Hq);
  __nv_bfloat16* orow = out + b * o_sb + h * o_sh;
  for (int d = lane * 2; d < D; d += 2 * kWarp) {
    float ax = 0.f, ay = 0.f;
    for (int s = 0; s < W; ++s) {
      const float* sl = src(s);
      const float w = __expf(__ldcg(sl + rows * D + row) - Mu) * invL;
      const float2 v = __ldcg(reinterpret_cast<const float2*>(sl + row * D + d));
      ax = fmaf(v.x, w, ax);
      ay = fmaf(v.y, w, ay);
    }
    *reinterpret_cast<uint32_t*>(orow + d) = pack_bf16x2(ax, ay);
  }
  leave();
}

}  // namespace
}  // namespace l3ci

extern "C" size_t l3ci_lse_exchange_bytes(int32_t ranks, int32_t B, int32_t Hq, int32_t D) {
  if (ranks <= 0 || B <= 0 || Hq <= 0 || D <= 0) return 0;
  const size_t rows = (size_t)B * Hq;
  const size_t slot_floats = rows * D + ((rows + 3) & ~(size_t)3);
  const size_t flag_words = (2 * (size_t)ranks * rows + 3) & ~(size_t)3;
  // data | flags | staging slot | control words (call number, finished warps) padded to 16 bytes
  return (2 * (size_t)ranks * slot_floats + flag_words + slot_floats + 4) * sizeof(float);
}

extern "C" int l3ci_lse_exchange_merge(void* const* bufs, int32_t rank, int32_t ranks, uint32_t epoch, void* out,
                                       int32_t B, int32_t Hq, int32_t D, int64_t o_sb, int64_t o_sh, int32_t* status,
                                       l3ci_stream_t stream_) {
  using namespace l3ci;
  clear_error();
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (ranks <= 0 || rank < 0 || rank >= ranks || B < 0 || Hq <= 0 || D <= 0)
    return fail(L3CI_ERR_INVALID, "lse_exchange_merge: bad size or rank");
  if (B == 0) return L3CI_OK;
  if (!bufs || !out) return fail(L3CI_ERR_INVALID, "lse_exchange_merge: null pointer");
  if (D % 4) return fail(L3CI_ERR_UNSUPPORTED, "lse_exchange_merge: head size %d is not a multiple of 4", D);
  if ((reinterpret_cast<uintptr_t>(out) & 3) || (o_sb & 1) || (o_sh & 1))
    return fail(L3CI_ERR_ALIGNMENT, "lse_exchange_merge: output rows must start on 4 bytes");
  const long long rows = (long long)B * Hq;
  const long long ctas = (rows + kMergeBlock / kWarp - 1) / (kMergeBlock / kWarp);
  lse_exchange_merge_kernel<<<(unsigned)ctas, kMergeBlock, 0, stream>>>(
      reinterpret_cast<float* const*>(bufs), rank, ranks, epoch, rows, Hq, D, static_cast<__nv_bfloat16*>(out), o_sb,
      o_sh, status, device_wait_limit_ns(kXchgWaitNs));
  L3CI_CHECK_LAUNCH("lse_exchange_merge_kernel");
  return L3CI_OK;
}

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
