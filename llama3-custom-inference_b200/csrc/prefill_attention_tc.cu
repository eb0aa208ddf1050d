// Causal GQA prefill attention on the 5th-generation tensor cores of sm_100a: tcgen05.mma with operands in shared
// memory (filled by bulk tensor copies) or tensor memory, accumulators in tensor memory (TMEM).
//
// Same computation as prefill_attention.cu (the reference's model.py:114-116 SDPA call), for prompts long enough
// that the arithmetic, not the launch, is what costs.  Two kernels, 128 query rows per head and CTA, 10 warps:
//   warp 0        producer: Q once, then K and V tiles of 128 keys through 2-stage rings of bulk tensor copies
//   warp 1        allocates TMEM and issues the MMAs: S = Q K_j^T into a 128-column score accumulator,
//                 O += P_j V_j into an output accumulator; tcgen05.commit signals the mbarriers.  All lanes run the
//                 issue code and one elected lane predicates the instructions (see tc_commit below).
//   warps 2-9     softmax, two groups of four warps.  Thread r of a group owns query row r (tcgen05.ld 32x32b gives
//                 a thread its row): the row of S_j goes to registers, p = 2^(s * scale - m_ref) is packed to bf16
//                 and stored over S_j as the A operand of the second MMA.  O stays in TMEM and the MMA accumulates
//                 into it; the reference maximum m_ref of a row only moves when the running maximum has outgrown it
//                 by more than 2^8 (p stays below 2^8, harmless in fp32 / bf16), and only then is the row of O
//                 rescaled in TMEM.  The arithmetic runs two lanes at a time (fma / add .f32x2, three-input max):
//                 the groups' own instructions, not the special-function unit, were what a tile cost.
// prefill_tc_pair_kernel (head ratio Hq / Hkv even): a CTA takes TWO query heads of one KV head; group e owns head
//                 hq0 + e with all its key tiles (its own Q tile, S_e, O_e), K and V tiles are loaded once for both.
//                 12 warps: the roles sit in whole warpgroups (warps 0-3: producer, MMA warp, two idle warps; warps
//                 4-11: the softmax groups) so that setmaxnreg can move registers from the first to the other two.
// prefill_tc_persist_kernel: the same as a persistent grid (one CTA per SM walks its items), when there are more
//                 (head pair, query block) items than SMs.
// prefill_tc_kernel (any head ratio): one head per CTA; group e takes the key tiles j with j % 2 == e with its own
//                 S_e, O_e and running (m_ref, l), and the two partial results of a row are merged at the end like
//                 two split-KV partials.
// K is the B operand as it lies in the cache ([keys][D], K-major); V is used MN-major, again as it lies.  Every
// wait is bounded; TMEM is freed on every path.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdlib.h>

#include "bf16x8.cuh"
#include "host_common.h"
#include "ptx_sm100.cuh"
#include "tensor_map.h"
#include "warp_reduce.cuh"

namespace l3ci {
namespace {

constexpr int kTcRows = 128;   // query rows per CTA (M of the MMA)
constexpr int kTcKeys = 128;   // keys per tile (N of S, K of P V)
constexpr int kTcStages = 2;
constexpr int kTcSoftmaxWarps = 8;                       // two groups of four: even tiles, odd tiles
constexpr int kTcThreads = 32 * (2 + kTcSoftmaxWarps);   // + producer warp + MMA warp
// The head-pair kernel keeps its roles in whole warpgroups (setmaxnreg acts on four warps at a time): warps 0-3 are
// producer, MMA warp and two idle warps, warps 4-11 the softmax groups.  384 threads start with 168 registers each.
constexpr int kTcPairThreads = 32 * (4 + kTcSoftmaxWarps);
constexpr int kTcPairRegsLow = 56, kTcPairRegsHigh = 224;
static_assert(4 * kTcPairRegsLow + kTcSoftmaxWarps * kTcPairRegsHigh <= 12 * 168, "the re-deal stays within the CTA's registers");
// The persistent kernel adds an output warpgroup (warps 12-15): 512 threads start with 128 registers each.
constexpr int kTcPersistThreads = kTcPairThreads + 128;
constexpr int kTcPersistRegsLow = 56, kTcPersistRegsHigh = 192, kTcPersistRegsOut = 72;
static_assert(4 * kTcPersistRegsLow + kTcSoftmaxWarps * kTcPersistRegsHigh + 4 * kTcPersistRegsOut <= 16 * 128, "register re-deal");
constexpr uint32_t kTmemCols = 512;                      // S_0, S_1 (128 columns each), O_0, O_1 (D columns each)

struct TcParams {
  __nv_bfloat16* out;
  int B, Hq, Hkv, R, T, n_keys, start_pos, m_blocks;
  long long o_sb, o_sh, o_st;
  float scale_log2e;
  int* status;
};

// ---- tcgen05 wrappers ----
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar, uint32_t elected) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
               "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}\n" ::"r"(bar), "r"(elected) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                       uint32_t elected) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %6, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(elected) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                       uint32_t elected) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %6, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(elected) : "memory");
}
// 32 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
// 64 consecutive 32-bit columns of this thread's TMEM lane in one instruction
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&r)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}

// fp32 arithmetic two lanes at a time and a three-input maximum: the softmax warps' own instructions, not the
// special-function unit, were what a score tile cost, so every instruction saved per element counts.
__device__ __forceinline__ unsigned long long f2_pack(uint32_t lo, uint32_t hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ unsigned long long f2_packf(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long f2_fma(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long f2_add(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Shared-memory matrix descriptor, 128-byte swizzle, rows (or 8-row groups) 1024 bytes apart: address and byte
// offsets in 16-byte units, descriptor version 1 (bits 46-47), layout type 2 = SWIZZLE_128B (bits 61-63).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: D fp32 (bits 4-5 = 1), A and B bf16 (bits 7-9, 10-12 = 1), B MN-major
// (bit 16), N / 8 (bits 17-22), M / 16 (bits 24-28).
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}

template <int D>
__global__ void __launch_bounds__(kTcThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                  const __grid_constant__ CUtensorMap vmap, const TcParams p) {
  constexpr int kHalves = D / 64;
  constexpr int kBoxBytes = 128 * 128;             // 128 rows of 128 bytes
  constexpr int kTileBytes = kHalves * kBoxBytes;  // a Q, K or V tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t q_smem = smem_u32(smem);
  const uint32_t k_smem = q_smem + kTileBytes;                 // [kTcStages]
  const uint32_t v_smem = k_smem + kTcStages * kTileBytes;     // [kTcStages]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (1 + 2 * kTcStages) * kTileBytes);
  enum { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, S_FULL = 9, P_FULL = 11, O_FULL = 13, N_BARS = 15 };
  float* xchg = reinterpret_cast<float*>(bars + N_BARS);       // [2 groups][128 rows][m_ref, l]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xchg + 4 * kTcRows);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < N_BARS; ++i) mbar_init(bar(i), (i == P_FULL || i == P_FULL + 1) ? kTcSoftmaxWarps / 2 : 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&qmap)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&kmap)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&vmap)) : "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_s[2] = {tmem, tmem + 128u};
  const uint32_t t_o[2] = {tmem + 256u, tmem + 256u + (uint32_t)D};

  // Longest query blocks first over the WHOLE launch (all heads' last block, then all heads' last but one, ...): the
  // CTAs are handed out in this order as SMs come free, which is longest-processing-time-first scheduling.  (With
  // the blocks of one head in a row, the last heads' long blocks started late: 16 % of the SM time stood idle.)
  const int heads_all = p.Hq * p.B;
  const int mb = p.m_blocks - 1 - (int)(blockIdx.x / heads_all);
  const int hq = (int)(blockIdx.x % heads_all) % p.Hq;
  const int b = (int)(blockIdx.x % heads_all) / p.Hq;
  const int hkv = hq / p.R;
  const int m0 = mb * kTcRows;
  const int last_row = min(m0 + kTcRows, p.T) - 1;
  const int keys = min(p.n_keys, p.start_pos + last_row + 1);
  const int n_tiles = (keys + kTcKeys - 1) / kTcKeys;
  bool ok = true;

  if (warp == 0) {
    // ---- producer ----
    const uint64_t policy = l2_evict_first_policy();
    if (lane == 0) {
      mbar_expect_tx(bar(Q_FULL), kTileBytes);
#pragma unroll
      for (int h = 0; h < kHalves; ++h) tma_load_4d(q_smem + h * kBoxBytes, &qmap, bar(Q_FULL), h * 64, m0, hq, b, policy);
    }
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j % kTcStages;
      const uint32_t par = ((j / kTcStages) - 1) & 1;
      if (j >= kTcStages && !mbar_wait_bounded(bar(K_EMPTY + s), par)) { ok = false; break; }
      if (lane == 0) {
        mbar_expect_tx(bar(K_FULL + s), kTileBytes);
#pragma unroll
        for (int h = 0; h < kHalves; ++h)
          tma_load_4d(k_smem + s * kTileBytes + h * kBoxBytes, &kmap, bar(K_FULL + s), h * 64, j * kTcKeys, hkv, b, policy);
      }
      if (j >= kTcStages && !mbar_wait_bounded(bar(V_EMPTY + s), par)) { ok = false; break; }
      if (lane == 0) {
        mbar_expect_tx(bar(V_FULL + s), kTileBytes);
#pragma unroll
        for (int h = 0; h < kHalves; ++h)
          tma_load_4d(v_smem + s * kTileBytes + h * kBoxBytes, &vmap, bar(V_FULL + s), h * 64, j * kTcKeys, hkv, b, policy);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ---- MMA issue (lane 0), the whole warp takes the waits ----
    constexpr uint32_t idesc_qk = instr_desc(kTcRows, kTcKeys, false);
    constexpr uint32_t idesc_pv = instr_desc(kTcRows, D, true);
    const uint32_t elected = lane == 0 ? 1u : 0u;
    const uint64_t q_desc = smem_desc(q_smem, 16, 1024);
    const uint64_t k_desc = smem_desc(k_smem, 16, 1024);
    const uint64_t v_desc = smem_desc(v_smem, kBoxBytes, 1024);
    auto issue_s = [&](int j) {
      const int s = j % kTcStages;
      const uint64_t kd = k_desc + (uint64_t)((s * kTileBytes) >> 4);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint64_t step = (uint64_t)(((ks >> 2) * kBoxBytes + (ks & 3) * 32) / 16);
        mma_ss(t_s[j & 1], q_desc + step, kd + step, idesc_qk, ks > 0, elected);
      }
      tc_commit(bar(S_FULL + (j & 1)), elected);
      tc_commit(bar(K_EMPTY + s), elected);
    };
    if (!mbar_wait_bounded(bar(Q_FULL), 0)) ok = false;
    if (ok && !mbar_wait_bounded(bar(K_FULL), 0)) ok = false;
    if (ok) {
      tc_fence_after();
      issue_s(0);
    }
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j % kTcStages;
      if (j + 1 < n_tiles) {
        if (!mbar_wait_bounded(bar(K_FULL + (j + 1) % kTcStages), ((j + 1) / kTcStages) & 1)) { ok = false; break; }
        tc_fence_after();
        issue_s(j + 1);
      }
      // O_e += P_j V_j (e = j % 2) once P_j is in TMEM (any rescaling of O_e happened before that) and V_j in
      // shared memory
      if (!mbar_wait_bounded(bar(P_FULL + (j & 1)), (j >> 1) & 1)) { ok = false; break; }
      if (!mbar_wait_bounded(bar(V_FULL + s), (j / kTcStages) & 1)) { ok = false; break; }
      tc_fence_after();
      {
        const uint64_t vd = v_desc + (uint64_t)((s * kTileBytes) >> 4);
#pragma unroll
        for (int kk = 0; kk < kTcKeys / 16; ++kk)
          mma_ts(t_o[j & 1], t_s[j & 1] + kk * 8, vd + (uint64_t)(kk * 128), idesc_pv, (j > 1 || kk > 0) ? 1u : 0u, elected);
        tc_commit(bar(O_FULL + (j & 1)), elected);
        tc_commit(bar(V_EMPTY + s), elected);
      }
    }
  } else {
    // ---- softmax and output: group e = tiles j % 2 == e; thread owns query row r of its group's tiles ----
    const int q4 = warp & 3;                       // TMEM lane quarter this warp may touch
    const int e = (warp - 2) >> 2;                 // warps 2-5: even tiles, warps 6-9: odd tiles
    const int r = q4 * 32 + lane;
    const int t = m0 + r;                          // query index
    const int limit = p.start_pos + t;             // last key this row may see
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    const uint32_t ts = t_s[e] + lane_addr, to = t_o[e] + lane_addr;
    constexpr float kLazy = 8.f;                   // log2 of how far the running maximum may outgrow m_ref
    float m_ref = -INFINITY, l_run = 0.f;
    int done = 0;                                  // tiles of this group so far
    for (int j = e; j < n_tiles && ok; j += 2, ++done) {
      if (!mbar_wait_bounded(bar(S_FULL + e), done & 1)) { ok = false; break; }
      tc_fence_after();
      const int j0 = j * kTcKeys;
      const bool edge = j0 + kTcKeys - 1 > p.start_pos + m0 || j0 + kTcKeys > p.n_keys;  // some row of the block is cut
      uint32_t x[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(ts + c * 32, x[c]);
      tc_wait_ld();
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (edge) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = j0 + c * 32 + i;
            if (key > limit || key >= p.n_keys) x[c][i] = 0xff800000u;  // -inf
          }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          mx4[(i >> 1) & 3] = fmax3(mx4[(i >> 1) & 3], __uint_as_float(x[c][i]), __uint_as_float(x[c][i + 1]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2e;
      // Move the reference maximum (and rescale this warp's rows of O_e) only when some row needs it.
      if (__any_sync(kFullMask, mx > m_ref + kLazy)) {
        const float m_new = fmaxf(m_ref, mx);
        const float alpha = m_new == -INFINITY ? 1.f : fast_exp2(m_ref - m_new);
        if (done > 0) {
          // O_e holds the products of this group's earlier tiles once their MMA has completed
          if (!mbar_wait_bounded(bar(O_FULL + e), (done - 1) & 1)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t y[32];
            tmem_ld32(to + c * 32, y);
            tc_wait_ld();
            uint32_t lo[16], hi[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              lo[i] = __float_as_uint(__uint_as_float(y[i]) * alpha);
              hi[i] = __float_as_uint(__uint_as_float(y[16 + i]) * alpha);
            }
            tmem_st16(to + c * 32, lo);
            tmem_st16(to + c * 32 + 16, hi);
          }
          l_run *= alpha;
        }
        m_ref = m_new;
      }
      const float mu = m_ref == -INFINITY ? 0.f : m_ref;
      const unsigned long long scale2 = f2_packf(p.scale_log2e, p.scale_log2e), nmu2 = f2_packf(-mu, -mu);
      unsigned long long ps2[4] = {0ull, 0ull, 0ull, 0ull};   // four fp32 pairs of partial row sums
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
        // in stages over the whole chunk, so that the 32 exponentials are issued back to back
        unsigned long long t2[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) t2[i] = f2_fma(f2_pack(x[c][2 * i], x[c][2 * i + 1]), scale2, nmu2);
        float pe[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float t0, t1;
          f2_unpack(t2[i], t0, t1);
          pe[2 * i] = fast_exp2(t0);
          pe[2 * i + 1] = fast_exp2(t1);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          ps2[i & 3] = f2_add(ps2[i & 3], f2_packf(pe[2 * i], pe[2 * i + 1]));
          pk[i] = pack_bf16x2(pe[2 * i], pe[2 * i + 1]);
        }
        tmem_st16(ts + c * 16, pk);                // P_j: 64 packed columns over the first 64 of S_j
      }
      {
        float a0, a1, b0, b1;
        f2_unpack(f2_add(ps2[0], ps2[1]), a0, a1);
        f2_unpack(f2_add(ps2[2], ps2[3]), b0, b1);
        l_run += (a0 + a1) + (b0 + b1);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(P_FULL + e));
    }
    // this group's last product
    if (ok && done > 0 && !mbar_wait_bounded(bar(O_FULL + e), (done - 1) & 1)) ok = false;
    tc_fence_after();
    // Merge the two groups' partial results of a row like two split-KV partials; each of the two threads of a row
    // writes one half of the output columns.
    xchg[(e * kTcRows + r) * 2] = m_ref;
    xchg[(e * kTcRows + r) * 2 + 1] = l_run;
    asm volatile("bar.sync 1, %0;" ::"r"(32 * kTcSoftmaxWarps) : "memory");
    const float m_other = xchg[((e ^ 1) * kTcRows + r) * 2], l_other = xchg[((e ^ 1) * kTcRows + r) * 2 + 1];
    const float m_all = fmaxf(m_ref, m_other);
    const float a_me = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - m_all);
    const float a_ot = m_other == -INFINITY ? 0.f : fast_exp2(m_other - m_all);
    const float l_all = l_run * a_me + l_other * a_ot;
    const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
    constexpr int kOHalf = D / 2;
    const bool any_me = __any_sync(kFullMask, a_me != 0.f), any_ot = __any_sync(kFullMask, a_ot != 0.f);
    // The merged rows go through shared memory: a thread holds 64 or 32 columns of ONE row, and storing them straight
    // to global memory makes every store instruction of a warp touch 32 rows (32 sectors for 128 bytes of payload;
    // that epilogue took 5.9 us of a CTA's life, as long as four tiles of the main loop).  The K and V stages are
    // free by now: both groups have seen their last product complete before the barrier above.  Rows are 16 bytes
    // further apart than their length, so that the 16-byte stores of eight neighbouring rows fall into eight
    // different bank groups.
    constexpr int kPitch = D * 2 + 16;
    uint8_t* stage = smem + kTileBytes;
#pragma unroll
    for (int c = 0; c < kOHalf / 32; ++c) {
      uint32_t y0[32], y1[32];
      // (a group without tiles never wrote its accumulator: its columns are not read, let alone used)
      if (any_me) tmem_ld32(t_o[e] + lane_addr + e * kOHalf + c * 32, y0);
      if (any_ot) tmem_ld32(t_o[e ^ 1] + lane_addr + e * kOHalf + c * 32, y1);
      tc_wait_ld();
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float v0 = 0.f, v1 = 0.f;
        if (a_me != 0.f) {
          v0 = __uint_as_float(y0[i]) * a_me;
          v1 = __uint_as_float(y0[i + 1]) * a_me;
        }
        if (a_ot != 0.f) {
          v0 = fmaf(__uint_as_float(y1[i]), a_ot, v0);
          v1 = fmaf(__uint_as_float(y1[i + 1]), a_ot, v1);
        }
        w[i >> 1] = pack_bf16x2(v0 * inv, v1 * inv);
      }
      uint4* dst = reinterpret_cast<uint4*>(stage + r * kPitch + (e * kOHalf + c * 32) * 2);
#pragma unroll
      for (int q = 0; q < 4; ++q) dst[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
    }
    asm volatile("bar.sync 1, %0;" ::"r"(32 * kTcSoftmaxWarps) : "memory");
    // coalesced: 16-byte chunks, a row's chunks on neighbouring threads
    constexpr int kChunks = D * 2 / 16;
    const int sidx = (int)threadIdx.x - 64;   // 0 .. 255 over the softmax warps
    __nv_bfloat16* obase = p.out + (long long)b * p.o_sb + (long long)hq * p.o_sh;
    for (int id = sidx; id < kTcRows * kChunks; id += 32 * kTcSoftmaxWarps) {
      const int row = id / kChunks, ch = id % kChunks;
      if (m0 + row < p.T)
        *reinterpret_cast<uint4*>(obase + (long long)(m0 + row) * p.o_st + ch * 8) =
            *reinterpret_cast<const uint4*>(stage + row * kPitch + ch * 16);
    }
  }
  if (!ok && lane == 0 && p.status) atomicExch(p.status, (int)L3CI_ERR_DEVICE_WAIT);
  // Every thread comes here (all waits are bounded); then nothing of this CTA uses TMEM any more.
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

// The same, with TWO query heads of one KV head per CTA (Hq / Hkv even): softmax group e owns head hq0 + e with all
// its key tiles -- its own Q tile, score accumulator S_e, output accumulator O_e -- and the K and V tiles are loaded once
// for both, which halves the traffic from L2 into shared memory (1.2 GB a launch at B=4, T=2048 with one head per
// CTA: 5.7 TB/s, enough to make the MMA warp wait for K), halves the number of CTAs and with it the share of their
// start and end in the launch, and needs no merge of two partial results at the end.
template <int D>
__global__ void __launch_bounds__(kTcPairThreads, 1)
prefill_tc_pair_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                  const __grid_constant__ CUtensorMap vmap, const TcParams p) {
  constexpr int kHalves = D / 64;
  constexpr int kBoxBytes = 128 * 128;             // 128 rows of 128 bytes
  constexpr int kTileBytes = kHalves * kBoxBytes;  // a Q, K or V tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t q_smem = smem_u32(smem);
  const uint32_t k_smem = q_smem + 2 * kTileBytes;             // [kTcStages], behind the two Q tiles
  const uint32_t v_smem = k_smem + kTcStages * kTileBytes;     // [kTcStages]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (2 + 2 * kTcStages) * kTileBytes);
  enum { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, S_FULL = 9, P_FULL = 11, O_FULL = 13, N_BARS = 15 };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < N_BARS; ++i) mbar_init(bar(i), (i == P_FULL || i == P_FULL + 1) ? kTcSoftmaxWarps / 2 : 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&qmap)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&kmap)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&vmap)) : "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_s[2] = {tmem, tmem + 128u};
  const uint32_t t_o[2] = {tmem + 256u, tmem + 256u + (uint32_t)D};

  // longest query blocks first over the whole launch (see prefill_tc_kernel)
  const int pairs = p.Hq >> 1;
  const int pairs_all = pairs * p.B;
  const int mb = p.m_blocks - 1 - (int)(blockIdx.x / pairs_all);
  const int hq0 = 2 * ((int)(blockIdx.x % pairs_all) % pairs);   // the CTA's query heads: hq0, hq0 + 1 (R is even)
  const int b = (int)(blockIdx.x % pairs_all) / pairs;
  const int hkv = hq0 / p.R;
  const int m0 = mb * kTcRows;
  const int last_row = min(m0 + kTcRows, p.T) - 1;
  const int keys = min(p.n_keys, p.start_pos + last_row + 1);
  const int n_tiles = (keys + kTcKeys - 1) / kTcKeys;
  bool ok = true;

  // Registers follow the roles: the first warpgroup (producer, MMA warp, two idle warps) hands most of its share to
  // the two softmax warpgroups, whose threads carry a row of 128 scores each.
  // (each role's branch opens with its own setmaxnreg, so that the compiler sees which budget holds where)
  if (warp == 0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kTcPairRegsLow));
    // ---- producer ----
    const uint64_t policy = l2_evict_first_policy();
    if (lane == 0) {
      mbar_expect_tx(bar(Q_FULL), 2 * kTileBytes);
#pragma unroll
      for (int e = 0; e < 2; ++e)
#pragma unroll
        for (int h = 0; h < kHalves; ++h)
          tma_load_4d(q_smem + e * kTileBytes + h * kBoxBytes, &qmap, bar(Q_FULL), h * 64, m0, hq0 + e, b, policy);
    }
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j % kTcStages;
      const uint32_t par = ((j / kTcStages) - 1) & 1;
      if (j >= kTcStages && !mbar_wait_bounded(bar(K_EMPTY + s), par)) { ok = false; break; }
      if (lane == 0) {
        mbar_expect_tx(bar(K_FULL + s), kTileBytes);
#pragma unroll
        for (int h = 0; h < kHalves; ++h)
          tma_load_4d(k_smem + s * kTileBytes + h * kBoxBytes, &kmap, bar(K_FULL + s), h * 64, j * kTcKeys, hkv, b, policy);
      }
      if (j >= kTcStages && !mbar_wait_bounded(bar(V_EMPTY + s), par)) { ok = false; break; }
      if (lane == 0) {
        mbar_expect_tx(bar(V_FULL + s), kTileBytes);
#pragma unroll
        for (int h = 0; h < kHalves; ++h)
          tma_load_4d(v_smem + s * kTileBytes + h * kBoxBytes, &vmap, bar(V_FULL + s), h * 64, j * kTcKeys, hkv, b, policy);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kTcPairRegsLow));
    // ---- MMA issue (lane 0), the whole warp takes the waits ----
    constexpr uint32_t idesc_qk = instr_desc(kTcRows, kTcKeys, false);
    constexpr uint32_t idesc_pv = instr_desc(kTcRows, D, true);
    const uint32_t elected = lane == 0 ? 1u : 0u;
    const uint64_t q_desc = smem_desc(q_smem, 16, 1024);
    const uint64_t k_desc = smem_desc(k_smem, 16, 1024);
    const uint64_t v_desc = smem_desc(v_smem, kBoxBytes, 1024);
    // S_{e,j} = Q_e K_j^T into group e's score accumulator, which held P_{e,j-1}, read by an MMA issued before this one
    auto issue_s = [&](int e, int j) {
      const int s = j % kTcStages;
      const uint64_t qd = q_desc + (uint64_t)((e * kTileBytes) >> 4);
      const uint64_t kd = k_desc + (uint64_t)((s * kTileBytes) >> 4);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint64_t step = (uint64_t)(((ks >> 2) * kBoxBytes + (ks & 3) * 32) / 16);
        mma_ss(t_s[e], qd + step, kd + step, idesc_qk, ks > 0, elected);
      }
      tc_commit(bar(S_FULL + e), elected);
      if (e == 1) tc_commit(bar(K_EMPTY + s), elected);   // both heads have read the K stage
    };
    if (!mbar_wait_bounded(bar(Q_FULL), 0)) ok = false;
    if (ok && !mbar_wait_bounded(bar(K_FULL), 0)) ok = false;
    if (ok) {
      tc_fence_after();
      issue_s(0, 0);
      issue_s(1, 0);
    }
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j % kTcStages;
      if (!mbar_wait_bounded(bar(V_FULL + s), (j / kTcStages) & 1)) { ok = false; break; }
      for (int e = 0; e < 2; ++e) {
        // O_e += P_{e,j} V_j once P_{e,j} is in TMEM (any rescaling of O_e happened before that), then at once the
        // head's next scores, which go where P_{e,j} lay
        if (!mbar_wait_bounded(bar(P_FULL + e), j & 1)) { ok = false; break; }
        tc_fence_after();
        {
          const uint64_t vd = v_desc + (uint64_t)((s * kTileBytes) >> 4);
#pragma unroll
          for (int kk = 0; kk < kTcKeys / 16; ++kk)
            mma_ts(t_o[e], t_s[e] + kk * 8, vd + (uint64_t)(kk * 128), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u, elected);
          tc_commit(bar(O_FULL + e), elected);
          if (e == 1) tc_commit(bar(V_EMPTY + s), elected);
        }
        if (j + 1 < n_tiles) {
          if (e == 0) {
            if (!mbar_wait_bounded(bar(K_FULL + (j + 1) % kTcStages), ((j + 1) / kTcStages) & 1)) { ok = false; break; }
            tc_fence_after();
          }
          issue_s(e, j + 1);
        }
      }
    }
  } else if (warp >= 4) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kTcPairRegsHigh));
    // ---- softmax and output: group e = query head hq0 + e, all key tiles; thread owns query row r ----
    const int q4 = warp & 3;                       // TMEM lane quarter this warp may touch
    const int e = (warp - 4) >> 2;                 // warps 4-7: head hq0, warps 8-11: head hq0 + 1
    const int r = q4 * 32 + lane;
    const int t = m0 + r;                          // query index
    const int limit = p.start_pos + t;             // last key this row may see
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    const uint32_t ts = t_s[e] + lane_addr, to = t_o[e] + lane_addr;
    constexpr float kLazy = 8.f;                   // log2 of how far the running maximum may outgrow m_ref
    float m_ref = -INFINITY, l_run = 0.f;
    int done = 0;                                  // tiles of this group so far
    for (int j = 0; j < n_tiles && ok; ++j, ++done) {
      if (!mbar_wait_bounded(bar(S_FULL + e), done & 1)) { ok = false; break; }
      tc_fence_after();
      const int j0 = j * kTcKeys;
      const bool edge = j0 + kTcKeys - 1 > p.start_pos + m0 || j0 + kTcKeys > p.n_keys;  // some row of the block is cut
      uint32_t x[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(ts + c * 32, x[c]);
      tc_wait_ld();
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (edge) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = j0 + c * 32 + i;
            if (key > limit || key >= p.n_keys) x[c][i] = 0xff800000u;  // -inf
          }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          mx4[(i >> 1) & 3] = fmax3(mx4[(i >> 1) & 3], __uint_as_float(x[c][i]), __uint_as_float(x[c][i + 1]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2e;
      // Move the reference maximum (and rescale this warp's rows of O_e) only when some row needs it.
      if (__any_sync(kFullMask, mx > m_ref + kLazy)) {
        const float m_new = fmaxf(m_ref, mx);
        const float alpha = m_new == -INFINITY ? 1.f : fast_exp2(m_ref - m_new);
        if (done > 0) {
          // O_e holds the products of this group's earlier tiles once their MMA has completed
          if (!mbar_wait_bounded(bar(O_FULL + e), (done - 1) & 1)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t y[32];
            tmem_ld32(to + c * 32, y);
            tc_wait_ld();
            uint32_t lo[16], hi[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              lo[i] = __float_as_uint(__uint_as_float(y[i]) * alpha);
              hi[i] = __float_as_uint(__uint_as_float(y[16 + i]) * alpha);
            }
            tmem_st16(to + c * 32, lo);
            tmem_st16(to + c * 32 + 16, hi);
          }
          l_run *= alpha;
        }
        m_ref = m_new;
      }
      const float mu = m_ref == -INFINITY ? 0.f : m_ref;
      const unsigned long long scale2 = f2_packf(p.scale_log2e, p.scale_log2e), nmu2 = f2_packf(-mu, -mu);
      unsigned long long ps2[4] = {0ull, 0ull, 0ull, 0ull};   // four fp32 pairs of partial row sums
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
        // in stages over the whole chunk, so that the 32 exponentials are issued back to back
        unsigned long long t2[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) t2[i] = f2_fma(f2_pack(x[c][2 * i], x[c][2 * i + 1]), scale2, nmu2);
        float pe[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float t0, t1;
          f2_unpack(t2[i], t0, t1);
          pe[2 * i] = fast_exp2(t0);
          pe[2 * i + 1] = fast_exp2(t1);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          ps2[i & 3] = f2_add(ps2[i & 3], f2_packf(pe[2 * i], pe[2 * i + 1]));
          pk[i] = pack_bf16x2(pe[2 * i], pe[2 * i + 1]);
        }
        tmem_st16(ts + c * 16, pk);                // P_j: 64 packed columns over the first 64 of S_j
      }
      {
        float a0, a1, b0, b1;
        f2_unpack(f2_add(ps2[0], ps2[1]), a0, a1);
        f2_unpack(f2_add(ps2[2], ps2[3]), b0, b1);
        l_run += (a0 + a1) + (b0 + b1);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(P_FULL + e));
    }
    // this head's last product
    if (ok && done > 0 && !mbar_wait_bounded(bar(O_FULL + e), (done - 1) & 1)) ok = false;
    tc_fence_after();
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    // Both heads' MMAs have completed once both groups are here: the K and V stages are free and take the output
    // rows, which leave as 16-byte vectors (a thread holds one row; stored straight to global memory every store
    // instruction of a warp would touch 32 rows).  Rows are 16 bytes further apart than their length, so that the
    // 16-byte stores of eight neighbouring rows fall into eight different bank groups.
    asm volatile("bar.sync 1, %0;" ::"r"(32 * kTcSoftmaxWarps) : "memory");
    constexpr int kPitch = D * 2 + 16;
    uint8_t* stage = smem + 2 * kTileBytes + e * (kTcRows * kPitch);
    static_assert(2 * kTcRows * kPitch <= 2 * kTcStages * kTileBytes, "output staging fits the K and V stages");
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t y[32];
      tmem_ld32(to + c * 32, y);
      tc_wait_ld();
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) w[i >> 1] = pack_bf16x2(__uint_as_float(y[i]) * inv, __uint_as_float(y[i + 1]) * inv);
      uint4* dst = reinterpret_cast<uint4*>(stage + r * kPitch + c * 64);
#pragma unroll
      for (int q = 0; q < 4; ++q) dst[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
    }
    asm volatile("bar.sync %0, %1;" ::"r"(2 + e), "r"(32 * kTcSoftmaxWarps / 2) : "memory");   // this group's 128 threads
    // coalesced: 16-byte chunks, a row's chunks on neighbouring threads
    constexpr int kChunks = D * 2 / 16;
    __nv_bfloat16* obase = p.out + (long long)b * p.o_sb + (long long)(hq0 + e) * p.o_sh;
    for (int id = r; id < kTcRows * kChunks; id += 32 * kTcSoftmaxWarps / 2) {
      const int row = id / kChunks, ch = id % kChunks;
      if (m0 + row < p.T)
        *reinterpret_cast<uint4*>(obase + (long long)(m0 + row) * p.o_st + ch * 8) =
            *reinterpret_cast<const uint4*>(stage + row * kPitch + ch * 16);
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kTcPairRegsLow));   // the two idle warps of the first warpgroup
  }
  if (!ok && lane == 0 && p.status) atomicExch(p.status, (int)L3CI_ERR_DEVICE_WAIT);
  // Every thread comes here (all waits are bounded); then nothing of this CTA uses TMEM any more.
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

// The head-pair kernel as a PERSISTENT grid: one CTA per SM walks a list of (head pair, query block) items.  A CTA's
// start (tensor-memory allocation, and above all the 2.3-3.6 us until Q and the first K tile have landed) and its end
// (output pass) were 5 us of the 22 an item takes on average; here the producer asks for the next item's Q tiles as
// soon as the last scores of this one have been computed, the K / V rings and all barrier phases run on across
// items, and the next item's first scores are computed while the softmax groups still write this one's output.
// Items are dealt statically, longest first, in snake order over the CTAs (round r: item r * G + c for CTA c, then
// r * G + G - 1 - c, ...), which balances like a greedy longest-first deal.  The output leaves through a small
// staging buffer of its own, 32 columns at a time (the K and V stages belong to the next item by then), and it is
// written by a warpgroup of its own (warps 12-15): a softmax group hands over the row sums after its last tile and
// turns to the next item at once instead of waiting for the last product and writing 32 KB itself.
template <int D>
__global__ void __launch_bounds__(kTcPersistThreads, 1)
prefill_tc_persist_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                  const __grid_constant__ CUtensorMap vmap, const TcParams p) {
  constexpr int kHalves = D / 64;
  constexpr int kBoxBytes = 128 * 128;             // 128 rows of 128 bytes
  constexpr int kTileBytes = kHalves * kBoxBytes;  // a Q, K or V tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t q_smem = smem_u32(smem);
  const uint32_t k_smem = q_smem + 2 * kTileBytes;             // [kTcStages], behind the two Q tiles
  const uint32_t v_smem = k_smem + kTcStages * kTileBytes;     // [kTcStages]
  constexpr int kSPitch = 64 + 16;                                 // staging row: 32 output columns + padding
  uint8_t* stage_all = smem + (2 + 2 * kTcStages) * kTileBytes;    // [2 heads][128 rows][kSPitch]
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_all + 2 * kTcRows * kSPitch);
  // Q_EMPTY: the item's last scores have been computed, the Q tiles may take the next item's
  // L_FULL: a head's row sums of the item are in shared memory (its softmax group is done with the item);
  // O_READ: the output warpgroup has the head's O in registers (the accumulator may take the next item's products)
  enum { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, S_FULL = 9, P_FULL = 11, O_FULL = 13, Q_EMPTY = 15,
         L_FULL = 16, O_READ = 18, N_BARS = 20 };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
  float* lrow = reinterpret_cast<float*>(bars + N_BARS + 2);       // [2 heads][128 rows]
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < N_BARS; ++i) mbar_init(bar(i), (i == P_FULL || i == P_FULL + 1 || i >= L_FULL) ? kTcSoftmaxWarps / 2 : 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&qmap)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&kmap)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&vmap)) : "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_s[2] = {tmem, tmem + 128u};
  const uint32_t t_o[2] = {tmem + 256u, tmem + 256u + (uint32_t)D};

  // Items in launch order: longest query blocks first over all head pairs (see prefill_tc_kernel); this CTA's
  // item of round r is r * G + c (r even) or r * G + G - 1 - c (r odd), c = blockIdx.x, G = gridDim.x.
  const int pairs = p.Hq >> 1;
  const int pairs_all = pairs * p.B;
  const long long n_items = (long long)pairs_all * p.m_blocks;
  struct Item { int hq0, b, hkv, m0, n_tiles; bool valid; };
  auto item_of = [&](int round) {
    Item it;
    const long long idx = (long long)round * gridDim.x + ((round & 1) ? gridDim.x - 1 - blockIdx.x : blockIdx.x);
    it.valid = idx < n_items;
    const int mb = p.m_blocks - 1 - (int)(idx / pairs_all);
    it.hq0 = 2 * ((int)(idx % pairs_all) % pairs);
    it.b = (int)(idx % pairs_all) / pairs;
    it.hkv = it.hq0 / p.R;
    it.m0 = mb * kTcRows;
    const int last_row = min(it.m0 + kTcRows, p.T) - 1;
    const int keys = min(p.n_keys, p.start_pos + last_row + 1);
    it.n_tiles = (keys + kTcKeys - 1) / kTcKeys;
    return it;
  };
  bool ok = true;

  // Registers follow the roles: the first warpgroup (producer, MMA warp, two idle warps) hands most of its share to
  // the two softmax warpgroups, whose threads carry a row of 128 scores each.
  // (each role's branch opens with its own setmaxnreg, so that the compiler sees which budget holds where)
  if (warp == 0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kTcPersistRegsLow));
    // ---- producer ----
    const uint64_t policy = l2_evict_first_policy();
    int fill = 0;   // K (and V) tiles asked for so far, over all items: stage and phase follow from it
    for (int round = 0; ok; ++round) {
      const Item it = item_of(round);
      if (!it.valid) break;
      if (round > 0 && !mbar_wait_bounded(bar(Q_EMPTY), (round - 1) & 1)) { ok = false; break; }
      if (lane == 0) {
        mbar_expect_tx(bar(Q_FULL), 2 * kTileBytes);
#pragma unroll
        for (int e = 0; e < 2; ++e)
#pragma unroll
          for (int h = 0; h < kHalves; ++h)
            tma_load_4d(q_smem + e * kTileBytes + h * kBoxBytes, &qmap, bar(Q_FULL), h * 64, it.m0, it.hq0 + e, it.b, policy);
      }
      for (int j = 0; j < it.n_tiles && ok; ++j, ++fill) {
        const int s = fill % kTcStages;
        const uint32_t par = ((fill / kTcStages) - 1) & 1;
        if (fill >= kTcStages && !mbar_wait_bounded(bar(K_EMPTY + s), par)) { ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(bar(K_FULL + s), kTileBytes);
#pragma unroll
          for (int h = 0; h < kHalves; ++h)
            tma_load_4d(k_smem + s * kTileBytes + h * kBoxBytes, &kmap, bar(K_FULL + s), h * 64, j * kTcKeys, it.hkv, it.b, policy);
        }
        if (fill >= kTcStages && !mbar_wait_bounded(bar(V_EMPTY + s), par)) { ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(bar(V_FULL + s), kTileBytes);
#pragma unroll
          for (int h = 0; h < kHalves; ++h)
            tma_load_4d(v_smem + s * kTileBytes + h * kBoxBytes, &vmap, bar(V_FULL + s), h * 64, j * kTcKeys, it.hkv, it.b, policy);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kTcPersistRegsLow));
    // ---- MMA issue (lane 0), the whole warp takes the waits ----
    constexpr uint32_t idesc_qk = instr_desc(kTcRows, kTcKeys, false);
    constexpr uint32_t idesc_pv = instr_desc(kTcRows, D, true);
    const uint32_t elected = lane == 0 ? 1u : 0u;
    const uint64_t q_desc = smem_desc(q_smem, 16, 1024);
    const uint64_t k_desc = smem_desc(k_smem, 16, 1024);
    const uint64_t v_desc = smem_desc(v_smem, kBoxBytes, 1024);
    // S_{e,g} = Q_e K^T (g: tile number over all items) into head e's score accumulator, which held P_{e,g-1}, read by
    // an MMA issued before this one; `last`: the item's last tile, after which the Q tiles are free
    auto issue_s = [&](int e, int g, bool last) {
      const int s = g % kTcStages;
      const uint64_t qd = q_desc + (uint64_t)((e * kTileBytes) >> 4);
      const uint64_t kd = k_desc + (uint64_t)((s * kTileBytes) >> 4);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint64_t step = (uint64_t)(((ks >> 2) * kBoxBytes + (ks & 3) * 32) / 16);
        mma_ss(t_s[e], qd + step, kd + step, idesc_qk, ks > 0, elected);
      }
      tc_commit(bar(S_FULL + e), elected);
      if (e == 1) {
        tc_commit(bar(K_EMPTY + s), elected);   // both heads have read the K stage
        if (last) tc_commit(bar(Q_EMPTY), elected);
      }
    };
    int g0 = 0;   // tiles of the items before this one
    for (int round = 0; ok; ++round) {
      const Item it = item_of(round);
      if (!it.valid) break;
      const int n_tiles = it.n_tiles;
      if (!mbar_wait_bounded(bar(Q_FULL), round & 1)) { ok = false; break; }
      if (!mbar_wait_bounded(bar(K_FULL + g0 % kTcStages), (g0 / kTcStages) & 1)) { ok = false; break; }
      tc_fence_after();
      issue_s(0, g0, n_tiles == 1);
      issue_s(1, g0, n_tiles == 1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int g = g0 + j, s = g % kTcStages;
        if (!mbar_wait_bounded(bar(V_FULL + s), (g / kTcStages) & 1)) { ok = false; break; }
        for (int e = 0; e < 2; ++e) {
          // O_e += P_{e,g} V once P_{e,g} is in TMEM (any rescaling of O_e happened before that; on an item's first
          // tile the output warpgroup must have read the previous item's O_e), then at once the head's next scores,
          // which go where P_{e,g} lay
          if (!mbar_wait_bounded(bar(P_FULL + e), g & 1)) { ok = false; break; }
          if (j == 0 && round > 0 && !mbar_wait_bounded(bar(O_READ + e), (round - 1) & 1)) { ok = false; break; }
          tc_fence_after();
          {
            const uint64_t vd = v_desc + (uint64_t)((s * kTileBytes) >> 4);
#pragma unroll
            for (int kk = 0; kk < kTcKeys / 16; ++kk)
              mma_ts(t_o[e], t_s[e] + kk * 8, vd + (uint64_t)(kk * 128), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u, elected);
            tc_commit(bar(O_FULL + e), elected);
            if (e == 1) tc_commit(bar(V_EMPTY + s), elected);
          }
          if (j + 1 < n_tiles) {
            if (e == 0) {
              if (!mbar_wait_bounded(bar(K_FULL + (g + 1) % kTcStages), ((g + 1) / kTcStages) & 1)) { ok = false; break; }
              tc_fence_after();
            }
            issue_s(e, g + 1, j + 2 == n_tiles);
          }
        }
      }
      g0 += n_tiles;
    }
  } else if (warp >= 4 && warp < 4 + kTcSoftmaxWarps) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kTcPersistRegsHigh));
    // ---- softmax and output: group e = query head hq0 + e, all key tiles; thread owns query row r ----
    const int q4 = warp & 3;                       // TMEM lane quarter this warp may touch
    const int e = (warp - 4) >> 2;                 // warps 4-7: head hq0, warps 8-11: head hq0 + 1
    const int r = q4 * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    const uint32_t ts = t_s[e] + lane_addr, to = t_o[e] + lane_addr;
    constexpr float kLazy = 8.f;                   // log2 of how far the running maximum may outgrow m_ref
    int g0 = 0;                                    // tiles of the items before this one
    for (int round = 0; ok; ++round) {
    const Item it = item_of(round);
    if (!it.valid) break;
    const int m0 = it.m0, n_tiles = it.n_tiles;
    const int limit = p.start_pos + m0 + r;        // last key this row may see
    float m_ref = -INFINITY, l_run = 0.f;
    int done = 0;                                  // tiles of this item so far
    for (int j = 0; j < n_tiles && ok; ++j, ++done) {
      if (!mbar_wait_bounded(bar(S_FULL + e), (g0 + j) & 1)) { ok = false; break; }
      tc_fence_after();
      const int j0 = j * kTcKeys;
      const bool edge = j0 + kTcKeys - 1 > p.start_pos + m0 || j0 + kTcKeys > p.n_keys;  // some row of the block is cut
      uint32_t x[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(ts + c * 32, x[c]);
      tc_wait_ld();
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (edge) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = j0 + c * 32 + i;
            if (key > limit || key >= p.n_keys) x[c][i] = 0xff800000u;  // -inf
          }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          mx4[(i >> 1) & 3] = fmax3(mx4[(i >> 1) & 3], __uint_as_float(x[c][i]), __uint_as_float(x[c][i + 1]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2e;
      // Move the reference maximum (and rescale this warp's rows of O_e) only when some row needs it.
      if (__any_sync(kFullMask, mx > m_ref + kLazy)) {
        const float m_new = fmaxf(m_ref, mx);
        const float alpha = m_new == -INFINITY ? 1.f : fast_exp2(m_ref - m_new);
        if (done > 0) {
          // O_e holds the products of this group's earlier tiles once their MMA has completed
          if (!mbar_wait_bounded(bar(O_FULL + e), (g0 + done - 1) & 1)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t y[32];
            tmem_ld32(to + c * 32, y);
            tc_wait_ld();
            uint32_t lo[16], hi[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              lo[i] = __float_as_uint(__uint_as_float(y[i]) * alpha);
              hi[i] = __float_as_uint(__uint_as_float(y[16 + i]) * alpha);
            }
            tmem_st16(to + c * 32, lo);
            tmem_st16(to + c * 32 + 16, hi);
          }
          l_run *= alpha;
        }
        m_ref = m_new;
      }
      const float mu = m_ref == -INFINITY ? 0.f : m_ref;
      const unsigned long long scale2 = f2_packf(p.scale_log2e, p.scale_log2e), nmu2 = f2_packf(-mu, -mu);
      unsigned long long ps2[4] = {0ull, 0ull, 0ull, 0ull};   // four fp32 pairs of partial row sums
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
        // in stages over the whole chunk, so that the 32 exponentials are issued back to back
        unsigned long long t2[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) t2[i] = f2_fma(f2_pack(x[c][2 * i], x[c][2 * i + 1]), scale2, nmu2);
        float pe[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float t0, t1;
          f2_unpack(t2[i], t0, t1);
          pe[2 * i] = fast_exp2(t0);
          pe[2 * i + 1] = fast_exp2(t1);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          ps2[i & 3] = f2_add(ps2[i & 3], f2_packf(pe[2 * i], pe[2 * i + 1]));
          pk[i] = pack_bf16x2(pe[2 * i], pe[2 * i + 1]);
        }
        tmem_st16(ts + c * 16, pk);                // P_j: 64 packed columns over the first 64 of S_j
      }
      {
        float a0, a1, b0, b1;
        f2_unpack(f2_add(ps2[0], ps2[1]), a0, a1);
        f2_unpack(f2_add(ps2[2], ps2[3]), b0, b1);
        l_run += (a0 + a1) + (b0 + b1);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(P_FULL + e));
    }
    if (!ok) break;
    // The row sums go to the output warpgroup (which has read the previous item's before it arrived on O_READ), and
    // this group turns to the next item: the last product and the output pass are no longer its business.
    if (round > 0 && !mbar_wait_bounded(bar(O_READ + e), (round - 1) & 1)) { ok = false; break; }
    lrow[e * kTcRows + r] = l_run;
    __syncwarp();
    if (lane == 0) mbar_arrive(bar(L_FULL + e));
    g0 += n_tiles;
    }   // items
  } else if (warp >= 4 + kTcSoftmaxWarps) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kTcPersistRegsOut));
    // ---- output: thread owns row r of both heads' O, one head after the other ----
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    int g0 = 0;
    for (int round = 0; ok; ++round) {
      const Item it = item_of(round);
      if (!it.valid) break;
      const int m0 = it.m0;
      for (int e = 0; e < 2 && ok; ++e) {
        if (!mbar_wait_bounded(bar(L_FULL + e), round & 1)) { ok = false; break; }
        const float l_all = lrow[e * kTcRows + r];
        const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
        if (!mbar_wait_bounded(bar(O_FULL + e), (g0 + it.n_tiles - 1) & 1)) { ok = false; break; }   // the head's last product
        tc_fence_after();
        // 32 columns at a time through the staging rows (a thread holds one row; stored straight to global memory
        // every store instruction of a warp would touch 32 rows): out of tensor memory, scaled, packed, into shared
        // memory; then 16-byte chunks, a row's four chunks on neighbouring threads.
        uint8_t* stage = stage_all + e * (kTcRows * kSPitch);
        __nv_bfloat16* obase = p.out + (long long)it.b * p.o_sb + (long long)(it.hq0 + e) * p.o_sh;
        const uint32_t to = t_o[e] + lane_addr;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t y[32];
          tmem_ld32(to + c * 32, y);
          tc_wait_ld();
          if (c == D / 32 - 1) {   // O_e is in registers: the accumulator may take the next item's first product
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(O_READ + e));
          }
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) w[i >> 1] = pack_bf16x2(__uint_as_float(y[i]) * inv, __uint_as_float(y[i + 1]) * inv);
          uint4* dst = reinterpret_cast<uint4*>(stage + r * kSPitch);
#pragma unroll
          for (int q = 0; q < 4; ++q) dst[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
          asm volatile("bar.sync 2, 128;" ::: "memory");   // the output warpgroup
#pragma unroll
          for (int id = r; id < kTcRows * 4; id += 128) {
            const int row = id >> 2, ch = id & 3;
            if (m0 + row < p.T)
              *reinterpret_cast<uint4*>(obase + (long long)(m0 + row) * p.o_st + c * 32 + ch * 8) =
                  *reinterpret_cast<const uint4*>(stage + row * kSPitch + ch * 16);
          }
          asm volatile("bar.sync 2, 128;" ::: "memory");   // the rows may be written again
        }
      }
      g0 += it.n_tiles;
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kTcPersistRegsLow));   // the two idle warps of the first warpgroup
  }
  if (!ok && lane == 0 && p.status) atomicExch(p.status, (int)L3CI_ERR_DEVICE_WAIT);
  // Every thread comes here (all waits are bounded); then nothing of this CTA uses TMEM any more.
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

// Launch for prompts of at least one full block; called by l3ci_prefill_attention.
int launch_prefill_tc(const l3ci_prefill_args* a) {
  const int B = a->B, Hq = a->Hq, Hkv = a->Hkv, D = a->D, T = a->T, S = a->n_keys;
  if (!aligned16(a->q) || a->q_st % 8 || (Hq > 1 && a->q_sh % 8) || (B > 1 && a->q_sb % 8) || a->q_st <= 0 ||
      (Hq > 1 && a->q_sh <= 0) || (B > 1 && a->q_sb <= 0))
    return -1;  // Q cannot be described to the copy engine: the caller falls back to the other kernel
  if (!aligned16(a->out) || a->o_st % 8 || a->o_sh % 8 || a->o_sb % 8) return -1;  // output rows are written as 16-byte vectors
  CUtensorMap qmap, kmap, vmap;
  if (int st = make_kv_map(&qmap, a->q, D, T, Hq, B, a->q_st, a->q_sh, a->q_sb, kTcRows, 1)) return st;
  if (int st = make_kv_map(&kmap, a->k, D, S, Hkv, B, a->k_st, a->k_sh, a->k_sb, kTcKeys, 1)) return st;
  if (int st = make_kv_map(&vmap, a->v, D, S, Hkv, B, a->v_st, a->v_sh, a->v_sb, kTcKeys, 1)) return st;
  TcParams p;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.R = Hq / Hkv; p.T = T; p.n_keys = S; p.start_pos = a->start_pos;
  p.m_blocks = (T + kTcRows - 1) / kTcRows;
  p.o_sb = a->o_sb; p.o_sh = a->o_sh; p.o_st = a->o_st;
  const float scale = a->scale > 0.f ? a->scale : 1.0f / sqrtf((float)D);
  p.scale_log2e = scale * 1.4426950408889634f;
  p.status = a->status;
  const bool pair = (Hq / Hkv) % 2 == 0;   // two query heads of a KV head per CTA
  const long long items = (long long)B * (pair ? Hq / 2 : Hq) * p.m_blocks;
  if (items > 0x7fffffffLL) return fail(L3CI_ERR_INVALID, "prefill_attention: too many query blocks (%lld)", items);
  const int sms = sm_count();
  // More items than SMs: the persistent form (one CTA per SM walks its items); otherwise a CTA per item.
  static const bool no_persist = getenv("L3CI_PF_NO_PERSIST") != nullptr;
  const bool persist = pair && sms > 0 && items > sms && !no_persist;
  const long long ctas = persist ? sms : items;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(a->stream);
  const size_t tile = (size_t)(D / 64) * 128 * 128;
  const size_t smem = persist ? 1024 + 6 * tile + 2 * kTcRows * 80 + 20 * 8 + 16 + 2 * kTcRows * 4
                              : 1024 + ((pair ? 2 : 1) + 2 * kTcStages) * tile + 15 * 8 + 4 * kTcRows * 4 + 16;
  static bool configured[3][2][64] = {{{false}}};
  int dev = 0;
  L3CI_CUDA_TRY(cudaGetDevice(&dev));
  const int di = D == 64 ? 0 : 1, ki = persist ? 2 : pair ? 1 : 0;
  if (dev < 0 || dev >= 64 || !configured[ki][di][dev]) {
    const void* fn = persist ? (D == 64 ? (const void*)prefill_tc_persist_kernel<64> : (const void*)prefill_tc_persist_kernel<128>)
                     : pair  ? (D == 64 ? (const void*)prefill_tc_pair_kernel<64> : (const void*)prefill_tc_pair_kernel<128>)
                             : (D == 64 ? (const void*)prefill_tc_kernel<64> : (const void*)prefill_tc_kernel<128>);
    L3CI_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev >= 0 && dev < 64) configured[ki][di][dev] = true;
  }
  if (persist) {
    if (D == 64) prefill_tc_persist_kernel<64><<<(unsigned)ctas, kTcPersistThreads, smem, stream>>>(qmap, kmap, vmap, p);
    else prefill_tc_persist_kernel<128><<<(unsigned)ctas, kTcPersistThreads, smem, stream>>>(qmap, kmap, vmap, p);
  } else if (pair) {
    if (D == 64) prefill_tc_pair_kernel<64><<<(unsigned)ctas, kTcPairThreads, smem, stream>>>(qmap, kmap, vmap, p);
    else prefill_tc_pair_kernel<128><<<(unsigned)ctas, kTcPairThreads, smem, stream>>>(qmap, kmap, vmap, p);
  } else if (D == 64) prefill_tc_kernel<64><<<(unsigned)ctas, kTcThreads, smem, stream>>>(qmap, kmap, vmap, p);
  else prefill_tc_kernel<128><<<(unsigned)ctas, kTcThreads, smem, stream>>>(qmap, kmap, vmap, p);
  L3CI_CHECK_LAUNCH("prefill_tc_kernel");
  return L3CI_OK;
}

}  // namespace l3ci
