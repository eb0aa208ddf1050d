// Split-KV flash-decode attention for sm_100a: one query token per sequence against a bf16
// GQA KV cache, head size 64 or 128, one launch per call.
//
// Replaces flash_attention_decode with its split-KV and combine kernels
// (custom_kernels/custom_kernels.cu:13-177, 179-223, 233-338).  What is kept from the
// reference: every K/V byte is read from HBM once per KV head and shared by the R query heads
// of the group, fp32 softmax statistics, and a log-sum-exp combine of partial results.
// What is different:
//
//  * Persistent grid.  The work is the list of "columns" (sequence b, head group g, tile j of
//    kTile tokens); a column covers the same tokens for HG = gcd(Hkv, 8) neighbouring KV heads.
//    The list is cut into gridDim.x equal contiguous ranges, so every SM streams the same number
//    of bytes whatever the sequence lengths are.  A CTA has HG consumer warps and a producer
//    warp; consumer w owns KV head g*HG + w of every column, so a CTA walks HG*D*2 contiguous
//    bytes per token.
//  * The producer warp fills a kStages-deep ring of CTA-wide stages with bulk tensor copies
//    (cp.async.bulk.tensor, one box of all HG heads per 64-column half of K and of V, 128-byte
//    swizzle); full / empty mbarriers pair it with the consumers, no CTA-wide barrier in the loop.
//  * Q.K^T and P.V run on tensor cores (mma.sync m16n8k16 bf16) in transposed form, tokens and
//    output columns on the 16 rows of a tile and the query heads of the group on its 8 columns, so
//    that up to 8 query heads per KV head leave no padding; online softmax statistics live in
//    registers.  Tensor cores are there to spare issue slots, not for throughput: the kernel
//    waits on HBM.
//  * A (sequence, head) unit that is cut by a range boundary leaves an fp32 (m, l, o) record per
//    CTA and a count on the unit's arrival counter.  When a warp has streamed its whole range it
//    comes back to the (at most two) shared units it took part in, waits until all their records
//    are there and merges ITS SLICE of the output columns, lanes spread over the records, so the
//    merge costs one or two memory round trips however many CTAs share the unit.  The grid is
//    launched cooperatively (never more CTAs than fit on the device at once), which is what makes
//    waiting on other CTAs legitimate.  The last warp to leave resets the counter, so scratch stays
//    ready for the next call.
//  * Every wait (on an mbarrier, on an arrival counter) is bounded; if it runs out the warp records
//    L3CI_ERR_DEVICE_WAIT in the scratch header and moves on.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <math.h>

#include <mutex>

#include "bf16x8.cuh"
#include "flash_decode_plan.h"
#include "host_common.h"
#include "ptx_sm100.cuh"
#include "tensor_map.h"
#include "warp_reduce.cuh"

namespace l3ci {
namespace {

constexpr int kStages = 3;            // columns (one tile per head of the group) resident per CTA
constexpr int kStageBytes = 8192;     // K tile + V tile of one head in a stage
constexpr bool kScoresAhead = true;   // compute a tile's scores while the previous tile is still in its softmax
constexpr int kHeaderBytes = 256;     // scratch header: status word

template <int D>
struct FdCfg {
  static_assert(D == 64 || D == 128, "head size");
  static constexpr int kTile = fd_tile_tokens(D);         // tokens per tile
  static constexpr int kHalves = D / 64;                  // 128-byte column blocks per row
  static constexpr int kBoxBytes = kTile * 128;           // one TMA box: kTile rows of 128 bytes
  static constexpr int kKBytes = kHalves * kBoxBytes;     // K part of a stage
  static_assert(2 * kKBytes == kStageBytes, "stage size");
  static constexpr int KS = D / 16;        // k-steps of Q.K^T
  static constexpr int NT_S = kTile / 8;   // 8-token score tiles
  static constexpr int NT_O = D / 8;       // 8-column output tiles
  static constexpr int KS_PV = kTile / 16; // k-steps of P.V
};

struct FdParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;   // may be null
  float* o_partial;     // may be null
  float* lse;           // may be null
  const int* seq_lens;  // may be null
  float* records;       // scratch: per-CTA (m, l, o) records
  int* counters;        // scratch: one arrival counter per (b, kv head)
  int* status;          // scratch header
  int B, Hq, Hkv, R, n_seq, n_groups;
  long long q_sb, q_sh, o_sb, o_sh;
  float scale_log2e;
  int rec_floats;       // floats per record: R * D / 4 chunks of 8
  unsigned long long wait_ns;  // bound of a wait on other CTAs' arrival counters
};

// ---------------------------------------------------------------------------------------------
// Folding of partial attention states.  A state is (m, l, o): running maximum of the scaled scores
// (log2 domain), sum of exp2(score - m), and the unnormalised output.  Two states fold as
//   m' = max(m1, m2),  l' = l1*2^(m1-m') + l2*2^(m2-m'),  o' likewise.
// ---------------------------------------------------------------------------------------------
struct Chunk4 {
  float m, l, o[4];
  __device__ __forceinline__ void clear() { m = -INFINITY; l = 0.f; o[0] = o[1] = o[2] = o[3] = 0.f; }
  __device__ __forceinline__ void fold(float m2, float l2, float x, float y, float z, float w) {
    const float mn = fmaxf(m, m2);
    const float mu = mn == -INFINITY ? 0.f : mn;
    const float a = fast_exp2(m - mu), b = fast_exp2(m2 - mu);
    m = mn;
    l = fmaf(l, a, l2 * b);
    o[0] = fmaf(o[0], a, x * b); o[1] = fmaf(o[1], a, y * b);
    o[2] = fmaf(o[2], a, z * b); o[3] = fmaf(o[3], a, w * b);
  }
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Merge of a unit shared by the n CTAs first_cta .. first_cta + n - 1, as done by participant `me`
// (0-based) for head-warp `warp`.  The unit's R x D outputs are cut into 4-column chunks and the
// chunks are dealt evenly to the n participants.  A participant spreads its lanes over its chunks,
// lpc lanes per chunk (a power of two, as many as 32 lanes allow); the lanes of a chunk take every
// lpc-th record, fold them in registers (up to 8 records' loads in flight per lane) and meet in a
// shuffle butterfly.  So a unit shared by many CTAs costs each of them a handful of loads, and a
// unit shared by two or three costs one round of loads.  Neighbouring lanes hold neighbouring chunks
// of the same record (the lanes of one chunk are 32 / lpc apart), so a load instruction of the warp
// reads runs of consecutive 32-byte chunks instead of 32 scattered ones.
template <int D>
struct SliceJob {
  static constexpr int C4 = D / 4;  // chunks per output row (a power of two)
  static constexpr int kBatch = 8;  // (chunk, record) loads a lane has in flight
  int b, head, n, R;
  int q0, q1, lg, lpc, per_pass, sub, slot;
  const float* rec0;   // record of the first participant (position 1 of its CTA)
  const float* rec1;   // record of the second participant (position 0); later ones follow at rec_stride
  long long rec_stride;
  struct Loads { float m[kBatch], l[kBatch]; float4 v[kBatch]; bool act[kBatch]; };

  __device__ __forceinline__ void setup(const FdParams& p, int b_, int head_, int first_cta, int n_, int me, int HG,
                                        int warp, int lane) {
    b = b_; head = head_; n = n_; R = p.R;
    const int Q = R * C4;
    q0 = (int)((unsigned)me * (unsigned)Q / (unsigned)n);  // me < n <= CTAs of a launch, Q <= 512: fits 32 bits
    q1 = (int)((unsigned)(me + 1) * (unsigned)Q / (unsigned)n);
    lg = 5;
    while (lg > 0 && ((q1 - q0) << lg) > kWarp) --lg;
    lpc = 1 << lg;
    per_pass = kWarp >> lg;
    slot = lane & (per_pass - 1);  // which of the pass's chunks
    sub = lane >> (5 - lg);        // which of the chunk's lpc lanes
    rec0 = p.records + (long long)fd_record_index(first_cta, first_cta, HG, warp) * p.rec_floats;
    rec1 = p.records + (long long)fd_record_index(first_cta + 1, first_cta, HG, warp) * p.rec_floats;
    rec_stride = 2LL * HG * p.rec_floats;
  }
  // True when one round of loads covers the whole job.
  __device__ __forceinline__ bool single_round() const { return q1 - q0 <= per_pass && n <= kBatch * lpc; }

  __device__ __forceinline__ void load(Loads& ld, int base, int k0, int lane) const {
    const int q = q0 + base + slot;
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int rec = k0 + sub + j * lpc;
      ld.act[j] = q < q1 && rec < n;
      if (ld.act[j]) {
        const float* ch = (rec == 0 ? rec0 : rec1 + (rec - 1) * rec_stride) + q * 8;
        ld.v[j] = __ldcg(reinterpret_cast<const float4*>(ch));
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(ch + 4));
        ld.m[j] = ml.x;
        ld.l[j] = ml.y;
      }
    }
  }
  __device__ __forceinline__ void fold(Chunk4& acc, const Loads& ld) const {
#pragma unroll
    for (int j = 0; j < kBatch; ++j)
      if (ld.act[j]) acc.fold(ld.m[j], ld.l[j], ld.v[j].x, ld.v[j].y, ld.v[j].z, ld.v[j].w);
  }
  // Butterfly over the lanes of a chunk, then the chunk's four outputs are normalised and written.
  __device__ __forceinline__ void finish(Chunk4& acc, const FdParams& p, int base, int lane) const {
    for (int off = kWarp >> 1; off >= per_pass; off >>= 1) {
      const float m2 = __shfl_xor_sync(kFullMask, acc.m, off), l2 = __shfl_xor_sync(kFullMask, acc.l, off);
      const float x = __shfl_xor_sync(kFullMask, acc.o[0], off), y = __shfl_xor_sync(kFullMask, acc.o[1], off);
      const float z = __shfl_xor_sync(kFullMask, acc.o[2], off), w = __shfl_xor_sync(kFullMask, acc.o[3], off);
      acc.fold(m2, l2, x, y, z, w);
    }
    const int q = q0 + base + slot;
    if (q < q1 && sub == 0) {
      const int r = q / C4, d = (q & (C4 - 1)) * 4;
      const long long hq = (long long)head * R + r;
      const float inv = acc.l > 0.f ? 1.f / acc.l : 0.f;
      if (p.out) {
        __nv_bfloat16* ob = p.out + (long long)b * p.o_sb + hq * p.o_sh + d;
        *reinterpret_cast<uint32_t*>(ob) = pack_bf16x2(acc.o[0] * inv, acc.o[1] * inv);
        *reinterpret_cast<uint32_t*>(ob + 2) = pack_bf16x2(acc.o[2] * inv, acc.o[3] * inv);
      }
      if (p.o_partial) {
        float* ob = p.o_partial + ((long long)b * p.Hq + hq) * D + d;
        *reinterpret_cast<float4*>(ob) = make_float4(acc.o[0] * inv, acc.o[1] * inv, acc.o[2] * inv, acc.o[3] * inv);
        if (d == 0)
          p.lse[(long long)b * p.Hq + hq] = acc.l > 0.f ? (acc.m + log2f(acc.l)) * 0.6931471805599453f : -INFINITY;
      }
    }
  }
  // The general form: as many passes over chunks and rounds over records as the job needs.
  __device__ __forceinline__ void run(const FdParams& p, int lane) const {
    for (int base = 0; base < q1 - q0; base += per_pass) {
      Chunk4 acc;
      acc.clear();
      for (int k0 = 0; k0 < n; k0 += kBatch * lpc) {
        Loads ld;
        load(ld, base, k0, lane);
        fold(acc, ld);
      }
      finish(acc, p, base, lane);
    }
  }
};

// Waits (bounded) until the participants of this warp's (at most two) shared units have all announced their
// records: counter c[w] must reach n[w] for every w with on[w].  Both counters are polled in the same round
// trip.  Every lane reads with acquire semantics (one request per warp), so the record loads that follow need
// no fence.
__device__ __forceinline__ bool wait_for_records(const FdParams& p, const int* const* c, const int* n, const bool* on,
                                                 int lane) {
  auto poll = [&]() {
    const int v0 = on[0] ? ld_acquire_gpu(c[0]) : 0;
    const int v1 = on[1] ? ld_acquire_gpu(c[1]) : 0;
    return (!on[0] || v0 >= n[0]) && (!on[1] || v1 >= n[1]);
  };
  if (__all_sync(kFullMask, poll())) return true;
  const unsigned long long t0 = global_ns();
  for (uint32_t it = 0;; ++it) {
    __nanosleep(32);
    if (__all_sync(kFullMask, poll())) return true;
    if ((it & 15u) == 15u && __any_sync(kFullMask, global_ns() - t0 > p.wait_ns)) {
      if (lane == 0) atomicExch(p.status, (int)L3CI_ERR_DEVICE_WAIT);
      return false;
    }
  }
}

// Merges this warp's slices of its (at most two) shared units and counts the warp out of them: the counter of a
// unit goes from n (all records announced) to 2n (all participants past their wait), and whoever brings it to 2n
// zeroes it for the next launch.  The count-out is issued before the records are loaded, so its round trip
// overlaps theirs.  When both merges fit in one round of loads each, the loads of the second unit are issued
// before the first is folded, so the two merges cost one memory round trip.  If the wait runs out the units are
// left unmerged and the counters as they are.  Kept out of line so that its registers do not weigh on the
// streaming loop.
template <int D>
__device__ __noinline__ void merge_shared_units(const FdParams& p, const int* def_b, const int* def_head,
                                                const int* def_first, const int* def_n, int cta, int HG, int warp,
                                                int lane) {
  SliceJob<D> job[2];
  const bool on[2] = {def_n[0] > 1, def_n[1] > 1};
  int* const counter[2] = {p.counters + def_b[0] * p.Hkv + def_head[0], p.counters + def_b[1] * p.Hkv + def_head[1]};
  if (!wait_for_records(p, counter, def_n, on, lane)) return;
  int left[2] = {0, 0};
  if (lane == 0) {
#pragma unroll
    for (int w = 0; w < 2; ++w)
      if (on[w]) left[w] = atomicAdd(counter[w], 1);
  }
#pragma unroll
  for (int w = 0; w < 2; ++w)
    if (on[w]) job[w].setup(p, def_b[w], def_head[w], def_first[w], def_n[w], cta - def_first[w], HG, warp, lane);
  if (on[0] && on[1] && job[0].single_round() && job[1].single_round()) {
    typename SliceJob<D>::Loads l0, l1;
    job[0].load(l0, 0, 0, lane);
    job[1].load(l1, 0, 0, lane);
    Chunk4 a0, a1;
    a0.clear();
    a1.clear();
    job[0].fold(a0, l0);
    job[0].finish(a0, p, 0, lane);
    job[1].fold(a1, l1);
    job[1].finish(a1, p, 0, lane);
  } else {
    if (on[0]) job[0].run(p, lane);
    if (on[1]) job[1].run(p, lane);
  }
  if (lane == 0) {
#pragma unroll
    for (int w = 0; w < 2; ++w)
      if (on[w] && left[w] == 2 * def_n[w] - 1) *counter[w] = 0;
  }
}

// ---------------------------------------------------------------------------------------------
// The kernel.  blockDim.x = 32 * (HG + 1): HG consumer warps, one per KV head of the group, and one producer
// warp.  Dynamic shared memory (1024-byte aligned by hand):
//   [kStages] stages | full[kStages], empty[kStages] mbarriers | prefix[B+1] | len[B]
// A stage holds one column: K then V, each as kHalves boxes of [HG heads][kTile tokens][128 bytes], so the
// tile of head w starts w * kBoxBytes into a box and all heads of a token arrive by the same bulk copy (the
// issue of a bulk tensor copy keeps a warp busy for some hundred cycles; four copies per column and CTA, issued
// by a warp that does nothing else, keep that off the warps that do the arithmetic).  full[s] completes when
// the stage's bytes have landed, empty[s] when all HG consumers have released it.
// ---------------------------------------------------------------------------------------------
template <int D, bool RHI>
__global__ void __launch_bounds__(288, 1)
flash_decode_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                    const FdParams p) {
  using C = FdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int HG = (blockDim.x >> 5) - 1;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int gid = lane >> 2;  // MMA row within the 8-row half
  const int tig = lane & 3;   // MMA column pair

  const uint32_t cta_stage_bytes = (uint32_t)HG * kStageBytes;
  uint8_t* stages = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * cta_stage_bytes);  // full[kStages], empty[kStages]
  int* s_pref = reinterpret_cast<int*>(bars + 2 * kStages);
  int* s_len = s_pref + (p.B + 1);

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bars[s]), 1);
      mbar_init(smem_u32(&bars[kStages + s]), HG);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&kmap)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&vmap)) : "memory");
  }
  __syncthreads();

  // ---- column prefix over sequences (only when lengths differ) ----
  FdWalker wk;
  wk.B = p.B; wk.n_groups = p.n_groups; wk.n_seq = p.n_seq; wk.tile = C::kTile;
  wk.pref = nullptr; wk.lens = nullptr;
  int total;
  if (p.seq_lens && p.B <= 8 * kWarp) {
    // Up to 256 sequences: every warp scans the lengths by itself (all warps write the same values to the
    // shared arrays), which saves the two CTA-wide barriers of the general path.
    const int chunk = (p.B + kWarp - 1) / kWarp;  // <= 8 consecutive sequences per lane
    const int beg = min(lane * chunk, p.B), end = min(beg + chunk, p.B);
    int sum = 0;
    for (int b = beg; b < end; ++b) {
      const int len = min(max(__ldg(p.seq_lens + b), 0), p.n_seq);
      s_len[b] = len;
      sum += p.n_groups * fd_tiles(len, C::kTile);
    }
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int n = __shfl_up_sync(kFullMask, incl, d);
      if (lane >= d) incl += n;
    }
    // Every value is written whole (never read-modify-written), so warps writing the same entry agree.
    int run = incl - sum;
    for (int b = beg; b < end; ++b) {
      run += p.n_groups * fd_tiles(min(max(__ldg(p.seq_lens + b), 0), p.n_seq), C::kTile);
      s_pref[b + 1] = run;
    }
    if (lane == 0) s_pref[0] = 0;
    __syncwarp();
    wk.pref = s_pref;
    wk.lens = s_len;
    total = __shfl_sync(kFullMask, incl, kWarp - 1);
  } else if (p.seq_lens) {
    for (int b = threadIdx.x; b < p.B; b += blockDim.x) {
      const int len = min(max(__ldg(p.seq_lens + b), 0), p.n_seq);
      s_len[b] = len;
      s_pref[b + 1] = p.n_groups * fd_tiles(len, C::kTile);
    }
    __syncthreads();
    if (warp == 0) {
      const int chunk = (p.B + 31) >> 5;
      const int beg = min(lane * chunk, p.B), end = min(beg + chunk, p.B);
      int sum = 0;
      for (int b = beg; b < end; ++b) sum += s_pref[b + 1];
      int incl = sum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(kFullMask, incl, d);
        if (lane >= d) incl += n;
      }
      int run = incl - sum;
      for (int b = beg; b < end; ++b) {
        run += s_pref[b + 1];
        s_pref[b + 1] = run;
      }
      if (lane == 0) s_pref[0] = 0;
    }
    __syncthreads();
    wk.pref = s_pref;
    wk.lens = s_len;
    total = s_pref[p.B];
  } else {
    total = p.B * p.n_groups * fd_tiles(p.n_seq, C::kTile);
  }

  // The host sizes the grid from the padded length; with shorter sequences there may be fewer
  // columns than CTAs.  Only the first G CTAs work, so that every working CTA owns >= 1 column.
  // Short sequences: whole units per CTA, no cross-CTA merge.  Otherwise: equal contiguous ranges.
  const int units = p.B * p.n_groups;
  const bool whole = fd_whole_units(total, units, (int)gridDim.x);
  const int G = whole ? min((int)gridDim.x, units) : fd_active_ctas((int)gridDim.x, total);
  const int cta = blockIdx.x;
  if (cta >= G) return;
  int c0, c1;
  if (whole) {
    auto unit_col = [&](int u) {
      const int b = u / p.n_groups, g = u - b * p.n_groups;
      return b >= p.B ? total : wk.pref_of(b) + g * fd_tiles(wk.len_of(b), C::kTile);
    };
    c0 = unit_col(fd_range_begin(cta, units, G));
    c1 = unit_col(fd_range_begin(cta + 1, units, G));
  } else {
    c0 = fd_range_begin(cta, total, G);
    c1 = fd_range_begin(cta + 1, total, G);
  }

  const uint32_t stage0 = smem_u32(stages);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = full0 + kStages * 8;
  const uint32_t half_stride = (uint32_t)HG * C::kBoxBytes;  // between the 64-column halves of a K or V tile

  if (warp == HG) {
    // ---- producer warp: one column per step into the next free stage ----
    const uint64_t policy = l2_evict_first_policy();
    FdCursor prod = wk.seek(c0);
    int k = 0;
    bool alive = true;
    for (; prod.col < c1; wk.advance(prod), ++k) {
      const int stage = k % kStages;
      if (k >= kStages && !mbar_wait_bounded(empty0 + stage * 8, ((k / kStages) - 1) & 1)) { alive = false; break; }
      if (lane == 0) {
        const uint32_t bar = full0 + stage * 8;
        const uint32_t dst = stage0 + stage * cta_stage_bytes;
        const int tok = prod.j * C::kTile;
        const int head = prod.g * HG;
        mbar_expect_tx(bar, cta_stage_bytes);
#pragma unroll
        for (int h = 0; h < C::kHalves; ++h) tma_load_4d(dst + h * half_stride, &kmap, bar, h * 64, tok, head, prod.b, policy);
#pragma unroll
        for (int h = 0; h < C::kHalves; ++h)
          tma_load_4d(dst + HG * C::kKBytes + h * half_stride, &vmap, bar, h * 64, tok, head, prod.b, policy);
      }
      __syncwarp();
    }
    // Stay until the consumers have released the last columns: the shared memory of a CTA must not go away
    // under a copy in flight.  A consumer that gave up never releases; then these waits run out too.
    for (int j = max(k - kStages, 0); alive && j < k; ++j)
      alive = mbar_wait_bounded(empty0 + (j % kStages) * 8, (j / kStages) & 1);
    if (!alive && lane == 0) atomicExch(p.status, (int)L3CI_ERR_DEVICE_WAIT);
    return;
  }

  FdCursor cons = wk.seek(c0);

  // ---- lane constants of the ldmatrix addresses ----
  // Scores are computed transposed, S^T = K Q^T, and so is the output, O^T = V^T P^T: the 16 rows of a
  // tensor-core tile are tokens (or output columns) and its 8 columns are the query heads that share this KV
  // head.  With up to 8 query heads per KV head no row of a tile is padding, which halves the tensor-core
  // instructions and the accumulator registers against tiles whose 16 rows are query heads.
  const int mat = lane >> 3, r8 = lane & 7;
  // K as A operand: matrices (tok 0-7, chunk c), (tok 8-15, c), (tok 0-7, c+1), (tok 8-15, c+1)
  const uint32_t k_row_off = (r8 + 8 * (mat & 1)) * 128;
  const uint32_t k_x = (mat >> 1) ^ r8;
  // V, transposed, as A operand: matrices (tok 0-7, chunk c), (tok 0-7, c+1), (tok 8-15, c), (tok 8-15, c+1)
  const uint32_t v_row_off = (r8 + 8 * (mat >> 1)) * 128;
  const uint32_t v_x = (mat & 1) ^ r8;

  // ---- per-segment state ----
  constexpr int NB = RHI ? 2 : 1;    // blocks of 8 query rows
  constexpr int MB = C::kTile / 16;  // blocks of 16 tokens in a tile
  constexpr int MT = D / 16;         // blocks of 16 output columns
  // This thread's query rows are nb * 8 + 2 * tig + j (j = 0, 1); its tokens / output columns are gid and gid + 8
  // of a block of 16.
  uint32_t qb[C::KS][NB][2];
  float o[NB][MT][4];
  float m_run[NB][2], l_run[NB][2];
  bool seg_start = true;
  int k_iter = 0;
  const int R = p.R;
  bool ok = true;
  int def_b[2] = {0, 0}, def_head[2] = {0, 0}, def_first[2] = {0, 0}, def_n[2] = {0, 0};  // shared units to merge at the end

  // S^T = K Q^T for the kTile tokens of the tile at kb.  The k-steps are dealt to kChains accumulator sets that
  // are added at the end, so that no tensor-core instruction waits on more than one predecessor.
  auto qk_scores = [&](uint32_t kb, float (&sc)[NB][MB][4]) {
    constexpr int kChains = C::KS / 2;
    float part[kChains][NB][MB][4];
#pragma unroll
    for (int c = 0; c < kChains; ++c)
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) part[c][nb][mb][0] = part[c][nb][mb][1] = part[c][nb][mb][2] = part[c][nb][mb][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < C::KS; ++ks) {
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        uint32_t a0, a1, a2, a3;
        const uint32_t addr = kb + (ks >> 2) * half_stride + mb * 2048 + k_row_off + (((2u * (ks & 3)) ^ k_x) << 4);
        ldsm_x4(addr, a0, a1, a2, a3);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) mma_bf16(part[ks % kChains][nb][mb], a0, a1, a2, a3, qb[ks][nb][0], qb[ks][nb][1]);
      }
    }
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float a = part[0][nb][mb][e];
#pragma unroll
          for (int c = 1; c < kChains; ++c) a += part[c][nb][mb][e];
          sc[nb][mb][e] = a;
        }
  };
  // Reductions over the 8 lanes that hold the same query rows (same tig).
  auto rows_max = [&](float v) {
    v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 4));
    v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 8));
    return fmaxf(v, __shfl_xor_sync(kFullMask, v, 16));
  };
  auto rows_sum = [&](float v) {
    v += __shfl_xor_sync(kFullMask, v, 4);
    v += __shfl_xor_sync(kFullMask, v, 8);
    return v + __shfl_xor_sync(kFullMask, v, 16);
  };
  // Hands every pair of adjacent output columns of every query row of this thread to emit(nb, j, row, d, v0, v1)
  // (d even, v0/v1 the unnormalised outputs of columns d, d + 1).  A thread holds columns gid and gid + 8 of a
  // block; neighbours in gid swap one value each so that both end up with an aligned pair.
  auto for_each_pair = [&](auto&& emit) {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int row = nb * 8 + 2 * tig + j;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const float x = o[nb][mt][j], y = o[nb][mt][2 + j];
          const bool odd = gid & 1;
          const float got = __shfl_xor_sync(kFullMask, odd ? x : y, 4);
          if (row < R) emit(nb, j, row, 16 * mt + (odd ? gid + 7 : gid), odd ? got : x, odd ? y : got);
        }
      }
  };
  float s[NB][MB][4];
  bool have_s = false;
  while (cons.col < c1) {
    const int head = cons.g * HG + warp;
    if (seg_start) {
      const __nv_bfloat16* qp = p.q + (long long)cons.b * p.q_sb + (long long)(head * R) * p.q_sh;
#pragma unroll
      for (int ks = 0; ks < C::KS; ++ks) {
        const int col = ks * 16 + 2 * tig;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          const int row = nb * 8 + gid;
          qb[ks][nb][0] = row < R ? ld_global_u32(qp + row * p.q_sh + col) : 0u;
          qb[ks][nb][1] = row < R ? ld_global_u32(qp + row * p.q_sh + col + 8) : 0u;
        }
      }
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) o[nb][mt][0] = o[nb][mt][1] = o[nb][mt][2] = o[nb][mt][3] = 0.f;
        m_run[nb][0] = m_run[nb][1] = -INFINITY;
        l_run[nb][0] = l_run[nb][1] = 0.f;
      }
      seg_start = false;
    }

    const int stage = k_iter % kStages;
    const uint32_t kb = stage0 + stage * cta_stage_bytes + warp * C::kBoxBytes;
    const uint32_t vb = kb + HG * C::kKBytes;
    if (!have_s) {
      if (!mbar_wait_bounded(full0 + stage * 8, (k_iter / kStages) & 1)) { ok = false; break; }
      qk_scores(kb, s);
    }
    // Scores of the next tile, when it continues this unit: its K is normally in shared memory already, and its
    // chain of tensor-core instructions has nothing to do with the softmax and the P.V of the current tile, so
    // the two overlap in the instruction stream.
    const bool more = !fd_unit_ends(cons, c1);
    const bool ahead = kScoresAhead && more;
    float s_next[NB][MB][4];
    if (ahead) {
      const int st2 = (k_iter + 1) % kStages;
      if (!mbar_wait_bounded(full0 + st2 * 8, ((k_iter + 1) / kStages) & 1)) { ok = false; break; }
      qk_scores(stage0 + st2 * cta_stage_bytes + warp * C::kBoxBytes, s_next);
    }

    // ---- mask the tail of the sequence, online softmax (log2 domain) ----
    const int tok0 = cons.j * C::kTile;
    if (tok0 + C::kTile > cons.len) {
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          const int t = tok0 + mb * 16 + gid;
          if (t >= cons.len) s[nb][mb][0] = s[nb][mb][1] = -INFINITY;
          if (t + 8 >= cons.len) s[nb][mb][2] = s[nb][mb][3] = -INFINITY;
        }
    }
    uint32_t pb[NB][MB][2];  // P^T as B operand, one 16-token k-step per mb
    float alpha[NB][2];
    bool moved = false;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      float mu[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float mx = -INFINITY;
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) mx = fmaxf(mx, fmaxf(s[nb][mb][j], s[nb][mb][2 + j]));
        mx = rows_max(mx) * p.scale_log2e;
        const float mn = fmaxf(m_run[nb][j], mx);
        mu[j] = mn == -INFINITY ? 0.f : mn;
        alpha[nb][j] = fast_exp2(m_run[nb][j] - mu[j]);
        m_run[nb][j] = mn;
        moved |= alpha[nb][j] != 1.f;
      }
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        const float p0 = fast_exp2(fmaf(s[nb][mb][0], p.scale_log2e, -mu[0]));
        const float p1 = fast_exp2(fmaf(s[nb][mb][1], p.scale_log2e, -mu[1]));
        const float p2 = fast_exp2(fmaf(s[nb][mb][2], p.scale_log2e, -mu[0]));
        const float p3 = fast_exp2(fmaf(s[nb][mb][3], p.scale_log2e, -mu[1]));
        ps0 += p0 + p2;
        ps1 += p1 + p3;
        // (token gid | gid + 8, rows 2 tig, 2 tig + 1)  ->  (row gid, tokens 2 tig, 2 tig + 1 | + 8)
        pb[nb][mb][0] = movmatrix_trans(pack_bf16x2(p0, p1));
        pb[nb][mb][1] = movmatrix_trans(pack_bf16x2(p2, p3));
      }
      l_run[nb][0] = fmaf(l_run[nb][0], alpha[nb][0], ps0);
      l_run[nb][1] = fmaf(l_run[nb][1], alpha[nb][1], ps1);
    }
    // Rescale the accumulator only when some row's maximum moved (warp-uniform test).
    if (__any_sync(kFullMask, moved)) {
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          o[nb][mt][0] *= alpha[nb][0];
          o[nb][mt][1] *= alpha[nb][1];
          o[nb][mt][2] *= alpha[nb][0];
          o[nb][mt][3] *= alpha[nb][1];
        }
    }

    // ---- O^T += V^T P^T ----
#pragma unroll
    for (int kk = 0; kk < MB; ++kk) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t a0, a1, a2, a3;
        const uint32_t addr = vb + (mt >> 2) * half_stride + kk * 2048 + v_row_off + (((2u * (mt & 3)) ^ v_x) << 4);
        ldsm_x4_trans(addr, a0, a1, a2, a3);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) mma_bf16(o[nb][mt], a0, a1, a2, a3, pb[nb][kk][0], pb[nb][kk][1]);
      }
    }

    // ---- release the stage to the producer ----
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + stage * 8);
    ++k_iter;
    have_s = ahead;
    if (ahead) {
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[nb][mb][e] = s_next[nb][mb][e];
    }

    // ---- end of this (sequence, head) unit inside the CTA's range? ----
    if (!more) {
      seg_start = true;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        l_run[nb][0] = rows_sum(l_run[nb][0]);
        l_run[nb][1] = rows_sum(l_run[nb][1]);
      }
      const int u0 = wk.unit_begin(cons);
      const int cfirst = whole ? cta : fd_cta_of(u0, total, G);
      const int clast = whole ? cta : fd_cta_of(u0 + cons.tc - 1, total, G);
      const long long hq0 = (long long)head * R;

      if (cfirst == clast) {
        // The whole unit was seen by this warp: normalise and write.
        float inv[NB][2];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
          for (int j = 0; j < 2; ++j) inv[nb][j] = l_run[nb][j] > 0.f ? 1.f / l_run[nb][j] : 0.f;
        if (p.out) {
          __nv_bfloat16* ob = p.out + (long long)cons.b * p.o_sb + hq0 * p.o_sh;
          for_each_pair([&](int nb, int j, int row, int d, float v0, float v1) {
            *reinterpret_cast<uint32_t*>(ob + row * p.o_sh + d) = pack_bf16x2(v0 * inv[nb][j], v1 * inv[nb][j]);
          });
        }
        if (p.o_partial) {
          float* ob = p.o_partial + ((long long)cons.b * p.Hq + hq0) * D;
          float* lb = p.lse + (long long)cons.b * p.Hq + hq0;
          for_each_pair([&](int nb, int j, int row, int d, float v0, float v1) {
            *reinterpret_cast<float2*>(ob + row * D + d) = make_float2(v0 * inv[nb][j], v1 * inv[nb][j]);
          });
          if (gid == 0) {
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                const int row = nb * 8 + 2 * tig + j;
                if (row < R)
                  lb[row] = l_run[nb][j] > 0.f ? (m_run[nb][j] + log2f(l_run[nb][j])) * 0.6931471805599453f : -INFINITY;
              }
          }
        }
      } else {
        // Shared with other CTAs: leave an unnormalised record and a count on the unit's arrival counter.
        float* rec = p.records + (long long)fd_record_index(cta, cfirst, HG, warp) * p.rec_floats;
        for_each_pair([&](int nb, int j, int row, int d, float v0, float v1) {
          float* ch = rec + (row * (D / 4) + (d >> 2)) * 8;  // the chunk of columns d & ~3 .. d | 3
          __stcg(reinterpret_cast<float2*>(ch + (d & 3)), make_float2(v0, v1));
          if ((d & 3) == 0) __stcg(reinterpret_cast<float2*>(ch + 4), make_float2(m_run[nb][j], l_run[nb][j]));
        });
        // The record is announced (and the unit merged) after the whole range has been streamed.  A warp
        // has at most two such units: one that began in an earlier CTA, one that continues in the next.
        const int which = cta == cfirst ? 1 : 0;
        def_b[which] = cons.b;
        def_head[which] = head;
        def_first[which] = cfirst;
        def_n[which] = clast - cfirst + 1;
      }
    }
    wk.advance(cons);
  }

  if (!ok) {
    // A column never arrived.  Record it and leave; shared units stay unmerged.  The producer warp notices
    // the missing release, gives the copies in flight a bounded time to land and ends the CTA.
    if (lane == 0) atomicExch(p.status, (int)L3CI_ERR_DEVICE_WAIT);
    return;
  }
  // ---- shared units ----
  // Announce this warp's records (one fence for both), then merge this CTA's slice of each unit once every
  // participant has announced.
  if (def_n[0] > 1 || def_n[1] > 1) {
    __threadfence();
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (int w = 0; w < 2; ++w)
        if (def_n[w] > 1) atomicAdd(p.counters + def_b[w] * p.Hkv + def_head[w], 1);
    }
    merge_shared_units<D>(p, def_b, def_head, def_first, def_n, cta, HG, warp, lane);
  }
}

// Writes zeros for a call without any cached token.
__global__ void zero_out_kernel(__nv_bfloat16* out, float* o_partial, float* lse, int B, int Hq, int D,
                                long long o_sb, long long o_sh) {
  const long long n = (long long)B * Hq * D;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int d = (int)(i % D);
    const long long bh = i / D;
    const int h = (int)(bh % Hq);
    const long long b = bh / Hq;
    if (out) out[b * o_sb + h * o_sh + d] = __float2bfloat16(0.f);
    if (o_partial) o_partial[i] = 0.f;
    if (lse && d == 0) lse[bh] = -INFINITY;
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
// Floats of one (m, l, o) record: R * D / 4 chunks of {o[4], m, l, -, -}.  A chunk is the unit a lane of the
// merge reads, and it is one 32-byte sector: the row's maximum and sum travel with every four outputs, so a
// merge of n records reads n sectors per chunk instead of 3 n (the sums and maxima of a row are wanted by all
// the lanes, in several CTAs, that hold chunks of that row).
int record_floats(int R, int D) { return R * D * 2; }

// Scratch layout: header | arrival counters | records.  The counter area has the same place and size
// for every call with up to kFixedCounters (sequence, kv head) units, so a scratch buffer that was zeroed
// once can serve calls of any shape: counters are left at zero by the kernel, records are written before
// they are read.  Larger batches get a counter area of their own size (then a change of shape needs the
// buffer zeroed again).
constexpr size_t kFixedCounters = 65536;
size_t counters_bytes(int B, int Hkv) {
  const size_t units = (size_t)B * Hkv;
  return ((units > kFixedCounters ? units : kFixedCounters) * sizeof(int) + 255) & ~(size_t)255;
}

size_t smem_bytes(int HG, int B, bool ragged) {
  size_t s = 1024 + (size_t)HG * kStages * kStageBytes + 2 * kStages * 8;
  if (ragged) s += (size_t)(2 * B + 1) * sizeof(int);
  return s;
}

// Launches the kernel cooperatively: the runtime refuses a grid that cannot be resident all at once,
// which the kernel relies on when a warp waits for the records of other CTAs.  The grid is clamped to
// what fits (blocks per SM from the occupancy calculator, cached per device and launch shape).
template <int D, bool RHI>
int launch_fd(const CUtensorMap& kmap, const CUtensorMap& vmap, const FdParams& p, int grid, int HG,
              size_t smem, cudaStream_t stream) {
  struct Cached { size_t configured = 0; int block = 0; size_t smem = 0; int per_sm = 0; };
  static Cached cache[64];
  static std::mutex mu;
  int dev = 0;
  L3CI_CUDA_TRY(cudaGetDevice(&dev));
  const int block = (HG + 1) * 32;  // HG consumer warps and the producer warp
  int per_sm = 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    Cached local;
    Cached& c = dev < 64 ? cache[dev] : local;
    if (c.configured < smem) {
      L3CI_CUDA_TRY(cudaFuncSetAttribute(flash_decode_kernel<D, RHI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
      c.configured = smem;
    }
    if (c.block != block || c.smem != smem) {
      L3CI_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&c.per_sm, flash_decode_kernel<D, RHI>, block, smem));
      c.block = block;
      c.smem = smem;
    }
    per_sm = c.per_sm;
  }
  if (per_sm <= 0) return fail(L3CI_ERR_UNSUPPORTED, "flash_decode: kernel does not fit on an SM with %zu bytes of shared memory", smem);
  const int resident = per_sm * sm_count();
  if (grid > resident) grid = resident;
  void* args[] = {const_cast<CUtensorMap*>(&kmap), const_cast<CUtensorMap*>(&vmap), const_cast<FdParams*>(&p)};
  L3CI_CUDA_TRY(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(&flash_decode_kernel<D, RHI>), dim3(grid),
                                            dim3(block), args, smem, stream));
  return L3CI_OK;
}

}  // namespace
}  // namespace l3ci

extern "C" size_t l3ci_flash_decode_scratch_bytes(int32_t B, int32_t Hq, int32_t Hkv, int32_t D) {
  using namespace l3ci;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || Hq % Hkv) return 0;
  const int R = Hq / Hkv;
  const int sms = sm_count();
  if (sms <= 0) return 0;
  // Records: 2 per CTA per warp; CTAs * warps is 8 per SM whatever the head grouping is.
  const size_t records = (size_t)fd_max_ctas(sms, fd_head_group(Hkv)) * fd_head_group(Hkv) * 2;
  return kHeaderBytes + counters_bytes(B, Hkv) + records * (size_t)record_floats(R, D) * sizeof(float);
}

namespace l3ci {
namespace {
// Whether a call with valid sizes goes to the static-deal kernel, which uses no scratch (the one rule for
// l3ci_flash_decode and l3ci_flash_decode_static).
bool takes_static_deal(const l3ci_flash_decode_args* a) {
  if (a->B <= 0 || a->Hkv <= 0 || a->Hq <= 0 || a->Hq % a->Hkv || a->n_seq <= 0 || (a->D != 64 && a->D != 128)) return false;
  const int R = a->Hq / a->Hkv;
  if (a->max_ctas < 0) return R <= 8;
  return a->max_ctas == 0 && flash_decode_small_applies(a->B, a->Hq, a->Hkv, a->D, a->n_seq, a->seq_lens != nullptr);
}

// Validates the arguments and launches; `a->scratch` must already be what the call may use.
int flash_decode_launch(const l3ci_flash_decode_args* a) {
  clear_error();
  if (!a) return fail(L3CI_ERR_INVALID, "flash_decode: null args");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(a->stream);
  const int B = a->B, Hq = a->Hq, Hkv = a->Hkv, D = a->D, n_seq = a->n_seq;
  if (B < 0 || Hq <= 0 || Hkv <= 0 || n_seq < 0) return fail(L3CI_ERR_INVALID, "flash_decode: bad size B=%d Hq=%d Hkv=%d n_seq=%d", B, Hq, Hkv, n_seq);
  if (Hq % Hkv) return fail(L3CI_ERR_INVALID, "flash_decode: %d query heads not divisible by %d kv heads", Hq, Hkv);
  if (D != 64 && D != 128) return fail(L3CI_ERR_UNSUPPORTED, "Unsupported head size for flash_decode kernel: %d", D);
  const int R = Hq / Hkv;
  if (R > 16) return fail(L3CI_ERR_UNSUPPORTED, "Unsupported QKV head ratio for flash_decode kernel: %d", R);
  if (B == 0) return L3CI_OK;
  if (!a->q || (!a->out && !a->o_partial)) return fail(L3CI_ERR_INVALID, "flash_decode: null q or no output");
  if ((a->o_partial == nullptr) != (a->lse == nullptr)) return fail(L3CI_ERR_INVALID, "flash_decode: o_partial and lse go together");
  if ((reinterpret_cast<uintptr_t>(a->q) & 3) || (a->q_sb & 1) || (a->q_sh & 1) ||
      (a->out && ((reinterpret_cast<uintptr_t>(a->out) & 3) || (a->o_sb & 1) || (a->o_sh & 1))) ||
      (a->o_partial && !aligned16(a->o_partial)))
    return fail(L3CI_ERR_ALIGNMENT, "flash_decode: q/out rows must start on 4 bytes");

  if (n_seq == 0) {
    zero_out_kernel<<<64, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(a->out), a->o_partial, a->lse, B, Hq, D,
                                            a->o_sb, a->o_sh);
    L3CI_CHECK_LAUNCH("zero_out_kernel");
    return L3CI_OK;
  }
  if (!a->k || !a->v) return fail(L3CI_ERR_INVALID, "flash_decode: null k or v");
  if (!aligned16(a->k) || !aligned16(a->v) || (n_seq > 1 && (a->k_st % 8 || a->v_st % 8)) ||
      (Hkv > 1 && (a->k_sh % 8 || a->v_sh % 8)) || (B > 1 && (a->k_sb % 8 || a->v_sb % 8)))
    return fail(L3CI_ERR_ALIGNMENT, "flash_decode: k/v rows must start on 16 bytes and strides be multiples of 8 elements");
  if ((n_seq > 1 && (a->k_st <= 0 || a->v_st <= 0)) || (Hkv > 1 && (a->k_sh <= 0 || a->v_sh <= 0)) ||
      (B > 1 && (a->k_sb <= 0 || a->v_sb <= 0)))
    return fail(L3CI_ERR_INVALID, "flash_decode: k/v strides must be positive");

  const int tile = fd_tile_tokens(D);
  const int HG = fd_head_group(Hkv);
  const int n_groups = Hkv / HG;
  const long long max_cols = (long long)B * n_groups * fd_tiles(n_seq, tile);
  if (max_cols > 0x3fffffffLL) return fail(L3CI_ERR_INVALID, "flash_decode: too many tiles (%lld)", max_cols);
  const bool ragged = a->seq_lens != nullptr;
  if (ragged && B > 4096) return fail(L3CI_ERR_UNSUPPORTED, "flash_decode: seq_lens supports at most 4096 sequences, got %d", B);

  const int sms = sm_count();
  if (sms <= 0) return fail(L3CI_ERR_CUDA, "flash_decode: no CUDA device");
  int grid = fd_max_ctas(sms, HG);
  if (a->max_ctas > 0 && a->max_ctas < grid) grid = a->max_ctas;
  if (max_cols < grid) grid = (int)max_cols;

  // Where the static deal of units to warps, CTAs or clusters is expected to be faster (flash_decode_small.cu),
  // nothing goes through global memory and the scratch is neither needed nor touched.  A positive max_ctas asks
  // for the persistent kernel.
  if (takes_static_deal(a)) return flash_decode_small_launch(a, a->max_ctas < -1 ? -a->max_ctas : 0);

  const size_t need = l3ci_flash_decode_scratch_bytes(B, Hq, Hkv, D);
  if (!a->scratch || a->scratch_bytes < need)
    return fail(L3CI_ERR_SCRATCH, "flash_decode: scratch has %zu bytes, needs %zu", a->scratch_bytes, need);
  if (reinterpret_cast<uintptr_t>(a->scratch) & 255) return fail(L3CI_ERR_ALIGNMENT, "flash_decode: scratch must be 256-byte aligned");

  const size_t smem = smem_bytes(HG, B, ragged);
  if ((long long)smem > max_smem_optin()) return fail(L3CI_ERR_UNSUPPORTED, "flash_decode: needs %zu bytes of shared memory", smem);

  CUtensorMap kmap, vmap;
  if (int st = make_kv_map(&kmap, a->k, D, n_seq, Hkv, B, a->k_st, a->k_sh, a->k_sb, tile, HG)) return st;
  if (int st = make_kv_map(&vmap, a->v, D, n_seq, Hkv, B, a->v_st, a->v_sh, a->v_sb, tile, HG)) return st;

  FdParams p;
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.o_partial = a->o_partial;
  p.lse = a->lse;
  p.seq_lens = a->seq_lens;
  uint8_t* sc = static_cast<uint8_t*>(a->scratch);
  p.status = reinterpret_cast<int*>(sc);
  p.counters = reinterpret_cast<int*>(sc + kHeaderBytes);
  p.records = reinterpret_cast<float*>(sc + kHeaderBytes + counters_bytes(B, Hkv));
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.R = R; p.n_seq = n_seq; p.n_groups = n_groups;
  p.q_sb = a->q_sb; p.q_sh = a->q_sh; p.o_sb = a->o_sb; p.o_sh = a->o_sh;
  const float scale = a->scale > 0.f ? a->scale : 1.0f / sqrtf((float)D);
  p.scale_log2e = scale * 1.4426950408889634f;
  p.rec_floats = record_floats(R, D);
  p.wait_ns = device_wait_limit_ns(kWaitLimitNs);

  if (D == 64) {
    return R > 8 ? launch_fd<64, true>(kmap, vmap, p, grid, HG, smem, stream)
                 : launch_fd<64, false>(kmap, vmap, p, grid, HG, smem, stream);
  }
  return R > 8 ? launch_fd<128, true>(kmap, vmap, p, grid, HG, smem, stream)
               : launch_fd<128, false>(kmap, vmap, p, grid, HG, smem, stream);
}
}  // namespace
}  // namespace l3ci

extern "C" int l3ci_flash_decode(const l3ci_flash_decode_args* a) { return l3ci::flash_decode_launch(a); }

// ---------------------------------------------------------------------------------------------
// Sequence-sharded decode with the cross-GPU exchange and merge in the kernel's tail (one launch per step).
// ---------------------------------------------------------------------------------------------
extern "C" size_t l3ci_flash_decode_exchange_bytes(int32_t ranks, int32_t B, int32_t Hq, int32_t D) {
  if (ranks <= 0 || B <= 0 || Hq <= 0 || D <= 0) return 0;
  // [2 parities][ranks][rows * (D + 1)] 64-bit words, then 2 control words
  return (2 * (size_t)ranks * (size_t)B * Hq * (D + 1) + 2) * sizeof(unsigned long long);
}

extern "C" int l3ci_flash_decode_exchange(const l3ci_flash_decode_args* a, void* const* bufs, int32_t rank, int32_t ranks,
                                          uint32_t epoch, int32_t* status) {
  using namespace l3ci;
  clear_error();
  if (!a) return fail(L3CI_ERR_INVALID, "flash_decode_exchange: null args");
  if (a->B <= 0 || a->Hq <= 0 || a->Hkv <= 0 || a->Hq % a->Hkv || a->n_seq < 0 || (a->D != 64 && a->D != 128))
    return fail(L3CI_ERR_INVALID, "flash_decode_exchange: bad size B=%d Hq=%d Hkv=%d D=%d n_seq=%d", a->B, a->Hq, a->Hkv, a->D, a->n_seq);
  if (!a->q || !a->out || a->o_partial || a->lse)
    return fail(L3CI_ERR_INVALID, "flash_decode_exchange: needs q and out, and takes no o_partial / lse");
  if (!bufs || rank < 0 || rank >= ranks) return fail(L3CI_ERR_INVALID, "flash_decode_exchange: bad rank %d of %d or no buffers", rank, ranks);
  if (a->n_seq > 0 && (!a->k || !a->v)) return fail(L3CI_ERR_INVALID, "flash_decode_exchange: null k or v");
  if ((reinterpret_cast<uintptr_t>(a->q) & 3) || (a->q_sb & 1) || (a->q_sh & 1) || (reinterpret_cast<uintptr_t>(a->out) & 3) ||
      (a->o_sb & 1) || (a->o_sh & 1))
    return fail(L3CI_ERR_ALIGNMENT, "flash_decode_exchange: q/out rows must start on 4 bytes");
  if (a->n_seq > 0 && (!aligned16(a->k) || !aligned16(a->v) || (a->n_seq > 1 && (a->k_st % 8 || a->v_st % 8 || a->k_st <= 0 || a->v_st <= 0)) ||
                       (a->Hkv > 1 && (a->k_sh % 8 || a->v_sh % 8)) || (a->B > 1 && (a->k_sb % 8 || a->v_sb % 8))))
    return fail(L3CI_ERR_ALIGNMENT, "flash_decode_exchange: k/v rows must start on 16 bytes and strides be positive multiples of 8 elements");
  // Only the static-deal kernel has the exchange in its tail.  An empty shard (n_seq == 0) still takes part: it
  // sends zeros with a log-sum-exp of -inf.
  if (a->Hq / a->Hkv > 8 || a->max_ctas > 0 || (a->n_seq > 0 && a->max_ctas == 0 && !takes_static_deal(a)))
    return fail(L3CI_ERR_UNSUPPORTED, "flash_decode_exchange: these sizes go to the persistent kernel, which has no fused exchange; "
                                      "use l3ci_flash_decode with o_partial / lse and l3ci_lse_exchange_merge");
  FdExchange x{bufs, rank, ranks, epoch, status};
  return flash_decode_small_launch(a, a->max_ctas < -1 ? -a->max_ctas : 0, &x);
}

extern "C" int l3ci_flash_decode_kernel_choice(int32_t B, int32_t Hq, int32_t Hkv, int32_t D, int32_t n_seq, int32_t ragged) {
  using namespace l3ci;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || (D != 64 && D != 128) || n_seq <= 0) return -1;
  if (!flash_decode_small_applies(B, Hq, Hkv, D, n_seq, ragged != 0)) return 0;
  return flash_decode_small_split_code(B, Hkv, D, n_seq);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant: the scratch lives in this library's own device image.
// ---------------------------------------------------------------------------------------------
// Every GPU that loads the library holds these bytes until the process exits.  In host code the name
// below is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_fd_static_scratch[L3CI_STATIC_SCRATCH_BYTES];

namespace l3ci {
namespace {
// Device address of g_fd_static_scratch on the current device, looked up once per device (with that
// device current) and remembered.  The first look-up on a device may make the runtime load this library's
// device image, array included; inside a stream capture that is refused here with a clear message rather
// than left to fail in the driver.
int static_scratch_address(void** out, cudaStream_t stream) {
  static void* address[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  L3CI_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(L3CI_ERR_UNSUPPORTED, "flash_decode_static: device index %d", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!address[dev]) {
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess) (void)cudaGetLastError();
    if (capturing != cudaStreamCaptureStatusNone)
      return fail(L3CI_ERR_INVALID, "flash_decode_static: the first call on a device looks up the built-in scratch "
                                    "and must be made outside a stream capture");
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_fd_static_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(L3CI_ERR_CUDA, "flash_decode_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    address[dev] = ptr;
  }
  *out = address[dev];
  return L3CI_OK;
}
}  // namespace
}  // namespace l3ci

extern "C" int l3ci_flash_decode_static(const l3ci_flash_decode_args* a) {
  using namespace l3ci;
  clear_error();
  if (!a) return fail(L3CI_ERR_INVALID, "flash_decode_static: null args");
  if (a->B <= 0 || a->Hq <= 0 || a->Hkv <= 0 || a->Hq % a->Hkv) return flash_decode_launch(a);  // reports the bad size
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(a->stream);
  void* area = nullptr;
  if (int st = static_scratch_address(&area, stream)) return st;
  l3ci_flash_decode_args b = *a;
  b.scratch = area;
  b.scratch_bytes = (size_t)L3CI_STATIC_SCRATCH_BYTES;
  // A call that the static-deal kernel takes needs no scratch at all: no size limit applies, nothing is cleared.
  if (takes_static_deal(a)) return flash_decode_launch(&b);
  const size_t need = l3ci_flash_decode_scratch_bytes(a->B, a->Hq, a->Hkv, a->D);
  if (need == 0 || need > (size_t)L3CI_STATIC_SCRATCH_BYTES || (size_t)a->B * a->Hkv > kFixedCounters)
    return fail(L3CI_ERR_SCRATCH,
                "flash_decode_static: this shape needs %zu bytes of scratch (B*Hkv = %lld units), the built-in area holds "
                "%zu bytes and %zu units; use l3ci_flash_decode with caller-provided scratch",
                need, (long long)a->B * a->Hkv, (size_t)L3CI_STATIC_SCRATCH_BYTES, kFixedCounters);
  // The area keeps whatever the previous call (of any shape) left.  Records are written before they are read;
  // the status word and the arrival counters of this call's units must start at zero.
  const size_t clear = kHeaderBytes + (((size_t)a->B * a->Hkv * sizeof(int) + 255) & ~(size_t)255);
  L3CI_CUDA_TRY(cudaMemsetAsync(area, 0, clear, stream));
  return flash_decode_launch(&b);
}

extern "C" int l3ci_flash_decode_poll(void* scratch, size_t scratch_bytes, l3ci_stream_t stream_) {
  using namespace l3ci;
  clear_error();
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!scratch || scratch_bytes < (size_t)kHeaderBytes) return fail(L3CI_ERR_INVALID, "flash_decode_poll: no scratch");
  int status = 0;
  L3CI_CUDA_TRY(cudaMemcpyAsync(&status, scratch, sizeof(int), cudaMemcpyDeviceToHost, stream));
  L3CI_CUDA_TRY(cudaStreamSynchronize(stream));
  if (status != 0) {
    // Records need no clearing; the header and every counter do.
    L3CI_CUDA_TRY(cudaMemsetAsync(scratch, 0, scratch_bytes, stream));
    return fail(status, "flash_decode: a bounded wait on a bulk copy ran out in an earlier launch");
  }
  return L3CI_OK;
}
