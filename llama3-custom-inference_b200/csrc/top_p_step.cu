// Nucleus (top-p) sampling step of a decode loop as one kernel: per sequence, the temperature softmax of its logits
// row, the nucleus of probability mass p, one draw from it, and the token bookkeeping that follows.
//
// The reference's sampling branch (model.py:367-369 `probs = softmax(logits / temperature)`, `sample_top_p`,
// model.py:400-423) sorts the whole vocabulary (128 256 entries) in descending order, takes the cumulative sum, drops
// every entry whose PRECEDING mass exceeds p, renormalises, draws with torch.multinomial and maps the draw back
// through the sort permutation: half a dozen full-vocabulary kernels per generated token.  The nucleus does not need
// the order, only its boundary: entry i is kept iff the mass of the entries that sort strictly before it is <= p.
// Here row b's CTA
//   1. reduces (max, sum of exp) online in one pass over the row,
//   2. finds the boundary of the nucleus by a two-level search over the bit pattern of the bf16 LOGITS (the weight
//      e_i = exp((x_i - max) / T) is monotone in the logit, and a bf16 logit has only 65 536 patterns): each level
//      histograms the MASS per byte value in shared memory (2^-40 fixed point, integer atomics: exact sums) and a
//      block-wide suffix scan finds the byte in which the preceding mass crosses p * sum; entries whose logit equals the boundary pattern tie exactly and are kept in
//      index order as long as the mass before them is <= p * sum (a stable descending sort puts them in that order),
//   3. draws u in [0, 1) from a Philox4x32-10 stream keyed by (seed; row, step) and walks the nucleus in INDEX order
//      (a block-wide scan of per-thread nucleus mass, then the owning thread walks its 128 entries) to the entry
//      where the running mass passes u * nucleus mass.  Any fixed order gives the multinomial distribution; index
//      order needs no permutation.
// Batches of up to half the SMs run as a cluster of two CTAs per row (see peer_value below).
// It then writes the token exactly as l3ci_greedy_step does.  Weights are recomputed from the logits in every pass
// (same expression, same bits; the row is 256 KB and stays in L2), nothing is sorted and nothing leaves the SM.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include "bf16x8.cuh"
#include "host_common.h"
#include "ptx_sm100.cuh"
#include "warp_reduce.cuh"

namespace l3ci {
namespace {

constexpr int kTopPBlock = 1024;
constexpr int kTopPWarps = kTopPBlock / kWarp;

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11): first word of the block.
__device__ __forceinline__ uint32_t philox_first(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}

// Block-wide exclusive prefix sum over the threads in index order, and the total.
template <typename T>
__device__ __forceinline__ T block_exclusive_scan(T v, T* red, T& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T inc = v;
#pragma unroll
  for (int d = 1; d < kWarp; d <<= 1) {
    const T o = __shfl_up_sync(kFullMask, inc, d);
    if (lane >= d) inc += o;
  }
  __syncthreads();
  if (lane == kWarp - 1) red[warp] = inc;
  __syncthreads();
  T w = red[lane], winc = w;
#pragma unroll
  for (int d = 1; d < kWarp; d <<= 1) {
    const T o = __shfl_up_sync(kFullMask, winc, d);
    if (lane >= d) winc += o;
  }
  total = __shfl_sync(kFullMask, winc, kWarp - 1);
  const T before_warp = __shfl_sync(kFullMask, winc - w, warp);
  return before_warp + inc - v;
}

typedef unsigned long long u64;

// Several CTAs per row (a cluster of 2, 4 or 8 while rows x CTAs fit the device): each walks its share of the row in
// every pass, and the few numbers a pass yields (maximum, histogram, totals of the scans) are read from the peers'
// shared memory.  All CTAs then hold the same values and take the same decisions; sums are integers, so the split
// changes no bit.
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
template <typename T>
__device__ __forceinline__ T ld_peer(const T* mine, uint32_t peer) {
  static_assert(sizeof(T) == 4 || sizeof(T) == 8, "32- or 64-bit values");
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(mine)), "r"(peer));
  if constexpr (sizeof(T) == 4) {
    uint32_t v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
    return *reinterpret_cast<T*>(&v);
  } else {
    u64 v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(remote) : "memory");
    return *reinterpret_cast<T*>(&v);
  }
}
// The CTAs' values of one quantity: each writes its own to a slot (no slot is used twice in a launch, so one cluster
// barrier per exchange is enough) and reads the others' after the barrier.  `before`: the sum over the CTAs in front
// of this one (the first CTA takes the front of the row); returns the sum over all.
template <int kCtas, typename T>
__device__ __forceinline__ T peer_sum(T mine, T* slot, uint32_t rank, T& before) {
  before = T(0);
  if constexpr (kCtas == 1) return mine;
  if (threadIdx.x == 0) *slot = mine;
  cluster_barrier();
  T all = T(0);
#pragma unroll
  for (uint32_t c = 0; c < (uint32_t)kCtas; ++c) {
    const T v = c == rank ? mine : ld_peer(slot, c);
    if (c < rank) before += v;
    all += v;
  }
  return all;
}
template <int kCtas>
__device__ __forceinline__ float peer_max(float mine, float* slot, uint32_t rank) {
  if constexpr (kCtas == 1) return mine;
  if (threadIdx.x == 0) *slot = mine;
  cluster_barrier();
  float m = mine;
#pragma unroll
  for (uint32_t c = 0; c < (uint32_t)kCtas; ++c)
    if (c != rank) m = fmaxf(m, ld_peer(slot, c));
  return m;
}

struct RowView {
  const __nv_bfloat16* row;
  long long vocab, nvec;   // nvec 16-byte vectors, then vocab - 8 * nvec scalars
  long long v_begin, v_end, s_begin;   // this CTA's vectors and where its scalars start (vocab: none)
  float scale, shift;      // weight of logit x: exp2(x * scale - shift), at most 1
  // The weight as a 2^-40 fixed-point integer.  (The hardware exponential, one instruction: a row is walked four
  // times and an SM has to evaluate 128 256 weights per pass; the same instruction on the same input gives the same
  // bits in every pass.)  All masses below are sums of these integers: exact, the same in whatever order they are
  // added (thousands of float additions of equal small terms into one accumulator all round the same way: torch's
  // own fp32 softmax is 7e-5 off on such rows), and addable with the integer atomics of shared memory — a float add
  // there is a compare-and-swap loop, which with 32 lanes on a few dozen hot bins retried ten times per add.
  __device__ __forceinline__ u64 weight(float x) const { return __float2ull_rn(fast_exp2(fmaf(x, scale, -shift)) * 1099511627776.f); }
};

// Order-preserving 16-bit key of a bf16 logit given as fp32 (larger logit, larger key; -0 and +0 share a key).  The
// weight is a monotone function of the logit and a bf16 logit has 65 536 patterns, so the nucleus boundary can be
// searched on the logit's own bits: two levels of 8 bits, and entries tie exactly when their logits are equal.
__device__ __forceinline__ uint32_t logit_key(float x) {
  const uint32_t u = __float_as_uint(x) >> 16;
  if (u == 0x8000u) return 0x8000u;                      // -0 -> +0
  return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u);
}

constexpr int kCopies = 8;   // histogram copies (warp w adds to copy w % 8): spreads the adds over more banks and keeps a
                             // 16-bit limb's sum below 2^32 (a copy sees at most 4 warps x 4096 entries)

// One level of the search: among all entries (level 0) or those whose key has `prefix` in its high byte (level 1), the
// byte value in which the mass of the strictly larger keys crosses `budget`.  Masses are histogrammed per byte value as
// three 16-bit limbs of the fixed-point weight (integer atomics), summed exactly, and a block-wide suffix scan over the
// 256 values finds the crossing.  Returns the byte (0xffffffff: the candidates all fit the budget) and subtracts the
// mass above it from `budget`.  On level 0 the budget is not known yet: the pass yields the sum of all weights
// (`total_out`) and the budget becomes top_p times it.  All threads take part and get the same answer.
template <int kCtas>
__device__ __forceinline__ uint32_t search_level(const RowView& rv, int level, uint32_t prefix, float top_p, u64& total_out,
                                                 u64& budget, uint32_t* limbs, u64* red, int* s_pick, u64* s_above, uint32_t rank) {
  for (int i = threadIdx.x; i < kCopies * 3 * 256; i += kTopPBlock) limbs[i] = 0u;
  __syncthreads();
  uint32_t* mine = limbs + ((threadIdx.x >> 5) % kCopies) * 3 * 256;
  // a thread adds up consecutive entries that fall into the same bin and issues the atomics once per run
  int run_bin = -1;
  u64 run_q = 0;
  auto flush = [&]() {
    if (run_bin >= 0) {
      atomicAdd(mine + run_bin, (uint32_t)(run_q & 0xffffu));
      atomicAdd(mine + 256 + run_bin, (uint32_t)((run_q >> 16) & 0xffffu));
      atomicAdd(mine + 512 + run_bin, (uint32_t)(run_q >> 32));
    }
  };
  auto visit = [&](float x) {
    const uint32_t key = logit_key(x);
    if (level != 0 && (key >> 8) != prefix) return;
    const int bin = level == 0 ? (int)(key >> 8) : (int)(key & 255u);
    const u64 q = rv.weight(x);
    if (bin == run_bin) run_q += q;
    else { flush(); run_bin = bin; run_q = q; }
  };
  for (long long v = rv.v_begin + threadIdx.x; v < rv.v_end; v += kTopPBlock) {
    float f[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(rv.row) + v), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) visit(f[j]);
  }
  for (long long i = rv.s_begin + threadIdx.x; i < rv.vocab; i += kTopPBlock) visit(__bfloat162float(rv.row[i]));
  flush();
  __syncthreads();
  if constexpr (kCtas > 1) cluster_barrier();   // the peers' histograms are complete too
  // thread t < 256 owns byte value d = 255 - t (a prefix scan over threads is then a suffix scan over byte values):
  // the wanted value is the largest d whose inclusive suffix sum exceeds the budget, i.e. the mass strictly above it
  // is still within the budget and the mass down to it is not
  u64 h = 0;
  const int d = 255 - (int)threadIdx.x;
  if (threadIdx.x < 256) {
#pragma unroll
    for (int c = 0; c < kCopies; ++c) {
      const uint32_t* l = limbs + c * 3 * 256;
      h += (u64)l[d] + ((u64)l[256 + d] << 16) + ((u64)l[512 + d] << 32);
      if constexpr (kCtas > 1) {
#pragma unroll
        for (uint32_t pc = 0; pc < (uint32_t)kCtas; ++pc)
          if (pc != rank) h += (u64)ld_peer(l + d, pc) + ((u64)ld_peer(l + 256 + d, pc) << 16) + ((u64)ld_peer(l + 512 + d, pc) << 32);
      }
    }
  }
  if constexpr (kCtas > 1) cluster_barrier();   // all have read: the histograms may be cleared for the next level
  u64 total;
  const u64 before = block_exclusive_scan<u64>(h, red, total);   // mass of the byte values above d
  total_out = total;
  if (level == 0) budget = (u64)((double)top_p * (double)total);
  if (threadIdx.x == 0) { *s_pick = -1; *s_above = total; }
  __syncthreads();
  if (threadIdx.x < 256 && before <= budget && before + h > budget) { *s_pick = d; *s_above = before; }
  __syncthreads();
  const int pick = *s_pick;
  if (pick < 0) return 0xffffffffu;
  budget -= *s_above;
  return (uint32_t)pick;
}

template <int kCtas>
__global__ void __launch_bounds__(kTopPBlock)
top_p_step_kernel(const __nv_bfloat16* __restrict__ logits, long long vocab, long long row_stride, float inv_temperature,
                  float top_p, unsigned long long seed, long long* __restrict__ out_tokens, long long out_stride,
                  long long out_cols, long long* __restrict__ steps, long long* __restrict__ next_input,
                  int* __restrict__ positions, int* __restrict__ seq_lens, int* __restrict__ nucleus_count,
                  float* __restrict__ nucleus_mass) {
  __shared__ uint32_t limbs[kCopies * 3 * 256];
  __shared__ float redf[kTopPWarps];
  __shared__ u64 red[kTopPWarps];
  __shared__ long long redl[kTopPWarps];
  __shared__ int s_pick;
  __shared__ u64 s_above;
  __shared__ int s_owner;
  __shared__ long long s_token;
  __shared__ u64 s_slots[8];     // values for the peer CTA, one slot per exchange
  pdl_wait();               // the previous kernel of the stream has completed; its writes are visible
  pdl_launch_dependents();  // the next one may be set up while this one runs
  const long long b = blockIdx.x / kCtas;
  const uint32_t rank = kCtas > 1 ? cluster_rank() : 0u;
  RowView rv;
  rv.row = logits + b * row_stride;
  rv.vocab = vocab;
  rv.nvec = (reinterpret_cast<uintptr_t>(rv.row) & 15u) == 0 ? vocab / kVecElems : 0;
  rv.scale = inv_temperature * 1.4426950408889634f;
  // this CTA's share of the row in the passes that take it in any order: half of the vectors each, the scalars
  // behind them with the last CTA
  rv.v_begin = rv.nvec * rank / kCtas;
  rv.v_end = rv.nvec * (rank + 1) / kCtas;
  rv.s_begin = rank == kCtas - 1 ? rv.nvec * kVecElems : vocab;

  // ---- 1. maximum of the row (the sum of the weights falls out of the first histogram) ----
  float m = -INFINITY;
  for (long long v = rv.v_begin + threadIdx.x; v < rv.v_end; v += kTopPBlock) {
    float f[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(rv.row) + v), f);
    m = fmaxf(m, fmaxf(fmaxf(fmaxf(f[0], f[1]), fmaxf(f[2], f[3])), fmaxf(fmaxf(f[4], f[5]), fmaxf(f[6], f[7]))));
  }
  for (long long i = rv.s_begin + threadIdx.x; i < vocab; i += kTopPBlock) m = fmaxf(m, __bfloat162float(rv.row[i]));
  m = group_max<kWarp>(m);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) redf[threadIdx.x >> 5] = m;
  __syncthreads();
  float row_max = group_max<kWarp>(redf[threadIdx.x & 31]);
  row_max = peer_max<kCtas>(row_max, reinterpret_cast<float*>(&s_slots[0]), rank);
  rv.shift = row_max * rv.scale;

  // ---- 2. boundary of the nucleus: the largest logit pattern k* whose strictly-larger mass is still <= p * Z ----
  uint32_t key_star = 0u;
  bool all_kept = false;
  u64 Z = 0, budget = 0, bud = 0;
  {
    const uint32_t hi = search_level<kCtas>(rv, 0, 0u, top_p, Z, bud, limbs, red, &s_pick, &s_above, rank);
    budget = (u64)((double)top_p * (double)Z);
    if (hi == 0xffffffffu) {
      all_kept = true;   // top_p >= 1
    } else {
      u64 unused;
      const uint32_t lo = search_level<kCtas>(rv, 1, hi, 0.f, unused, bud, limbs, red, &s_pick, &s_above, rank);
      key_star = (hi << 8) | (lo == 0xffffffffu ? 0u : lo);   // (the sums are exact, so the second level finds its byte)
    }
  }
  const u64 above = budget - bud;   // mass of the entries whose logit is strictly above the boundary pattern
  // weight of the boundary pattern: the bf16 logit it stands for, through the same expression as every entry
  const uint32_t bits_star = (key_star & 0x8000u) ? (key_star & 0x7fffu) : (~key_star & 0xffffu);
  const u64 w_star = rv.weight(__uint_as_float(bits_star << 16));

  // ---- 3. nucleus mass per thread over a CONTIGUOUS run of the row (index order), ties at the boundary counted ----
  // runs of a multiple of 8 entries, so that an aligned row is walked with 16-byte loads
  constexpr long long kRowThreads = (long long)kTopPBlock * kCtas;   // the first CTA takes the front of the row
  const long long per = ((vocab + kRowThreads - 1) / kRowThreads + kVecElems - 1) / kVecElems * kVecElems;
  const long long row_thread = (long long)rank * kTopPBlock + threadIdx.x;
  const long long i_begin = row_thread * per < vocab ? row_thread * per : vocab;
  const long long i_end = i_begin + per < vocab ? i_begin + per : vocab;
  // calls fn(index, logit) for the entries of this thread's run in increasing order until fn returns true
  auto walk = [&](auto&& fn) {
    long long i = i_begin;
    if (rv.nvec > 0) {
      for (; i + kVecElems <= i_end; i += kVecElems) {
        float f[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(rv.row) + i / kVecElems), f);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (fn(i + j, f[j])) return;
      }
    }
    for (; i < i_end; ++i)
      if (fn(i, __bfloat162float(rv.row[i]))) return;
  };
  u64 w_mine = 0;
  long long n_eq = 0, n_above = 0;
  walk([&](long long, float x) {
    const uint32_t key = logit_key(x);
    if (all_kept || key > key_star) { w_mine += rv.weight(x); ++n_above; }
    else if (key == key_star) ++n_eq;
    return false;
  });
  long long eq_total;
  long long eq_before = block_exclusive_scan<long long>(n_eq, redl, eq_total);
  {   // index order over the CTAs: a CTA's entries come after all of those in front of it
    long long front;
    eq_total = peer_sum<kCtas>(eq_total, reinterpret_cast<long long*>(&s_slots[1]), rank, front);
    eq_before += front;
  }
  // entries equal to the boundary pattern, in index order: the j-th is kept while above + j * w* <= budget
  long long eq_kept = 0;
  if (!all_kept && eq_total > 0) {
    eq_kept = w_star > 0 ? (long long)((budget > above ? budget - above : 0) / w_star) + 1 : eq_total;
    if (eq_kept > eq_total) eq_kept = eq_total;
  }
  long long eq_mine = eq_kept - eq_before;
  eq_mine = eq_mine < 0 ? 0 : (eq_mine > n_eq ? n_eq : eq_mine);
  const u64 mass_mine = w_mine + (u64)eq_mine * w_star;
  u64 mass_total;
  u64 mass_before = block_exclusive_scan<u64>(mass_mine, red, mass_total);
  {
    u64 front;
    mass_total = peer_sum<kCtas>(mass_total, &s_slots[2], rank, front);
    mass_before += front;
  }

  // ---- 4. the draw: u in [0, 1) with 32 bits, target = floor(u * nucleus mass) < nucleus mass ----
  const long long step = steps ? steps[b] : 0;
  const uint32_t r = philox_first((uint32_t)seed, (uint32_t)(seed >> 32), (uint32_t)b, (uint32_t)(b >> 32), (uint32_t)step,
                                  (uint32_t)(step >> 32));
  const u64 target = __umul64hi(mass_total, (u64)r << 32);
  if (threadIdx.x == 0) s_owner = kTopPBlock;
  __syncthreads();
  if (mass_mine > 0 && mass_before <= target && target < mass_before + mass_mine) s_owner = (int)threadIdx.x;   // exactly one thread
  __syncthreads();
  // The thread whose run holds the target sits in one of the CTAs; that CTA writes the token.  An empty nucleus (a
  // row of NaNs) has no such thread: the first CTA's first thread stands in.
  const bool mine = s_owner < kTopPBlock || (mass_total == 0 && rank == 0);
  const int owner = s_owner < kTopPBlock ? s_owner : 0;
  if (mine && (int)threadIdx.x == owner) {
    u64 run = mass_before;
    long long eq_seen = eq_before, tok = -1, last = -1;
    walk([&](long long i, float x) {
      const uint32_t key = logit_key(x);
      bool in = all_kept || key > key_star;
      if (!in && key == key_star) { in = eq_seen < eq_kept; ++eq_seen; }
      if (!in) return false;
      last = i;
      run += rv.weight(x);
      if (run > target) { tok = i; return true; }
      return false;
    });
    if (tok < 0) tok = last >= 0 ? last : (i_begin < vocab ? i_begin : 0);
    s_token = tok;
  }
  __syncthreads();
  if (mine && threadIdx.x == 0) {
    const long long tok = s_token;
    if (out_tokens && steps) {
      if (step >= 0 && step < out_cols) out_tokens[b * out_stride + step] = tok;
      steps[b] = step + 1;
    } else if (out_tokens) {
      out_tokens[b * out_stride] = tok;
    }
    if (next_input) next_input[b] = tok;
    if (positions) positions[b] += 1;
    if (seq_lens) seq_lens[b] += 1;
    if (nucleus_mass) nucleus_mass[b] = Z > 0 ? (float)((double)mass_total / (double)Z) : 0.f;
  }
  if (nucleus_count) {
    long long total;
    block_exclusive_scan<long long>(n_above + eq_mine, redl, total);
    long long front;
    total = peer_sum<kCtas>(total, reinterpret_cast<long long*>(&s_slots[3]), rank, front);
    if (threadIdx.x == 0 && rank == 0) nucleus_count[b] = (int)total;
  }
  if constexpr (kCtas > 1) cluster_barrier();   // no CTA leaves while a peer may still read its shared memory
}

}  // namespace
}  // namespace l3ci

extern "C" int l3ci_top_p_step(const void* logits, int64_t rows, int64_t vocab, int64_t row_stride, float temperature,
                               float top_p, uint64_t seed, int64_t* out_tokens, int64_t out_stride, int64_t out_cols,
                               int64_t* steps, int64_t* next_input, int32_t* positions, int32_t* seq_lens,
                               int32_t* nucleus_count, float* nucleus_mass, l3ci_stream_t stream_) {
  using namespace l3ci;
  clear_error();
  if (rows < 0 || vocab <= 0 || row_stride < vocab) return fail(L3CI_ERR_INVALID, "top_p_step: bad size");
  if (!(temperature > 0.f)) return fail(L3CI_ERR_INVALID, "top_p_step: temperature must be positive (use l3ci_greedy_step for 0)");
  if (!(top_p > 0.f)) return fail(L3CI_ERR_INVALID, "top_p_step: top_p must be positive");
  if (rows == 0) return L3CI_OK;
  if (!logits || (!out_tokens && !next_input)) return fail(L3CI_ERR_INVALID, "top_p_step: null logits or no output");
  if (rows > 0x7fffffffLL) return fail(L3CI_ERR_INVALID, "top_p_step: too many rows");
  if (steps && (!out_tokens || out_cols <= 0)) return fail(L3CI_ERR_INVALID, "top_p_step: steps needs out_tokens and its width");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const auto lp = static_cast<const __nv_bfloat16*>(logits);
  const float inv_t = 1.0f / temperature;
  const int sms = sm_count();
  // Small batches: a cluster of CTAs per row, as many (8, 4, 2) as still run all at once, so that the batch covers
  // the device (64 rows: 128 SMs; one row: 8).  A 148-SM part holds 15 clusters of 8, 33 of 4 or 74 of 2 of these
  // CTAs at a time (cudaOccupancyMaxActiveClusters); the bounds scale with the SM count.
  const int ctas_per_row = sms <= 0 ? 1 : rows * 148 <= 15LL * sms ? 8 : rows * 148 <= 33LL * sms ? 4 : 2 * rows <= sms ? 2 : 1;
  // (a cluster size the device or its partition cannot place falls back to the next smaller one)
  for (int c = ctas_per_row; c > 1; c /= 2) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(c * rows));
    cfg.blockDim = dim3(kTopPBlock);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)c;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    auto launch = [&](auto kernel) {
      return cudaLaunchKernelEx(&cfg, kernel, lp, (long long)vocab, (long long)row_stride, inv_t, top_p, (unsigned long long)seed,
                                reinterpret_cast<long long*>(out_tokens), (long long)out_stride, (long long)out_cols,
                                reinterpret_cast<long long*>(steps), reinterpret_cast<long long*>(next_input), positions, seq_lens,
                                nucleus_count, nucleus_mass);
    };
    const cudaError_t e = c == 8 ? launch(top_p_step_kernel<8>) : c == 4 ? launch(top_p_step_kernel<4>) : launch(top_p_step_kernel<2>);
    if (e == cudaSuccess) return L3CI_OK;
    (void)cudaGetLastError();   // not placed: nothing ran
  }
  L3CI_LAUNCH("top_p_step_kernel", top_p_step_kernel<1>, dim3((unsigned)rows), dim3(kTopPBlock), 0, stream,
              lp, (long long)vocab, (long long)row_stride, inv_t, top_p, (unsigned long long)seed,
              reinterpret_cast<long long*>(out_tokens), (long long)out_stride, (long long)out_cols, reinterpret_cast<long long*>(steps),
              reinterpret_cast<long long*>(next_input), positions, seq_lens, nucleus_count, nucleus_mass);
  return L3CI_OK;
}
