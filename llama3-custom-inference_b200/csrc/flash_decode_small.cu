// Decode attention without a pass through global memory: the partial results of one unit (a sequence's KV head)
// meet in shared memory.
//
// The persistent kernel of flash_decode.cu balances any mix of lengths over the whole device, and pays for it
// with fixed latencies per launch (tensor-map fetch, cross-CTA merge through global memory) of about 10 us.  That
// is most of a call like the reference's own example (one sequence of 256 tokens, benchmark_kernel.py:160-163:
// 0.5 MB of K and V) and a third of a batched decode step of a few thousand tokens per sequence.  Here a unit is
// dealt statically: to W of a CTA's eight warps (8 / W units per CTA, for many short units), to the eight warps
// of one CTA, or to the C CTAs of a thread-block cluster (for few long units), whose per-CTA results meet through
// distributed shared memory.  K and V rows go from global to shared memory with 16-byte asynchronous copies
// (written in the 128-byte-swizzled layout that ldmatrix expects), three tiles in flight per warp; the tile
// arithmetic is the one of the persistent kernel (S^T = K Q^T and O^T = V^T P^T on mma.sync.m16n8k16, tokens on
// the rows of a tile, the group's query heads on its 8 columns).  Taken by l3ci_flash_decode where
// fd_static_applies (flash_decode_plan.h) expects it to be faster, for at most 8 query heads per KV head; results
// agree with the persistent kernel's within rounding.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include "bf16x8.cuh"
#include "flash_decode_plan.h"
#include "host_common.h"
#include "ptx_sm100.cuh"
#include "warp_reduce.cuh"

namespace l3ci {
namespace {

constexpr int kSmWarps = 8;
constexpr int kSmSlots = 3;  // tiles in flight per warp
// Few CTAs with long runs of tiles each have an SM's intake to themselves: there the warps wait on their own
// instructions, not on memory, and 12 warps with 2 tiles in flight each (the same shared memory) issue more
// (131072 tokens of one sequence: 84 us instead of 91; short runs lose a little to the finer deal).
constexpr int kClWarps = 12;
constexpr int kClSlots = 2;
static_assert(kClWarps * kClSlots == kSmWarps * kSmSlots, "both shapes of a CTA fill the same shared memory");

struct SmallParams {
  const __nv_bfloat16 *q, *k, *v;
  __nv_bfloat16* out;
  float* o_partial;
  float* lse;
  const int* seq_lens;
  int B, Hq, Hkv, R, n_seq;
  int lgW, lgC;  // log2 of: warps per unit (1, 2, 4, 8), CTAs per unit (a cluster; > 1 only with 8 warps per unit)
  long long q_sb, q_sh, k_sb, k_sh, k_st, v_sb, v_sh, v_st, o_sb, o_sh;
  float scale_log2e;
  // kExchange instances: the KV sequence is sharded over `xranks` GPUs and the per-GPU results are merged here
  unsigned long long* const* xbufs;  // device array of the ranks' exchange buffers (peer-mapped), [xrank] the local one
  int xrank, xranks;
  unsigned xepoch;                   // call number, the same on all ranks; 0 = kept in the buffer's control words
  int* xstatus;                      // optional: receives L3CI_ERR_DEVICE_WAIT when a peer's values do not arrive
  unsigned long long xwait_ns;
};

// ---------------------------------------------------------------------------------------------
// Exchange of shard results across GPUs, folded into the tail of the decode kernel.
//
// With the KV sequence of a long context sharded over W GPUs, every GPU runs this kernel on its shard and ends up,
// per output element (query row, column), with a softmax-normalised value and the row's log-sum-exp.  Instead of
// writing them out for a second kernel, the thread that holds an element
//   1. stores (value, call number) as ONE 64-bit word into the same place of every peer's exchange buffer (plain
//      stores over NVLink; the thread of column 0 also sends the row's log-sum-exp),
//   2. polls its own buffer until the W - 1 peers' words for that element and that row carry this call's number
//      (a 64-bit store is single-copy atomic: a word that shows the number holds the value, so there is no fence,
//      no separate flag and no second round trip),
//   3. merges the W values by log-sum-exp and writes the bf16 output.
// Buffer (64-bit words): [2 parities][W source ranks][rows * (D + 1)], word row * (D + 1) + col, col == D for the
// log-sum-exp; then 2 control words (call number | CTAs finished).  Call e uses parity e & 1: a rank can only
// start call e + 2 after it finished call e + 1, which needed every peer's words of call e + 1, which a peer sends
// only at the end of a kernel that runs after its own call e has finished reading.  The wait is bounded: when it
// runs out the element is left unwritten and the status word set.  Loads of remote memory: none.
// ---------------------------------------------------------------------------------------------
constexpr int kXchgMaxRanks = 8;

__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

struct XchgView {
  long long words;   // rows * (D + 1)
  unsigned epoch;
  unsigned long long* ctrl;
};
template <int D>
__device__ __forceinline__ XchgView xchg_begin(const SmallParams& p) {
  XchgView x;
  x.words = (long long)p.B * p.Hq * (D + 1);
  x.ctrl = p.xbufs[p.xrank] + 2LL * p.xranks * x.words;
  // (read before this CTA counts itself finished; the number only moves once every CTA has)
  x.epoch = p.xepoch ? p.xepoch : (unsigned)__ldcg(reinterpret_cast<const unsigned*>(x.ctrl)) + 1u;
  return x;
}
// Steps 1-3 for the element (row, col) of this GPU's shard result; returns false if the wait ran out.
template <int D>
__device__ __forceinline__ bool xchg_element(const SmallParams& p, const XchgView& x, long long row, int col, float val,
                                             float lse, float& merged) {
  const int W = p.xranks, me = p.xrank;
  const long long at = row * (D + 1) + col, at_lse = row * (D + 1) + D;
  const long long mine = ((long long)(x.epoch & 1u) * W + me) * x.words;
  const unsigned long long tag = (unsigned long long)x.epoch << 32;
#pragma unroll
  for (int s = 0; s < kXchgMaxRanks; ++s)
    if (s < W && s != me) {
      unsigned long long* dst = p.xbufs[s] + mine;
      st_relaxed_sys_u64(dst + at, tag | __float_as_uint(val));
      if (col == 0) st_relaxed_sys_u64(dst + at_lse, tag | __float_as_uint(lse));
    }
  const unsigned long long* loc = p.xbufs[me] + (long long)(x.epoch & 1u) * W * x.words;
  float v[kXchgMaxRanks], l[kXchgMaxRanks];
  unsigned got = 0;
#pragma unroll
  for (int s = 0; s < kXchgMaxRanks; ++s) {
    v[s] = 0.f;
    l[s] = -INFINITY;
    if (s >= W || s == me) got |= 1u << s;
  }
  v[me & (kXchgMaxRanks - 1)] = val;
  l[me & (kXchgMaxRanks - 1)] = lse;
  unsigned long long t0 = 0;
  for (unsigned it = 0; got != (1u << kXchgMaxRanks) - 1u; ++it) {
#pragma unroll
    for (int s = 0; s < kXchgMaxRanks; ++s)
      if (!((got >> s) & 1u)) {
        const unsigned long long a = ld_relaxed_sys_u64(loc + s * x.words + at);
        const unsigned long long b = ld_relaxed_sys_u64(loc + s * x.words + at_lse);
        if ((unsigned)(a >> 32) == x.epoch && (unsigned)(b >> 32) == x.epoch) {
          v[s] = __uint_as_float((unsigned)a);
          l[s] = __uint_as_float((unsigned)b);
          got |= 1u << s;
        }
      }
    if ((it & 31u) == 31u) {
      const unsigned long long now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > p.xwait_ns) {
        if (p.xstatus) atomicExch(p.xstatus, (int)L3CI_ERR_DEVICE_WAIT);
        return false;
      }
    }
  }
  float M = -INFINITY;
#pragma unroll
  for (int s = 0; s < kXchgMaxRanks; ++s) M = fmaxf(M, l[s]);
  const float Mu = M == -INFINITY ? 0.f : M;
  float L = 0.f, acc = 0.f;
#pragma unroll
  for (int s = 0; s < kXchgMaxRanks; ++s) {
    const float w = __expf(l[s] - Mu);  // exp(-inf) = 0: an empty shard, or a rank beyond W
    L += w;
    acc = fmaf(v[s], w, acc);
  }
  merged = L > 0.f ? acc / L : 0.f;
  return true;
}
// The last CTA of the launch to finish advances the call number kept in the buffer (xepoch == 0).
__device__ __forceinline__ void xchg_end(const SmallParams& p, const XchgView& x) {
  if (p.xepoch == 0u && threadIdx.x == 0) {
    unsigned* c = reinterpret_cast<unsigned*>(x.ctrl);
    if (atomicAdd(c + 2, 1u) == gridDim.x - 1u) {
      c[2] = 0u;
      __threadfence();
      c[0] = x.epoch;
    }
  }
}

// (policy: the cache is read once, so its lines are the first to leave L2: 3-4 % on calls of a few clusters)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid, uint64_t policy) {
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;" ::"r"(dst), "l"(src), "r"(bytes), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// All threads of all CTAs of the cluster: shared-memory writes before it are visible to the cluster after it.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Reads a float at this CTA's shared address `addr`, but in the shared memory of CTA `cta` of the cluster.
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr, uint32_t cta) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(cta));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// kCluster: launched as clusters of CTAs per unit (the instances without hold no cluster instruction and are
// launched without the cluster attribute, which starts sooner).  kWholeCta: all eight warps on one unit, known at compile time
// (the merge loops then unroll without predicates: 0.5 us on a call of a few microseconds).
// kWide: 12 warps x 2 tiles in flight instead of 8 x 3 (cluster instances on long runs of tiles).
// kExchange: the results of this launch are one GPU's shard of a sequence-sharded cache; the exchange with the
// other GPUs and the merge happen in the kernel's tail (above) and `out` receives the merged attention.
template <int D, bool kCluster, bool kWholeCta, bool kWide = false, bool kExchange = false>
__global__ void __launch_bounds__(32 * (kWide ? kClWarps : kSmWarps))
flash_decode_small_kernel(const SmallParams p) {
  static_assert(kWholeCta || !kCluster, "a cluster works on one unit with all warps of its CTAs");
  static_assert(kCluster || !kWide, "the wide shape is built for cluster instances only");
  constexpr int NW = kWide ? kClWarps : kSmWarps;  // warps of the CTA
  constexpr int NS = kWide ? kClSlots : kSmSlots;  // tiles in flight per warp
  constexpr int kTile = fd_tile_tokens(D);   // tokens per tile: 4 KB of K and 4 KB of V
  constexpr int kHalves = D / 64;
  constexpr int kBoxBytes = kTile * 128;     // one 64-column half of a tile
  constexpr int kTileBytes = 2 * kHalves * kBoxBytes;  // K then V
  constexpr int KS = D / 16, MB = kTile / 16, MT = D / 16;
  constexpr int kStateFloats = 8 * D + 16;   // o[8 rows][D], m[8], l[8]
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* states = reinterpret_cast<float*>(smem);  // [NW][kStateFloats], over the tile slots once all warps are done
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  // (shifts, not divisions: they sit on the path to the first copy)
  const int R = p.R, lgW = kWholeCta ? 0 : p.lgW, lgC = kCluster ? p.lgC : 0;
  const int W = kWholeCta ? NW : 1 << lgW, C = 1 << lgC;
  const int U = kWholeCta ? 1 : NW >> lgW;          // units per CTA
  uint32_t cta_rank = 0;
  if constexpr (kCluster) cta_rank = cluster_cta_rank();
  const int n_units = p.B * p.Hkv;
  pdl_wait();               // the previous kernel of the stream has completed; its writes are visible
  pdl_launch_dependents();  // the next one may be set up while this one runs
  const int unit0 = (int)(blockIdx.x >> lgC) * U;   // first unit of this CTA (of this cluster)
  const int unit = unit0 + (kWholeCta ? 0 : warp >> lgW);
  const bool has_unit = unit < n_units;
  const int b = has_unit ? unit / p.Hkv : 0, head = has_unit ? unit % p.Hkv : 0;
  const int len = !has_unit ? 0 : p.seq_lens ? min(max(__ldg(p.seq_lens + b), 0), p.n_seq) : p.n_seq;

  // this warp's tiles: the unit's tiles are dealt in contiguous runs to its C * W warps
  const int n_tiles = (len + kTile - 1) / kTile;
  const int part = (int)cta_rank * W + (kWholeCta ? warp : warp & (W - 1)), parts = C * W;
  const int t_each = kWholeCta ? (n_tiles >> lgC) / NW : n_tiles >> (lgW + lgC);
  const int t_more = n_tiles - t_each * parts;  // the first t_more parts get one more
  const int t_begin = part * t_each + min(part, t_more), t_end = t_begin + t_each + (part < t_more ? 1 : 0);
  const __nv_bfloat16* kbase = p.k + (long long)b * p.k_sb + (long long)head * p.k_sh;
  const __nv_bfloat16* vbase = p.v + (long long)b * p.v_sb + (long long)head * p.v_sh;
  const uint32_t buf0 = smem_u32(smem) + warp * NS * kTileBytes;

  // Copy of one tile: 16-byte chunk c (0..7) of 128-byte row r of half h goes to chunk position c ^ (r & 7).  A
  // pass of the warp covers 4 rows x 8 chunks; lane (r0, c) keeps one pointer per tensor and steps it by 4 rows
  // (the copies are a third of the instructions of a tile otherwise).  Always one commit group per call, empty
  // past the warp's last tile, so that "all but the newest NS - 1 groups" is the tile about to be used.
  const uint64_t policy = l2_evict_first_policy();
  const int r0 = lane >> 3, c8 = lane & 7;
  const __nv_bfloat16* klane = kbase + (long long)r0 * p.k_st + c8 * 8;
  const __nv_bfloat16* vlane = vbase + (long long)r0 * p.v_st + c8 * 8;
  const long long k4 = 4 * p.k_st, v4 = 4 * p.v_st;
  // row r0 + 4 j sits at (r0 + 4 j) * 128, its chunk at c ^ r0 ^ (4 * (j & 1)) since r0 < 4
  const uint32_t d_even = r0 * 128 + ((c8 ^ r0) << 4), d_odd = r0 * 128 + ((c8 ^ r0 ^ 4) << 4);
  auto fetch = [&](int tile, int slot) {
    if (tile < t_end) {
      const uint32_t dst = buf0 + slot * kTileBytes;
      const long long t0 = (long long)tile * kTile;
      const __nv_bfloat16* kp = klane + t0 * p.k_st;
      const __nv_bfloat16* vp = vlane + t0 * p.v_st;
      if (tile * kTile + kTile <= len) {
#pragma unroll
        for (int j = 0; j < kTile / 4; ++j) {
          const uint32_t d = dst + j * 512 + ((j & 1) ? d_odd : d_even);
#pragma unroll
          for (int h = 0; h < kHalves; ++h) {
            cp_async16(d + h * kBoxBytes, kp + h * 64, true, policy);
            cp_async16(d + (kHalves + h) * kBoxBytes, vp + h * 64, true, policy);
          }
          kp += k4;
          vp += v4;
        }
      } else {  // the sequence ends inside this tile: rows past its end are zero-filled, nothing is read for them
#pragma unroll
        for (int j = 0; j < kTile / 4; ++j) {
          const uint32_t d = dst + j * 512 + ((j & 1) ? d_odd : d_even);
          const bool ok = tile * kTile + r0 + 4 * j < len;
#pragma unroll
          for (int h = 0; h < kHalves; ++h) {
            cp_async16(d + h * kBoxBytes, ok ? kp + h * 64 : kbase, ok, policy);
            cp_async16(d + (kHalves + h) * kBoxBytes, ok ? vp + h * 64 : vbase, ok, policy);
          }
          kp += k4;
          vp += v4;
        }
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int i = 0; i < NS; ++i) fetch(t_begin + i, i);

  // Q^T fragments of the group's query heads (rows >= R are zero)
  uint32_t qb[KS][2];
  {
    const __nv_bfloat16* qp = p.q + (long long)b * p.q_sb + (long long)(head * R) * p.q_sh;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int col = ks * 16 + 2 * tig;
      qb[ks][0] = gid < R ? ld_global_u32(qp + gid * p.q_sh + col) : 0u;
      qb[ks][1] = gid < R ? ld_global_u32(qp + gid * p.q_sh + col + 8) : 0u;
    }
  }
  const int mat = lane >> 3, r8 = lane & 7;
  const uint32_t k_row_off = (r8 + 8 * (mat & 1)) * 128, k_x = (mat >> 1) ^ r8;
  const uint32_t v_row_off = (r8 + 8 * (mat >> 1)) * 128, v_x = (mat & 1) ^ r8;
  float o[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // this thread's query rows 2 tig, 2 tig + 1

  for (int t = t_begin; t < t_end; ++t) {
    const int slot = (t - t_begin) % NS;
    cp_async_wait<NS - 1>();
    __syncwarp();
    const uint32_t kb = buf0 + slot * kTileBytes, vb = kb + kHalves * kBoxBytes;
    // S^T = K Q^T
    // (the k-steps go to kAcc accumulator sets summed at the end: a chain of KS dependent MMAs is 20 cycles each)
    constexpr int kAcc = MB == 1 ? 4 : 2;
    float sp[kAcc][MB][4];
#pragma unroll
    for (int a = 0; a < kAcc; ++a)
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) sp[a][mb][0] = sp[a][mb][1] = sp[a][mb][2] = sp[a][mb][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        uint32_t a0, a1, a2, a3;
        ldsm_x4(kb + (ks >> 2) * kBoxBytes + mb * 2048 + k_row_off + (((2u * (ks & 3)) ^ k_x) << 4), a0, a1, a2, a3);
        mma_bf16(sp[ks % kAcc][mb], a0, a1, a2, a3, qb[ks][0], qb[ks][1]);
      }
    float s[MB][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float acc = sp[0][mb][e];
#pragma unroll
        for (int a = 1; a < kAcc; ++a) acc += sp[a][mb][e];
        s[mb][e] = acc;
      }
    // mask the end of the sequence (rows beyond len were zero-filled: finite scores, masked here)
    const int tok0 = t * kTile;
    if (tok0 + kTile > len) {
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        const int tk = tok0 + mb * 16 + gid;
        if (tk >= len) s[mb][0] = s[mb][1] = -INFINITY;
        if (tk + 8 >= len) s[mb][2] = s[mb][3] = -INFINITY;
      }
    }
    // online softmax in the log2 domain; reductions over the 8 lanes of a column pair
    uint32_t pb[MB][2];
    float alpha[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float mx = -INFINITY;
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) mx = fmaxf(mx, fmaxf(s[mb][j], s[mb][2 + j]));
      mx = fmaxf(mx, __shfl_xor_sync(kFullMask, mx, 4));
      mx = fmaxf(mx, __shfl_xor_sync(kFullMask, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(kFullMask, mx, 16)) * p.scale_log2e;
      const float mn = fmaxf(m_run[j], mx);
      const float mu = mn == -INFINITY ? 0.f : mn;
      alpha[j] = fast_exp2(m_run[j] - mu);
      m_run[j] = mn;
      float ps = 0.f;
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        s[mb][j] = fast_exp2(fmaf(s[mb][j], p.scale_log2e, -mu));
        s[mb][2 + j] = fast_exp2(fmaf(s[mb][2 + j], p.scale_log2e, -mu));
        ps += s[mb][j] + s[mb][2 + j];
      }
      l_run[j] = fmaf(l_run[j], alpha[j], ps);
    }
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
      pb[mb][0] = movmatrix_trans(pack_bf16x2(s[mb][0], s[mb][1]));
      pb[mb][1] = movmatrix_trans(pack_bf16x2(s[mb][2], s[mb][3]));
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      o[mt][0] *= alpha[0]; o[mt][1] *= alpha[1];
      o[mt][2] *= alpha[0]; o[mt][3] *= alpha[1];
    }
    // O^T += V^T P^T
#pragma unroll
    for (int kk = 0; kk < MB; ++kk)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t a0, a1, a2, a3;
        ldsm_x4_trans(vb + (mt >> 2) * kBoxBytes + kk * 2048 + v_row_off + (((2u * (mt & 3)) ^ v_x) << 4), a0, a1, a2, a3);
        mma_bf16(o[mt], a0, a1, a2, a3, pb[kk][0], pb[kk][1]);
      }
    __syncwarp();
    fetch(t + NS, slot);
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with its slots: the states go over them

  // ---- this warp's state to shared memory: o[row][col], m[row], l[row] for rows 0..7 ----
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    l_run[j] += __shfl_xor_sync(kFullMask, l_run[j], 4);
    l_run[j] += __shfl_xor_sync(kFullMask, l_run[j], 8);
    l_run[j] += __shfl_xor_sync(kFullMask, l_run[j], 16);
  }
  float* st = states + warp * kStateFloats;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int row = 2 * tig + j;
      st[row * D + 16 * mt + gid] = o[mt][j];
      st[row * D + 16 * mt + gid + 8] = o[mt][2 + j];
    }
  if (gid == 0) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      st[8 * D + 2 * tig + j] = m_run[j];
      st[8 * D + 8 + 2 * tig + j] = l_run[j];
    }
  }
  __syncthreads();

  XchgView xv{};
  if constexpr (kExchange) xv = xchg_begin<D>(p);
  // ---- first level: the W states of each of this CTA's units.  Every thread folds them for its output elements
  //      (weights recomputed per element: a table built by a few threads first was slower by 0.5 us) ----
  float* cstate = states + NW * kStateFloats;  // [R * D] unnormalised sums, then m[8], l[8] (used with C > 1)
  const int RD = R * D;
  for (int u = 0; u < U; ++u) {
    const bool live = unit0 + u < n_units;
    const int ub = live ? (unit0 + u) / p.Hkv : 0, uh = live ? (unit0 + u) - ub * p.Hkv : 0;
    const float* s0 = states + (u * W) * kStateFloats;
    for (int r = threadIdx.x; r < RD && live; r += 32 * NW) {
      const int row = r / D, col = r - row * D;
      float m_w[NW];
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        m_w[w] = w < W ? s0[w * kStateFloats + 8 * D + row] : -INFINITY;
        M = fmaxf(M, m_w[w]);
      }
      const float Mu = M == -INFINITY ? 0.f : M;
      float L = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w)
        if (w < W) {
          const float wgt = fast_exp2(m_w[w] - Mu);
          L = fmaf(s0[w * kStateFloats + 8 * D + 8 + row], wgt, L);
          acc = fmaf(s0[w * kStateFloats + row * D + col], wgt, acc);
        }
      if (kCluster) {
        cstate[r] = acc;
        if (col == 0) { cstate[8 * D + row] = M; cstate[8 * D + 8 + row] = L; }
      } else {
        float val = L > 0.f ? acc / L : 0.f;
        const float lse = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
        const long long hq = (long long)uh * R + row;
        if constexpr (kExchange) {
          if (!xchg_element<D>(p, xv, (long long)ub * p.Hq + hq, col, val, lse, val)) continue;
        }
        if (p.out) p.out[(long long)ub * p.o_sb + hq * p.o_sh + col] = __float2bfloat16(val);
        if (p.o_partial) {
          p.o_partial[((long long)ub * p.Hq + hq) * D + col] = val;
          if (col == 0) p.lse[(long long)ub * p.Hq + hq] = lse;
        }
      }
    }
  }
  if constexpr (!kCluster) {
    if constexpr (kExchange) {
      __syncthreads();  // every thread of the CTA has read the call number and is done with its elements
      xchg_end(p, xv);
    }
    return;
  }

  if constexpr (kCluster) {
  // ---- second level: the C per-CTA states of the unit, read through distributed shared memory; this CTA
  //      finishes its 1/C of the unit's output elements ----
  cluster_sync();
  const uint32_t cs = smem_u32(cstate);
  const int share = RD >> lgC;  // D is a multiple of 64 and C at most 8
  for (int r = (int)cta_rank * share + (int)threadIdx.x; r < ((int)cta_rank + 1) * share && has_unit; r += 32 * NW) {
    const int row = r / D, col = r - row * D;
    float m_c[8], l_c[8], a_c[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const bool on = c < C;
      m_c[c] = on ? ld_cluster_f32(cs + (8 * D + row) * 4, c) : -INFINITY;
      l_c[c] = on ? ld_cluster_f32(cs + (8 * D + 8 + row) * 4, c) : 0.f;
      a_c[c] = on ? ld_cluster_f32(cs + r * 4, c) : 0.f;
    }
    float M = -INFINITY;
#pragma unroll
    for (int c = 0; c < 8; ++c) M = fmaxf(M, m_c[c]);
    const float Mu = M == -INFINITY ? 0.f : M;
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float wgt = fast_exp2(m_c[c] - Mu);
      L = fmaf(l_c[c], wgt, L);
      acc = fmaf(a_c[c], wgt, acc);
    }
    float val = L > 0.f ? acc / L : 0.f;
    const float lse = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
    const long long hq = (long long)head * R + row;
    if constexpr (kExchange) {
      if (!xchg_element<D>(p, xv, (long long)b * p.Hq + hq, col, val, lse, val)) continue;
    }
    if (p.out) p.out[(long long)b * p.o_sb + hq * p.o_sh + col] = __float2bfloat16(val);
    if (p.o_partial) {
      p.o_partial[((long long)b * p.Hq + hq) * D + col] = val;
      if (col == 0) p.lse[(long long)b * p.Hq + hq] = lse;
    }
  }
  cluster_sync();  // no CTA leaves while a peer may still read its shared memory
  if constexpr (kExchange) xchg_end(p, xv);
  }
}

}  // namespace

constexpr size_t kSmallSmemBytes = 1024 + (size_t)kSmWarps * kSmSlots * 8192;  // the merge states reuse the slots

// Opt-in to the shared memory size, once per device and head size.
template <int D>
int configure_instances() {
  const int bytes = (int)kSmallSmemBytes;
  L3CI_CUDA_TRY(cudaFuncSetAttribute(flash_decode_small_kernel<D, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  L3CI_CUDA_TRY(cudaFuncSetAttribute(flash_decode_small_kernel<D, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  L3CI_CUDA_TRY(cudaFuncSetAttribute(flash_decode_small_kernel<D, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  L3CI_CUDA_TRY(cudaFuncSetAttribute(flash_decode_small_kernel<D, true, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  L3CI_CUDA_TRY(cudaFuncSetAttribute(flash_decode_small_kernel<D, false, true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  L3CI_CUDA_TRY(cudaFuncSetAttribute(flash_decode_small_kernel<D, true, true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  L3CI_CUDA_TRY(cudaFuncSetAttribute(flash_decode_small_kernel<D, false, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  L3CI_CUDA_TRY(cudaFuncSetAttribute(flash_decode_small_kernel<D, true, true, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return L3CI_OK;
}
int configure_small_kernel(int D) {
  static bool configured[2][64] = {{false}};
  int dev = 0;
  L3CI_CUDA_TRY(cudaGetDevice(&dev));
  const int di = D == 64 ? 0 : 1;
  if (dev >= 0 && dev < 64 && configured[di][dev]) return L3CI_OK;
  if (int st = D == 64 ? configure_instances<64>() : configure_instances<128>()) return st;
  if (dev >= 0 && dev < 64) configured[di][dev] = true;
  return L3CI_OK;
}

// Clusters of C CTAs of this kernel that the current device runs at once (cached; 0 when the query fails).  The
// SMs of a cluster lie in one GPC, so this is less than SMs / C.
int max_active_clusters(int D, int C) {
  static int cached[2][4][64];  // 0 = not asked yet, else answer + 1
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  const int di = D == 64 ? 0 : 1, ci = C == 2 ? 1 : C == 4 ? 2 : 3;
  if (cached[di][ci][dev]) return cached[di][ci][dev] - 1;
  int n = 0;
  if (configure_small_kernel(D) == L3CI_OK) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(C * 64));
    cfg.blockDim = dim3(32 * kClWarps);
    cfg.dynamicSmemBytes = kSmallSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = D == 64 ? cudaOccupancyMaxActiveClusters(&n, flash_decode_small_kernel<64, true, true, true>, &cfg)
                                  : cudaOccupancyMaxActiveClusters(&n, flash_decode_small_kernel<128, true, true, true>, &cfg);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      n = 0;
    }
  }
  cached[di][ci][dev] = n + 1;
  return n;
}

using UnitSplit = FdStaticSplit;
static_assert(kSmWarps == kFdStaticWarps, "the plan header deals to this kernel's warps");

// The split of fd_static_split with this device's answers for the clusters it holds at once.
UnitSplit unit_split(long long units, long long tiles, int sms, int D) {
  int max_clusters[3] = {0, 0, 0};
  if (units <= sms && tiles >= 32)
    for (int i = 0; i < 3; ++i) max_clusters[i] = max_active_clusters(D, 2 << i);
  return fd_static_split(units, tiles, sms, max_clusters);
}

// True when l3ci_flash_decode hands the call to this kernel (fd_static_applies has the rule and its reasons).
bool flash_decode_small_applies(int B, int Hq, int Hkv, int D, int n_seq, bool ragged) {
  const long long units = (long long)B * Hkv;
  const long long tiles = ((long long)n_seq + fd_tile_tokens(D) - 1) / fd_tile_tokens(D);
  const int sms = sm_count();
  if (sms <= 0 || Hq / Hkv > 8) return false;
  return fd_static_applies(unit_split(units, tiles, sms, D), units, tiles, D, n_seq, Hq / Hkv, ragged);
}

int flash_decode_small_split_code(int B, int Hkv, int D, int n_seq) {
  const long long tiles = ((long long)n_seq + fd_tile_tokens(D) - 1) / fd_tile_tokens(D);
  const UnitSplit s = unit_split((long long)B * Hkv, tiles, sm_count(), D);
  return 16 * s.C + s.W;
}

template <int D, bool kExchange>
int launch_instance(const SmallParams& p, const UnitSplit& s, bool wide, size_t smem, cudaStream_t stream) {
  if (s.C == 1) {  // (the instances without cluster instructions)
    const dim3 grid((unsigned)s.ctas), block(32 * kSmWarps);
    if (s.W == kSmWarps) L3CI_LAUNCH("flash_decode_small_kernel", flash_decode_small_kernel<D, false, true, false, kExchange>, grid, block, smem, stream, p);
    else L3CI_LAUNCH("flash_decode_small_kernel", flash_decode_small_kernel<D, false, false, false, kExchange>, grid, block, smem, stream, p);
    return L3CI_OK;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)s.ctas);
  cfg.blockDim = dim3(32 * (wide ? kClWarps : kSmWarps));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  // (Cluster launches stay plain: with programmatic stream serialization on top of the cluster attribute the
  // 131 072-token call measured 84.7 us against 83.7, a 16 384-token shard 15.41 against 15.29.)
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)s.C;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = wide ? cudaLaunchKernelEx(&cfg, flash_decode_small_kernel<D, true, true, true, kExchange>, p)
                             : cudaLaunchKernelEx(&cfg, flash_decode_small_kernel<D, true, true, false, kExchange>, p);
  if (e != cudaSuccess) return fail(L3CI_ERR_CUDA, "launch of flash_decode_small_kernel failed: %s", cudaGetErrorString(e));
  return L3CI_OK;
}

// split_code: 0 = unit_split's choice, else 16 * C + W (tuning).  `x`: the exchange of a sequence-sharded call.
int flash_decode_small_launch(const l3ci_flash_decode_args* a, int split_code, const FdExchange* x) {
  const long long units = (long long)a->B * a->Hkv;
  const long long tiles = ((long long)a->n_seq + fd_tile_tokens(a->D) - 1) / fd_tile_tokens(a->D);
  if (int st = configure_small_kernel(a->D)) return st;
  UnitSplit s = unit_split(units, tiles, sm_count(), a->D);
  if (split_code > 0) {
    s.C = split_code / 16;
    s.W = split_code % 16;
    const bool pow2 = (s.C & (s.C - 1)) == 0 && (s.W & (s.W - 1)) == 0;
    if (!pow2 || s.C < 1 || s.C > 8 || s.W < 1 || s.W > kSmWarps || (s.C > 1 && s.W != kSmWarps))
      return fail(L3CI_ERR_INVALID, "flash_decode: split code %d (16 * CTAs per unit + warps per unit)", split_code);
    s.ctas = 0;
  }
  if (s.ctas == 0) {  // forced, or more units than one wave holds: several waves
    const int U = kSmWarps / s.W;
    const long long ctas = (units + U - 1) / U * s.C;
    if (ctas > 0x7fffffffLL) return fail(L3CI_ERR_INVALID, "flash_decode: too many units (%lld)", units);
    s.ctas = (int)ctas;
  }
  SmallParams p;
  p.lgW = s.W == 8 ? 3 : s.W == 4 ? 2 : s.W == 2 ? 1 : 0;
  p.lgC = s.C == 8 ? 3 : s.C == 4 ? 2 : s.C == 2 ? 1 : 0;
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.k = static_cast<const __nv_bfloat16*>(a->k);
  p.v = static_cast<const __nv_bfloat16*>(a->v);
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.o_partial = a->o_partial;
  p.lse = a->lse;
  p.seq_lens = a->seq_lens;
  p.B = a->B; p.Hq = a->Hq; p.Hkv = a->Hkv; p.R = a->Hq / a->Hkv; p.n_seq = a->n_seq;
  p.q_sb = a->q_sb; p.q_sh = a->q_sh; p.k_sb = a->k_sb; p.k_sh = a->k_sh; p.k_st = a->k_st;
  p.v_sb = a->v_sb; p.v_sh = a->v_sh; p.v_st = a->v_st; p.o_sb = a->o_sb; p.o_sh = a->o_sh;
  const float scale = a->scale > 0.f ? a->scale : 1.0f / sqrtf((float)a->D);
  p.scale_log2e = scale * 1.4426950408889634f;
  p.xbufs = nullptr; p.xrank = 0; p.xranks = 1; p.xepoch = 0; p.xstatus = nullptr; p.xwait_ns = 0;
  if (x) {
    if (x->ranks < 1 || x->ranks > kXchgMaxRanks || x->rank < 0 || x->rank >= x->ranks || !x->bufs)
      return fail(L3CI_ERR_UNSUPPORTED, "flash_decode_exchange: %d ranks (1..%d are supported), rank %d", x->ranks, kXchgMaxRanks, x->rank);
    p.xbufs = reinterpret_cast<unsigned long long* const*>(x->bufs);
    p.xrank = x->rank; p.xranks = x->ranks; p.xepoch = x->epoch; p.xstatus = x->status;
    p.xwait_ns = device_wait_limit_ns(1000000000ull);
  }
  const size_t smem = kSmallSmemBytes;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(a->stream);
  const bool wide = fd_static_wide(s, tiles);
  if (a->D == 64) return x ? launch_instance<64, true>(p, s, wide, smem, stream) : launch_instance<64, false>(p, s, wide, smem, stream);
  return x ? launch_instance<128, true>(p, s, wide, smem, stream) : launch_instance<128, false>(p, s, wide, smem, stream);
}

}  // namespace l3ci
