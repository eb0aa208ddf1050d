// Causal GQA attention for T > 1 new tokens per sequence (prefill) on sm_100a.
//
// The reference sends this case to PyTorch (model.py:114-116: F.scaled_dot_product_attention(q, k, v,
// is_causal=True, enable_gqa=True) over the cache rows [0, T)); this is the same computation over the layout the
// model has (q [B,Hq,T,D] view of [B,T,Hq,D]; k, v [B,Hkv,S,D] views of the cache), generalised to a chunk that
// starts at `start_pos`: query t sees keys j <= start_pos + t, j < n_keys.
//
// One CTA = 64 query rows of one query head: four consumer warps of 16 rows each and one producer warp.  Keys and
// values arrive 64 at a time through a 2-stage ring of bulk tensor copies (the rank-4 map of the decode kernel
// with one head per box, 128-byte swizzle); S = Q K^T and O += P V run on mma.sync.m16n8k16 with Q in registers,
// P taken straight from the score accumulators, online softmax in the log2 domain.  The query heads that share a
// KV head run in neighbouring CTAs and meet its tiles in L2.  Query blocks are handed out last block first, so the
// CTAs with the most keys start first.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include "bf16x8.cuh"
#include "host_common.h"
#include "ptx_sm100.cuh"
#include "tensor_map.h"
#include "warp_reduce.cuh"

namespace l3ci {
// prefill_attention_tc.cu: the tcgen05 kernel; -1 when it cannot take the call (Q rows not 16-byte aligned)
int launch_prefill_tc(const l3ci_prefill_args* a);

namespace {

constexpr int kPfRows = 64;     // query rows per CTA
constexpr int kPfKeys = 64;     // keys per tile
constexpr int kPfStages = 2;
constexpr int kPfConsumers = 4;

struct PfParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  int B, Hq, Hkv, R, T, n_keys, start_pos, m_blocks;
  long long q_sb, q_sh, q_st, o_sb, o_sh, o_st;
  float scale_log2e;
  int* status;  // may be null
};

template <int D>
__global__ void __launch_bounds__(32 * (kPfConsumers + 1))
prefill_attention_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                         const PfParams p) {
  constexpr int kHalves = D / 64;                  // 128-byte column blocks per row
  constexpr int kBoxBytes = kPfKeys * 128;         // one box: 64 keys x 128 bytes
  constexpr int kTileBytes = kHalves * kBoxBytes;  // K (or V) tile
  constexpr int kStageBytes = 2 * kTileBytes;
  constexpr int KS = D / 16;                       // k-steps of Q K^T
  constexpr int NT_S = kPfKeys / 8;                // 8-key score tiles
  constexpr int NT_O = D / 8;                      // 8-column output tiles
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPfStages * kStageBytes);  // full[], empty[]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < kPfStages; ++s) {
      mbar_init(smem_u32(&bars[s]), 1);
      mbar_init(smem_u32(&bars[kPfStages + s]), kPfConsumers);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&kmap)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&vmap)) : "memory");
  }
  __syncthreads();

  // work item: query block (last first), then query head, then sequence
  // longest query blocks first over the whole launch: CTAs are handed out in this order as SMs come free
  const int heads_all = p.Hq * p.B;
  const int mb = p.m_blocks - 1 - (int)(blockIdx.x / heads_all);
  const int hq = (int)(blockIdx.x % heads_all) % p.Hq;
  const int b = (int)(blockIdx.x % heads_all) / p.Hq;
  const int hkv = hq / p.R;
  const int m0 = mb * kPfRows;
  // keys this block can see: j <= start_pos + (last row of the block), j < n_keys
  const int last_row = min(m0 + kPfRows, p.T) - 1;
  const int keys = min(p.n_keys, p.start_pos + last_row + 1);
  const int n_tiles = (keys + kPfKeys - 1) / kPfKeys;

  const uint32_t stage0 = smem_u32(smem);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = full0 + kPfStages * 8;

  if (warp == kPfConsumers) {
    // ---- producer warp ----
    const uint64_t policy = l2_evict_first_policy();
    bool alive = true;
    int k = 0;
    for (; k < n_tiles; ++k) {
      const int stage = k % kPfStages;
      if (k >= kPfStages && !mbar_wait_bounded(empty0 + stage * 8, ((k / kPfStages) - 1) & 1)) { alive = false; break; }
      if (lane == 0) {
        const uint32_t bar = full0 + stage * 8, dst = stage0 + stage * kStageBytes;
        mbar_expect_tx(bar, kStageBytes);
#pragma unroll
        for (int h = 0; h < kHalves; ++h) tma_load_4d(dst + h * kBoxBytes, &kmap, bar, h * 64, k * kPfKeys, hkv, b, policy);
#pragma unroll
        for (int h = 0; h < kHalves; ++h)
          tma_load_4d(dst + kTileBytes + h * kBoxBytes, &vmap, bar, h * 64, k * kPfKeys, hkv, b, policy);
      }
      __syncwarp();
    }
    // stay until the consumers have released the last tiles: no copy may be in flight when the CTA ends
    for (int j = max(k - kPfStages, 0); alive && j < k; ++j)
      alive = mbar_wait_bounded(empty0 + (j % kPfStages) * 8, (j / kPfStages) & 1);
    if (!alive && lane == 0 && p.status) atomicExch(p.status, (int)L3CI_ERR_DEVICE_WAIT);
    return;
  }

  // ---- consumer warps: rows m0 + 16 * warp + {gid, gid + 8} ----
  const int row_lo = m0 + warp * 16 + gid, row_hi = row_lo + 8;
  const __nv_bfloat16* qp = p.q + (long long)b * p.q_sb + (long long)hq * p.q_sh;
  uint32_t qa[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const int col = ks * 16 + 2 * tig;
    qa[ks][0] = row_lo < p.T ? ld_global_u32(qp + row_lo * p.q_st + col) : 0u;
    qa[ks][1] = row_hi < p.T ? ld_global_u32(qp + row_hi * p.q_st + col) : 0u;
    qa[ks][2] = row_lo < p.T ? ld_global_u32(qp + row_lo * p.q_st + col + 8) : 0u;
    qa[ks][3] = row_hi < p.T ? ld_global_u32(qp + row_hi * p.q_st + col + 8) : 0u;
  }
  const int mat = lane >> 3, r8 = lane & 7;
  // K as B operand: matrices (key 0-7, chunk c), (key 0-7, c+1), (key 8-15, c), (key 8-15, c+1)
  const uint32_t k_row_off = (r8 + 8 * (mat >> 1)) * 128, k_x = (mat & 1) ^ r8;
  // V, transposed, as B operand: matrices (key 0-7, chunk c), (key 8-15, c), (key 0-7, c+1), (key 8-15, c+1)
  const uint32_t v_row_off = (r8 + 8 * (mat & 1)) * 128, v_x = (mat >> 1) ^ r8;

  float o[NT_O][4];
#pragma unroll
  for (int nt = 0; nt < NT_O; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  // last key each of this thread's rows may see
  const int lim_lo = p.start_pos + row_lo, lim_hi = p.start_pos + row_hi;
  bool ok = true;

  for (int k = 0; k < n_tiles; ++k) {
    const int stage = k % kPfStages;
    if (!mbar_wait_bounded(full0 + stage * 8, (k / kPfStages) & 1)) { ok = false; break; }
    const uint32_t kb = stage0 + stage * kStageBytes, vb = kb + kTileBytes;

    // ---- S = Q K^T (16 rows x 64 keys per warp) ----
    float s[NT_S][4];
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int ntp = 0; ntp < NT_S / 2; ++ntp) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kb + (ks >> 2) * kBoxBytes + ntp * 2048 + k_row_off + (((2u * (ks & 3)) ^ k_x) << 4), b0, b1, b2, b3);
        mma_bf16(s[2 * ntp], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
        mma_bf16(s[2 * ntp + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
      }
    }

    // ---- causal mask (only tiles that reach past the first row's limit) and the end of the cache ----
    const int j0 = k * kPfKeys;
    if (j0 + kPfKeys - 1 > p.start_pos + m0 + warp * 16 || j0 + kPfKeys > p.n_keys) {
#pragma unroll
      for (int nt = 0; nt < NT_S; ++nt) {
        const int j = j0 + nt * 8 + 2 * tig;
        if (j > lim_lo || j >= p.n_keys) s[nt][0] = -INFINITY;
        if (j + 1 > lim_lo || j + 1 >= p.n_keys) s[nt][1] = -INFINITY;
        if (j > lim_hi || j >= p.n_keys) s[nt][2] = -INFINITY;
        if (j + 1 > lim_hi || j + 1 >= p.n_keys) s[nt][3] = -INFINITY;
      }
    }

    // ---- online softmax, log2 domain ----
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt) {
      mx_lo = fmaxf(mx_lo, fmaxf(s[nt][0], s[nt][1]));
      mx_hi = fmaxf(mx_hi, fmaxf(s[nt][2], s[nt][3]));
    }
    mx_lo = group_max<4>(mx_lo) * p.scale_log2e;
    mx_hi = group_max<4>(mx_hi) * p.scale_log2e;
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    const float mu_lo = mn_lo == -INFINITY ? 0.f : mn_lo, mu_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
    const float al_lo = fast_exp2(m_lo - mu_lo), al_hi = fast_exp2(m_hi - mu_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;
    float ps_lo = 0.f, ps_hi = 0.f;
    uint32_t pa[NT_S / 2][4];
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt) {
      const float p0 = fast_exp2(fmaf(s[nt][0], p.scale_log2e, -mu_lo));
      const float p1 = fast_exp2(fmaf(s[nt][1], p.scale_log2e, -mu_lo));
      const float p2 = fast_exp2(fmaf(s[nt][2], p.scale_log2e, -mu_hi));
      const float p3 = fast_exp2(fmaf(s[nt][3], p.scale_log2e, -mu_hi));
      ps_lo += p0 + p1;
      ps_hi += p2 + p3;
      pa[nt >> 1][(nt & 1) * 2] = pack_bf16x2(p0, p1);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(p2, p3);
    }
    l_lo = fmaf(l_lo, al_lo, ps_lo);
    l_hi = fmaf(l_hi, al_hi, ps_hi);
    if (__any_sync(kFullMask, al_lo != 1.f || al_hi != 1.f)) {
#pragma unroll
      for (int nt = 0; nt < NT_O; ++nt) {
        o[nt][0] *= al_lo; o[nt][1] *= al_lo;
        o[nt][2] *= al_hi; o[nt][3] *= al_hi;
      }
    }

    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < NT_S / 2; ++kk) {
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(vb + (np >> 2) * kBoxBytes + kk * 2048 + v_row_off + (((2u * (np & 3)) ^ v_x) << 4), b0, b1, b2, b3);
        mma_bf16(o[2 * np], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
        mma_bf16(o[2 * np + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + stage * 8);
  }
  if (!ok) {
    if (lane == 0 && p.status) atomicExch(p.status, (int)L3CI_ERR_DEVICE_WAIT);
    return;
  }

  // ---- normalise and write ----
  l_lo = group_sum<4>(l_lo);
  l_hi = group_sum<4>(l_hi);
  const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
  __nv_bfloat16* ob = p.out + (long long)b * p.o_sb + (long long)hq * p.o_sh;
#pragma unroll
  for (int nt = 0; nt < NT_O; ++nt) {
    const int d = nt * 8 + 2 * tig;
    if (row_lo < p.T) *reinterpret_cast<uint32_t*>(ob + row_lo * p.o_st + d) = pack_bf16x2(o[nt][0] * inv_lo, o[nt][1] * inv_lo);
    if (row_hi < p.T) *reinterpret_cast<uint32_t*>(ob + row_hi * p.o_st + d) = pack_bf16x2(o[nt][2] * inv_hi, o[nt][3] * inv_hi);
  }
}

template <int D>
int launch_prefill(const CUtensorMap& kmap, const CUtensorMap& vmap, const PfParams& p, cudaStream_t stream) {
  constexpr size_t smem = 1024 + (size_t)kPfStages * 2 * (D / 64) * kPfKeys * 128 + 2 * kPfStages * 8;
  static bool configured[64] = {false};
  int dev = 0;
  L3CI_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    L3CI_CUDA_TRY(cudaFuncSetAttribute(prefill_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const long long ctas = (long long)p.B * p.Hq * p.m_blocks;
  if (ctas > 0x7fffffffLL) return fail(L3CI_ERR_INVALID, "prefill_attention: too many query blocks (%lld)", ctas);
  prefill_attention_kernel<D><<<(unsigned)ctas, 32 * (kPfConsumers + 1), smem, stream>>>(kmap, vmap, p);
  L3CI_CHECK_LAUNCH("prefill_attention_kernel");
  return L3CI_OK;
}

}  // namespace
}  // namespace l3ci

extern "C" int l3ci_prefill_attention(const l3ci_prefill_args* a) {
  using namespace l3ci;
  clear_error();
  if (!a) return fail(L3CI_ERR_INVALID, "prefill_attention: null args");
  const int B = a->B, Hq = a->Hq, Hkv = a->Hkv, D = a->D, T = a->T, S = a->n_keys;
  if (B < 0 || Hq <= 0 || Hkv <= 0 || T < 0 || S < 0 || a->start_pos < 0)
    return fail(L3CI_ERR_INVALID, "prefill_attention: bad size B=%d Hq=%d Hkv=%d T=%d n_keys=%d start_pos=%d", B, Hq, Hkv, T, S, a->start_pos);
  if (Hq % Hkv) return fail(L3CI_ERR_INVALID, "prefill_attention: %d query heads not divisible by %d kv heads", Hq, Hkv);
  if (D != 64 && D != 128) return fail(L3CI_ERR_UNSUPPORTED, "Unsupported head size for prefill_attention kernel: %d", D);
  if (B == 0 || T == 0) return L3CI_OK;
  if (S == 0) return fail(L3CI_ERR_INVALID, "prefill_attention: no keys");
  if (!a->q || !a->k || !a->v || !a->out) return fail(L3CI_ERR_INVALID, "prefill_attention: null pointer");
  if ((reinterpret_cast<uintptr_t>(a->q) & 3) || (a->q_sb & 1) || (a->q_sh & 1) || (a->q_st & 1) ||
      (reinterpret_cast<uintptr_t>(a->out) & 3) || (a->o_sb & 1) || (a->o_sh & 1) || (a->o_st & 1))
    return fail(L3CI_ERR_ALIGNMENT, "prefill_attention: q/out rows must start on 4 bytes");
  if (!aligned16(a->k) || !aligned16(a->v) || (S > 1 && (a->k_st % 8 || a->v_st % 8)) ||
      (Hkv > 1 && (a->k_sh % 8 || a->v_sh % 8)) || (B > 1 && (a->k_sb % 8 || a->v_sb % 8)))
    return fail(L3CI_ERR_ALIGNMENT, "prefill_attention: k/v rows must start on 16 bytes and strides be multiples of 8 elements");
  if ((S > 1 && (a->k_st <= 0 || a->v_st <= 0)) || (Hkv > 1 && (a->k_sh <= 0 || a->v_sh <= 0)) ||
      (B > 1 && (a->k_sb <= 0 || a->v_sb <= 0)))
    return fail(L3CI_ERR_INVALID, "prefill_attention: k/v strides must be positive");
  if (a->variant < 0 || a->variant > 2) return fail(L3CI_ERR_INVALID, "prefill_attention: variant %d", a->variant);
  // By measurement (B=4, Hq=32, T=2048): the tcgen05 kernel wins at both head sizes (948 vs 321 TFLOP/s at 128,
  // 540 vs 278 at 64); prompts shorter than its block of 128 query rows, and q or out layouts the copy engine or
  // 16-byte stores cannot take, go to the mma.sync kernel.
  if (a->variant == 1 || (a->variant == 0 && T >= 128)) {
    const int st = launch_prefill_tc(a);
    if (st != -1) return st;
    if (a->variant == 1) return fail(L3CI_ERR_ALIGNMENT, "prefill_attention: the tcgen05 kernel needs 16-byte aligned q and out rows");
  }
  CUtensorMap kmap, vmap;
  if (int st = make_kv_map(&kmap, a->k, D, S, Hkv, B, a->k_st, a->k_sh, a->k_sb, kPfKeys, 1)) return st;
  if (int st = make_kv_map(&vmap, a->v, D, S, Hkv, B, a->v_st, a->v_sh, a->v_sb, kPfKeys, 1)) return st;
  PfParams p;
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.R = Hq / Hkv; p.T = T; p.n_keys = S; p.start_pos = a->start_pos;
  p.m_blocks = (T + kPfRows - 1) / kPfRows;
  p.q_sb = a->q_sb; p.q_sh = a->q_sh; p.q_st = a->q_st; p.o_sb = a->o_sb; p.o_sh = a->o_sh; p.o_st = a->o_st;
  const float scale = a->scale > 0.f ? a->scale : 1.0f / sqrtf((float)D);
  p.scale_log2e = scale * 1.4426950408889634f;
  p.status = a->status;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(a->stream);
  return D == 64 ? launch_prefill<64>(kmap, vmap, p, stream) : launch_prefill<128>(kmap, vmap, p, stream);
}
