// Decode attention for small problems: one CTA per (sequence, KV head), the cached tokens dealt to its eight
// warps, partial results merged through shared memory.
//
// The persistent kernel of flash_decode.cu pays fixed latencies per launch (tensor-map fetch, cross-CTA merge
// through global memory) of 7-8 us, which is all there is to a call like the reference's own example (one
// sequence of 256 tokens, benchmark_kernel.py:160-163: 0.5 MB of K and V).  Here nothing crosses a CTA: K and V
// rows go from global to shared memory with 16-byte asynchronous copies (written in the 128-byte-swizzled layout
// that ldmatrix expects), the tile arithmetic is the one of the large kernel (S^T = K Q^T and O^T = V^T P^T on
// mma.sync.m16n8k16, tokens on the rows of a tile, the group's query heads on its 8 columns), and the eight
// (m, l, o) states of a CTA meet in shared memory.  Taken by l3ci_flash_decode for short caches with at most 8
// query heads per KV head; results are the same within rounding.
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

struct SmallParams {
  const __nv_bfloat16 *q, *k, *v;
  __nv_bfloat16* out;
  float* o_partial;
  float* lse;
  const int* seq_lens;
  int B, Hq, Hkv, R, n_seq;
  long long q_sb, q_sh, k_sb, k_sh, k_st, v_sb, v_sh, v_st, o_sb, o_sh;
  float scale_log2e;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int D>
__global__ void __launch_bounds__(32 * kSmWarps)
flash_decode_small_kernel(const SmallParams p) {
  constexpr int kTile = fd_tile_tokens(D);   // tokens per tile: 4 KB of K and 4 KB of V
  constexpr int kHalves = D / 64;
  constexpr int kBoxBytes = kTile * 128;     // one 64-column half of a tile
  constexpr int kTileBytes = 2 * kHalves * kBoxBytes;  // K then V
  constexpr int KS = D / 16, MB = kTile / 16, MT = D / 16;
  constexpr int kStateFloats = 8 * D + 16;   // o[8 rows][D], m[8], l[8]
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* states = reinterpret_cast<float*>(smem);  // [kSmWarps][kStateFloats], over the tile slots once all warps are done
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int b = blockIdx.x / p.Hkv, head = blockIdx.x % p.Hkv;
  const int R = p.R;
  const int len = p.seq_lens ? min(max(__ldg(p.seq_lens + b), 0), p.n_seq) : p.n_seq;

  // this warp's tiles: tiles are dealt in contiguous runs
  const int n_tiles = (len + kTile - 1) / kTile;
  const int t_begin = (int)((long long)warp * n_tiles / kSmWarps), t_end = (int)((long long)(warp + 1) * n_tiles / kSmWarps);
  const __nv_bfloat16* kbase = p.k + (long long)b * p.k_sb + (long long)head * p.k_sh;
  const __nv_bfloat16* vbase = p.v + (long long)b * p.v_sb + (long long)head * p.v_sh;
  const uint32_t buf0 = smem_u32(smem) + warp * kSmSlots * kTileBytes;

  // copy of one tile: 16-byte chunk c (0..7) of 128-byte row r of half h goes to chunk position c ^ (r & 7)
  // (always one commit group per call, empty past the warp's last tile, so that "all but the newest
  // kSmSlots - 1 groups" is the tile about to be used)
  auto fetch = [&](int tile, int slot) {
    const uint32_t dst = buf0 + slot * kTileBytes;
    constexpr int kChunks = kHalves * kTile * 8;  // per tensor
#pragma unroll
    for (int i = lane; i < (tile < t_end ? kChunks : 0); i += 32) {
      const int c = i & 7, r = (i >> 3) % kTile, h = i / (8 * kTile);
      const int tok = tile * kTile + r;
      const bool ok = tok < len;
      const long long off = (long long)(ok ? tok : 0);
      const uint32_t d = h * kBoxBytes + r * 128 + ((c ^ (r & 7)) << 4);
      cp_async16(dst + d, kbase + off * p.k_st + h * 64 + c * 8, ok);
      cp_async16(dst + kHalves * kBoxBytes + d, vbase + off * p.v_st + h * 64 + c * 8, ok);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int i = 0; i < kSmSlots; ++i) fetch(t_begin + i, i);

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
    const int slot = (t - t_begin) % kSmSlots;
    cp_async_wait<kSmSlots - 1>();
    __syncwarp();
    const uint32_t kb = buf0 + slot * kTileBytes, vb = kb + kHalves * kBoxBytes;
    // S^T = K Q^T
    float s[MB][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) s[mb][0] = s[mb][1] = s[mb][2] = s[mb][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        uint32_t a0, a1, a2, a3;
        ldsm_x4(kb + (ks >> 2) * kBoxBytes + mb * 2048 + k_row_off + (((2u * (ks & 3)) ^ k_x) << 4), a0, a1, a2, a3);
        mma_bf16(s[mb], a0, a1, a2, a3, qb[ks][0], qb[ks][1]);
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
    fetch(t + kSmSlots, slot);
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

  // ---- merge of the eight states: one thread per output element ----
  for (int e = threadIdx.x; e < R * D; e += 32 * kSmWarps) {
    const int row = e / D, col = e - row * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kSmWarps; ++w) M = fmaxf(M, states[w * kStateFloats + 8 * D + row]);
    const float Mu = M == -INFINITY ? 0.f : M;
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kSmWarps; ++w) {
      const float wgt = fast_exp2(states[w * kStateFloats + 8 * D + row] - Mu);
      L = fmaf(states[w * kStateFloats + 8 * D + 8 + row], wgt, L);
      acc = fmaf(states[w * kStateFloats + row * D + col], wgt, acc);
    }
    const float val = L > 0.f ? acc / L : 0.f;
    const long long hq = (long long)head * R + row;
    if (p.out) p.out[(long long)b * p.o_sb + hq * p.o_sh + col] = __float2bfloat16(val);
    if (p.o_partial) {
      p.o_partial[((long long)b * p.Hq + hq) * D + col] = val;
      if (col == 0) p.lse[(long long)b * p.Hq + hq] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
    }
  }
}

}  // namespace

// True when the call is one for the small kernel (decided from host-side sizes only).
bool flash_decode_small_applies(int B, int Hq, int Hkv, int D, int n_seq) {
  const int R = Hq / Hkv;
  const long long tiles = (long long)(n_seq + fd_tile_tokens(D) - 1) / fd_tile_tokens(D);
  return R <= 8 && tiles <= 4 * kSmWarps && (long long)B * Hkv <= 32 && (long long)B * Hkv * tiles <= 512;
}

int flash_decode_small_launch(const l3ci_flash_decode_args* a) {
  SmallParams p;
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
  const size_t smem = 1024 + (size_t)kSmWarps * kSmSlots * 8192;  // the merge states (33 KB at most) reuse the slots
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(a->stream);
  static bool configured[2][64] = {{false}};
  int dev = 0;
  L3CI_CUDA_TRY(cudaGetDevice(&dev));
  const int di = a->D == 64 ? 0 : 1;
  if (dev < 0 || dev >= 64 || !configured[di][dev]) {
    if (a->D == 64) L3CI_CUDA_TRY(cudaFuncSetAttribute(flash_decode_small_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    else L3CI_CUDA_TRY(cudaFuncSetAttribute(flash_decode_small_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev >= 0 && dev < 64) configured[di][dev] = true;
  }
  const unsigned grid = (unsigned)(a->B * a->Hkv);
  if (a->D == 64) flash_decode_small_kernel<64><<<grid, 32 * kSmWarps, smem, stream>>>(p);
  else flash_decode_small_kernel<128><<<grid, 32 * kSmWarps, smem, stream>>>(p);
  L3CI_CHECK_LAUNCH("flash_decode_small_kernel");
  return L3CI_OK;
}

}  // namespace l3ci
