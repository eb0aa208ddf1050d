// Host-side construction of the tensor maps the attention kernels copy K/V tiles with.
#pragma once

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

#include <mutex>

#include "host_common.h"

namespace l3ci {

inline PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(f);
  });
  return fn;
}

// Rank-4 map over a [B, Hkv, n_seq, D] view: dims (d, token, head, batch), box 64 x tile tokens x HG heads.
inline int make_kv_map(CUtensorMap* map, const void* base, int D, int n_seq, int Hkv, int B, long long st,
                long long sh, long long sb, int tile, int HG) {
  auto enc = tensor_map_encoder();
  if (!enc) return fail(L3CI_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  const cuuint64_t row_bytes = (cuuint64_t)D * 2;
  // A dimension of extent 1 may carry any stride in the caller's view; give it a valid one.
  const cuuint64_t st_b = n_seq > 1 ? (cuuint64_t)st * 2 : row_bytes;
  const cuuint64_t sh_b = Hkv > 1 ? (cuuint64_t)sh * 2 : row_bytes;
  const cuuint64_t sb_b = B > 1 ? (cuuint64_t)sb * 2 : row_bytes;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)n_seq, (cuuint64_t)Hkv, (cuuint64_t)B};
  cuuint64_t strides[3] = {st_b, sh_b, sb_b};
  cuuint32_t box[4] = {64u, (cuuint32_t)tile, (cuuint32_t)HG, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box,
                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         D == 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(L3CI_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return L3CI_OK;
}


}  // namespace l3ci
