// Host-side helpers shared by the launchers: thread-local error text, launch checks,
// cached device properties.  Unlike the reference, whose cudaCheck is never called
// (custom_kernels/custom_kernels.cu:224-231), every launcher checks its arguments and the
// launch result and reports through the status code it returns.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/l3ci_b200.h"

namespace l3ci {

// Stores a printf-formatted message for l3ci_last_error() and returns `status`.
int fail(int status, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();

// Number of SMs of the current device (cached per device).
int sm_count();
// Largest opt-in dynamic shared memory per block of the current device (cached).
int max_smem_optin();

// Decode attention with units dealt statically to warps, CTAs or clusters (flash_decode_small.cu): whether
// l3ci_flash_decode hands a call of these sizes to it, and its launch (arguments already validated by the
// caller; split_code 0 = its own choice, else 16 * CTAs per unit + warps per unit).
// `FdExchange` (optional): the cross-GPU exchange of a sequence-sharded call, done in the kernel's tail.
struct FdExchange {
  void* const* bufs;
  int rank, ranks;
  unsigned epoch;
  int* status;
};
bool flash_decode_small_applies(int B, int Hq, int Hkv, int D, int n_seq, bool ragged);
int flash_decode_small_launch(const l3ci_flash_decode_args* a, int split_code, const FdExchange* x = nullptr);
// 16 * C + W of the split the static kernel would take for these sizes on the current device.
int flash_decode_small_split_code(int B, int Hkv, int D, int n_seq);

// Bound, in nanoseconds, of a device-side wait on other CTAs or other GPUs: the value set through
// l3ci_set_device_wait_limit_ns, else `default_ns`.
unsigned long long device_wait_limit_ns(unsigned long long default_ns);

// Programmatic dependent launch (l3ci_set_programmatic_launch): whether kernels are launched so that their grid may
// be set up while the previous kernel of the stream is still draining.
bool programmatic_launch_enabled();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define L3CI_CUDA_TRY(expr)                                                              \
  do {                                                                                   \
    cudaError_t e_ = (expr);                                                             \
    if (e_ != cudaSuccess)                                                               \
      return ::l3ci::fail(L3CI_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

// After a <<<>>> launch: picks up configuration errors without synchronising.
#define L3CI_CHECK_LAUNCH(name)                                                            \
  do {                                                                                     \
    cudaError_t e_ = cudaGetLastError();                                                   \
    if (e_ != cudaSuccess)                                                                 \
      return ::l3ci::fail(L3CI_ERR_CUDA, "launch of %s failed: %s", name,                  \
                          cudaGetErrorString(e_));                                         \
  } while (0)

#if defined(__CUDACC__)
// Launch of `kernel`, as <<<grid, block, smem, stream>>> would do it, or, when programmatic dependent launch is on,
// with the attribute that lets the grid be scheduled before the previous kernel of the stream has finished.  Kernels
// launched this way call pdl_wait() (ptx_sm100.cuh) before they touch global memory: it returns once the previous
// kernel has completed and its writes are visible, so the overlap is the launch itself, the CTAs' start and whatever
// a kernel does before its first global access; a kernel launched the plain way passes through it at once.
template <typename... Params, typename... Args>
cudaError_t launch_kernel(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = programmatic_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}
#define L3CI_LAUNCH(name, ...)                                                                     \
  do {                                                                                             \
    cudaError_t e_ = ::l3ci::launch_kernel(__VA_ARGS__);                                           \
    if (e_ != cudaSuccess)                                                                         \
      return ::l3ci::fail(L3CI_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e_)); \
  } while (0)
#endif

}  // namespace l3ci
