#include "host_common.h"

#include <stdarg.h>
#include <stdio.h>

#include <atomic>

namespace l3ci {

namespace {
thread_local char g_err[512] = {0};
constexpr int kMaxDev = 64;
int g_sms[kMaxDev] = {0};
int g_smem[kMaxDev] = {0};
std::atomic<unsigned long long> g_wait_limit_ns{0};  // 0: every kernel's own default
std::atomic<int> g_programmatic_launch{1};
}  // namespace

bool programmatic_launch_enabled() { return g_programmatic_launch.load(std::memory_order_relaxed) != 0; }

unsigned long long device_wait_limit_ns(unsigned long long default_ns) {
  const unsigned long long v = g_wait_limit_ns.load(std::memory_order_relaxed);
  return v ? v : default_ns;
}

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}

void clear_error() { g_err[0] = 0; }

static int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  return dev;
}

int sm_count() {
  const int dev = current_device();
  if (dev < 0) return 0;
  if (dev < kMaxDev && g_sms[dev]) return g_sms[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  if (dev < kMaxDev) g_sms[dev] = n;
  return n;
}

int max_smem_optin() {
  const int dev = current_device();
  if (dev < 0) return 0;
  if (dev < kMaxDev && g_smem[dev]) return g_smem[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 0;
  if (dev < kMaxDev) g_smem[dev] = n;
  return n;
}

}  // namespace l3ci

extern "C" {

const char* l3ci_status_string(int status) {
  switch (status) {
    case L3CI_OK: return "ok";
    case L3CI_ERR_INVALID: return "invalid argument";
    case L3CI_ERR_UNSUPPORTED: return "unsupported head size or query/kv head ratio";
    case L3CI_ERR_ALIGNMENT: return "rows must start on 16 bytes and strides be multiples of 8 elements";
    case L3CI_ERR_SCRATCH: return "scratch buffer too small";
    case L3CI_ERR_CUDA: return "CUDA call failed";
    case L3CI_ERR_DEVICE_WAIT: return "a bounded device-side wait ran out";
    default: return "unknown status";
  }
}

const char* l3ci_last_error(void) { return l3ci::g_err; }

const char* l3ci_version(void) { return "0.2.0"; }

int l3ci_set_programmatic_launch(int on) { return l3ci::g_programmatic_launch.exchange(on ? 1 : 0, std::memory_order_relaxed); }

uint64_t l3ci_set_device_wait_limit_ns(uint64_t ns) {
  return l3ci::g_wait_limit_ns.exchange(ns, std::memory_order_relaxed);
}

}  // extern "C"
