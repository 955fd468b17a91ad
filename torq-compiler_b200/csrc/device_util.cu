// Per-device facts the launchers need: SM count, "has this device seen this one-time set-up",
// and the limit of the kernels' bounded waits. One process may hold several devices through the
// C ABI, and function attributes (cudaFuncSetAttribute) are per device, so nothing here is a
// process-wide flag.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>

#include "kernels.h"

namespace tb200 {

namespace {
constexpr int kMaxDevices = 64;
}

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  return dev;
}

int current_sm_count() {
  static std::atomic<int> cache[kMaxDevices];
  const int dev = current_device();
  int n = cache[dev].load(std::memory_order_relaxed);
  if (n <= 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

bool first_use_on_device(std::atomic<unsigned long long>& done) {
  const unsigned long long bit = 1ull << current_device();
  return (done.load(std::memory_order_acquire) & bit) == 0;
}

void mark_used_on_device(std::atomic<unsigned long long>& done) {
  done.fetch_or(1ull << current_device(), std::memory_order_release);
}

unsigned long long wait_limit_ns() {
  // read on every call: a test changes it between executables
  const char* e = getenv("TB200_WAIT_LIMIT_MS");
  long ms = e && *e ? atol(e) : 2000;
  if (ms < 1) ms = 1;
  if (ms > 60000) ms = 60000;
  return (unsigned long long)ms * 1000000ull;
}

}  // namespace tb200
