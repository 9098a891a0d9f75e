// Per-device facts the launch planners need, looked up once per device under a lock.
#include <mutex>

#include "kernels.h"

namespace qb {

std::mutex& setup_mutex() {
  static std::mutex mu;
  return mu;
}

// Streaming multiprocessors of the current device (148 on B200).  A failed query (no device, as in a
// host-only check of the library) answers 148 so that size queries stay deterministic.
int sm_count() {
  static std::mutex mu;
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); return 148; }
  if (dev < 0 || dev >= 64) dev = 0;
  std::lock_guard<std::mutex> lk(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      return 148;
    }
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace qb
