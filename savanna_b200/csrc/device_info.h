// Host-side device queries shared by the launchers.
#pragma once
#include <cuda_runtime.h>

namespace sb {

// Number of SMs of the current device, queried once per device.  Launch geometry (persistent grids, "a few waves"
// caps) is sized from this value, never from a literal.
static inline int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace sb
