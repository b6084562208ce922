// Host-side helper: one-time set-up per DEVICE.
//
// cudaFuncSetAttribute (opt-in to more than 48 KiB of dynamic shared memory) belongs to the current device's
// context, so a process that calls the library on cuda:0 and later on cuda:1 has to set it on each.  A
// DeviceOnce keeps one flag per device ordinal under a mutex; `run` calls the set-up function the first time it
// sees the current device and afterwards returns that device's cached result.  The first use on a device also
// checks that it is an sm_100 part (compute capability 10.x): the kernels are built for sm_100a only.
#pragma once

#include <cuda_runtime.h>

#include <mutex>

#include "kda_b200.h"

namespace kda {

constexpr int kMaxDeviceOrdinals = 64;

struct DeviceOnce {
  std::mutex mu;
  bool done[kMaxDeviceOrdinals] = {};
  int result[kMaxDeviceOrdinals] = {};

  // Returns KDA_OK, KDA_E_DEVICE (not an sm_100 device), KDA_E_LIMIT (device ordinal beyond the table) or a
  // positive cudaError_t.  `setup` returns a cudaError_t and runs with the device current.
  template <class F>
  int run(F&& setup) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDeviceOrdinals) return KDA_E_LIMIT;
    std::lock_guard<std::mutex> lk(mu);
    if (!done[dev]) {
      int major = 0;
      e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
      if (e != cudaSuccess) return static_cast<int>(e);
      if (major != 10) {
        result[dev] = KDA_E_DEVICE;
      } else {
        e = setup();
        result[dev] = static_cast<int>(e);
      }
      done[dev] = true;
    }
    return result[dev];
  }
};

}  // namespace kda
