// Once-per-device set-up guard.  Some CUDA settings belong to a device, not to the process: the dynamic
// shared memory ceiling of a kernel (cudaFuncSetAttribute) has to be raised on every device the library
// launches on, and a symbol's device address (cudaGetSymbolAddress) differs from device to device.  A
// process-wide `static bool` would do the set-up on the first device only.  Plain C++ (no CUDA headers), so
// that the logic can be compiled and tested on a machine without a GPU.
#pragma once
#include <mutex>

namespace p0p {

class DeviceOnce {
 public:
  static constexpr int kMaxDevices = 64;
  // Runs fn() with the lock held unless it already succeeded for this device; fn returns 0 on success.
  // A failed set-up is not remembered: the next call tries again.  Returns fn's code (0 when already done),
  // -1 for a device ordinal outside [0, kMaxDevices).
  template <class F>
  int run(int device, F&& fn) {
    if (device < 0 || device >= kMaxDevices) return -1;
    std::lock_guard<std::mutex> lock(mu_);
    if (done_[device]) return 0;
    const int rc = fn();
    if (rc == 0) done_[device] = true;
    return rc;
  }
  bool done(int device) {
    if (device < 0 || device >= kMaxDevices) return false;
    std::lock_guard<std::mutex> lock(mu_);
    return done_[device];
  }

 private:
  std::mutex mu_;
  bool done_[kMaxDevices] = {};
};

}  // namespace p0p
