// State the library keeps per CUDA device (scratch, streams, the kernel attributes
// that have to be set on each device) lives in tables indexed by the device
// ordinal, never in a single process-wide variable: one host process may drive
// several GPUs.  Plain C++, so the CPU tests can use it directly.
#pragma once

namespace sdcab {

constexpr int kMaxDevices = 64;

template <typename T>
struct PerDevice {
  T slot[kMaxDevices] = {};
  // the entry of device `dev`, or nullptr when the ordinal is out of range
  T* get(int dev) { return (dev >= 0 && dev < kMaxDevices) ? &slot[dev] : nullptr; }
};

// "Has this been done on device `dev` yet?" -- true exactly once per device.
struct OncePerDevice {
  PerDevice<bool> done;
  bool first_time(int dev) {
    bool* d = done.get(dev);
    if (!d || *d) return false;
    *d = true;
    return true;
  }
};

}  // namespace sdcab
