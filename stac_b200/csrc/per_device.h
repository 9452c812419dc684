// Launch state that belongs to a GPU, not to the process: whether a kernel's opt-in to more
// than 48 KB of dynamic shared memory was made on that device, its SM count, the device
// address of a __device__ array.  A process that drives several GPUs keeps one entry per
// device ordinal.  Host-only C++ (no CUDA headers) so that it can be unit-tested without a GPU.
#pragma once

namespace stac {

constexpr int kMaxDevices = 64;

// One flag per device; set-up guarded by it must be idempotent (two host threads may both run it).
struct PerDeviceFlag {
  unsigned char done[kMaxDevices] = {};
  bool needs_setup(int dev) const { return !__atomic_load_n(&done[dev], __ATOMIC_ACQUIRE); }
  void mark(int dev) { __atomic_store_n(&done[dev], static_cast<unsigned char>(1), __ATOMIC_RELEASE); }
};

// One cached value per device (0 = not yet known).
template <typename T>
struct PerDeviceValue {
  T value[kMaxDevices] = {};
  T get(int dev) const { return __atomic_load_n(&value[dev], __ATOMIC_ACQUIRE); }
  void set(int dev, T v) { __atomic_store_n(&value[dev], v, __ATOMIC_RELEASE); }
};

inline bool device_index_ok(int dev) { return dev >= 0 && dev < kMaxDevices; }

}  // namespace stac
