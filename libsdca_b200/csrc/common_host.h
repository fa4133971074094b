// Host-side helpers shared by the translation units of the library: error
// bookkeeping, launch geometry and a grow-only device workspace.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <mutex>

#include "../../include/sdca_b200.h"
#include "per_device.h"

namespace sdcab {

// Records the CUDA error text for sdcab_last_error() and maps it to a status.
int record_cuda_error(cudaError_t err, const char* what);

#define SDCAB_CUDA_TRY(expr)                                          \
  do {                                                                \
    cudaError_t err__ = (expr);                                       \
    if (err__ != cudaSuccess) return ::sdcab::record_cuda_error(err__, #expr); \
  } while (0)

// Properties of the current device, queried once per device.
struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  size_t smem_optin = 0;  // largest dynamic shared memory per block
};
int get_device_info(DeviceInfo* info);

// Grow-only per-device scratch owned by the library; used only by the
// host-buffer entry points (the *_dev entry points allocate nothing unless
// their documentation says so).  The table is guarded by a mutex, and the
// host-buffer entry points hold host_call_mutex() of their device while they
// use the scratch, so concurrent calls from several host threads are
// serialised per device rather than racing on it.
struct Workspace {
  void* ptr = nullptr;
  size_t bytes = 0;
};
int workspace_reserve(int slot, size_t bytes, void** out);
// Same for page-locked host memory (staging of small results).
int pinned_reserve(size_t bytes, void** out);
// `count` (at most 4) non-blocking streams of the current device, created on
// first use on that device and kept for the life of the process.
int pipeline_streams(int count, cudaStream_t* out);
// The mutex that serialises host-buffer calls on the current device.
std::mutex* host_call_mutex();

}  // namespace sdcab
