// Status strings, error bookkeeping, device properties and the library-owned
// workspace of the host-buffer entry points.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common_host.h"

namespace sdcab {

static thread_local char g_last_error[512] = "";

int record_cuda_error(cudaError_t err, const char* what) {
  std::snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)",
                what ? what : "cuda", cudaGetErrorString(err), cudaGetErrorName(err));
  if (err == cudaErrorMemoryAllocation) return SDCAB_ERR_OUT_OF_MEMORY;
  if (err == cudaErrorNoDevice || err == cudaErrorInsufficientDriver) return SDCAB_ERR_NO_DEVICE;
  return SDCAB_ERR_CUDA;
}

static DeviceInfo g_info[kMaxDevices];
static std::mutex g_mutex;

int get_device_info(DeviceInfo* out) {
  int dev = -1;
  SDCAB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return SDCAB_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceInfo& info = g_info[dev];
  if (info.device != dev) {
    int sm = 0, smem = 0;
    SDCAB_CUDA_TRY(cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev));
    SDCAB_CUDA_TRY(cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    info.device = dev; info.sm_count = sm; info.smem_optin = static_cast<size_t>(smem);
  }
  *out = info;
  return SDCAB_OK;
}

static const int kSlots = 8;
static Workspace g_ws[kMaxDevices][kSlots];

int workspace_reserve(int slot, size_t bytes, void** out) {
  int dev = -1;
  SDCAB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices || slot < 0 || slot >= kSlots) return SDCAB_ERR_ARG;
  std::lock_guard<std::mutex> lock(g_mutex);
  Workspace& w = g_ws[dev][slot];
  if (w.bytes < bytes) {
    if (w.ptr) { cudaFree(w.ptr); w.ptr = nullptr; w.bytes = 0; }
    SDCAB_CUDA_TRY(cudaMalloc(&w.ptr, bytes));
    w.bytes = bytes;
  }
  *out = w.ptr;
  return SDCAB_OK;
}

static Workspace g_pinned[kMaxDevices];

int pinned_reserve(size_t bytes, void** out) {
  int dev = -1;
  SDCAB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return SDCAB_ERR_ARG;
  std::lock_guard<std::mutex> lock(g_mutex);
  Workspace& w = g_pinned[dev];
  if (w.bytes < bytes) {
    if (w.ptr) { cudaFreeHost(w.ptr); w.ptr = nullptr; w.bytes = 0; }
    SDCAB_CUDA_TRY(cudaHostAlloc(&w.ptr, bytes, cudaHostAllocDefault));
    w.bytes = bytes;
  }
  *out = w.ptr;
  return SDCAB_OK;
}

struct StreamSet {
  cudaStream_t s[4] = {nullptr, nullptr, nullptr, nullptr};
};
static PerDevice<StreamSet> g_streams;

int pipeline_streams(int count, cudaStream_t* out) {
  int dev = -1;
  SDCAB_CUDA_TRY(cudaGetDevice(&dev));
  StreamSet* set = g_streams.get(dev);
  if (!set || count < 0 || count > 4) return SDCAB_ERR_ARG;
  std::lock_guard<std::mutex> lock(g_mutex);
  for (int i = 0; i < count; ++i) {
    if (!set->s[i]) SDCAB_CUDA_TRY(cudaStreamCreateWithFlags(&set->s[i], cudaStreamNonBlocking));
    out[i] = set->s[i];
  }
  return SDCAB_OK;
}

static PerDevice<std::mutex> g_call_mutex;

std::mutex* host_call_mutex() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
  std::mutex* m = g_call_mutex.get(dev);
  return m ? m : g_call_mutex.get(0);
}

static int workspace_release_all() {
  int dev = -1;
  SDCAB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return SDCAB_ERR_ARG;
  std::lock_guard<std::mutex> lock(g_mutex);
  for (int s = 0; s < kSlots; ++s) {
    Workspace& w = g_ws[dev][s];
    if (w.ptr) cudaFree(w.ptr);
    w.ptr = nullptr; w.bytes = 0;
  }
  if (g_pinned[dev].ptr) cudaFreeHost(g_pinned[dev].ptr);
  g_pinned[dev].ptr = nullptr; g_pinned[dev].bytes = 0;
  return SDCAB_OK;
}

}  // namespace sdcab

namespace sdcab {
// tile choice of the double-precision products (declared in gemm_blocked.cuh; tests only)
static int g_gemm_f64_tile_mode = 0;
int gemm_f64_tile_mode() { return g_gemm_f64_tile_mode; }
void set_gemm_f64_tile_mode(int mode) { g_gemm_f64_tile_mode = mode; }
}  // namespace sdcab

extern "C" {

const char* sdcab_status_string(int status) {
  switch (status) {
    case SDCAB_OK: return "ok";
    case SDCAB_ERR_ARG: return "LIBSDCA:arg";
    case SDCAB_ERR_ARG_RANGE: return "LIBSDCA:arg_range";
    case SDCAB_ERR_ARG_CLASS: return "LIBSDCA:arg_class";
    case SDCAB_ERR_NOT_EMPTY: return "LIBSDCA:arg_not_empty";
    case SDCAB_ERR_LABELS_RANGE: return "LIBSDCA:labels_range";
    case SDCAB_ERR_PROX: return "LIBSDCA:prox";
    case SDCAB_ERR_OBJECTIVE: return "LIBSDCA:objective";
    case SDCAB_ERR_PRECISION: return "LIBSDCA:precision";
    case SDCAB_ERR_OUT_OF_MEMORY: return "LIBSDCA:out_of_memory";
    case SDCAB_ERR_NOT_IMPLEMENTED: return "LIBSDCA:not_implemented";
    case SDCAB_ERR_NUM_DIM: return "LIBSDCA:num_dim";
    case SDCAB_ERR_CUDA: return "cuda_error";
    case SDCAB_ERR_NO_DEVICE: return "no_cuda_device";
    case SDCAB_ERR_TOO_LARGE: return "too_large";
    case SDCAB_ERR_TIMEOUT: return "device_wait_timeout";
    case SDCAB_ERR_NCCL: return "nccl_error";
  }
  return "unknown";
}

const char* sdcab_last_error(void) { return sdcab::g_last_error; }

const char* sdcab_version(void) { return "sdca_b200 0.1 (sm_100a)"; }

int sdcab_release_workspace(void) { return sdcab::workspace_release_all(); }

int sdcab_host_alloc(void** ptr, size_t bytes) {
  SDCAB_CUDA_TRY(cudaHostAlloc(ptr, bytes, cudaHostAllocDefault));
  return SDCAB_OK;
}

int sdcab_host_free(void* ptr) {
  SDCAB_CUDA_TRY(cudaFreeHost(ptr));
  return SDCAB_OK;
}

}  // extern "C"
