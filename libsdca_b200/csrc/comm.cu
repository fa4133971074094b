// The collective of the sharded gap evaluation: one all-reduce (sum) of the
// 8 + m doubles of the sums vector over the ranks that hold the shards of
// examples, issued through NCCL on the caller's stream.  A C or C++ host gets the
// sharded evaluation from the C ABI alone; the only other collective of the path
// -- the d x m sum of a sharded W = X A' rebuild -- goes through the same
// communicator.
//
// NCCL is bound at run time (dlopen of libnccl.so.2): the library itself keeps no
// link-time dependency on it, a process that already carries an NCCL (a PyTorch
// process, say) shares that copy, and a single-GPU host needs none at all.
#include <dlfcn.h>
#include <nccl.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "common_host.h"

struct sdcab_comm {
  ncclComm_t comm;
  int rank, size, device;
};

namespace sdcab {
namespace {

struct Nccl {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

static Nccl g_nccl;
static std::mutex g_nccl_mutex;
static thread_local char g_comm_error[256] = "";

const Nccl* nccl() {
  std::lock_guard<std::mutex> lock(g_nccl_mutex);
  if (g_nccl.ok) return &g_nccl;
  if (!g_nccl.handle) {
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
      g_nccl.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (g_nccl.handle) break;
    }
  }
  if (!g_nccl.handle) {
    std::snprintf(g_comm_error, sizeof(g_comm_error), "NCCL not found: %s", dlerror());
    return nullptr;
  }
#define BIND(field, symbol)                                                        \
  g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(g_nccl.handle, symbol)); \
  if (!g_nccl.field) { std::snprintf(g_comm_error, sizeof(g_comm_error), "NCCL lacks %s", symbol); return nullptr; }
  BIND(GetUniqueId, "ncclGetUniqueId")
  BIND(CommInitRank, "ncclCommInitRank")
  BIND(CommInitAll, "ncclCommInitAll")
  BIND(CommDestroy, "ncclCommDestroy")
  BIND(AllReduce, "ncclAllReduce")
  BIND(GetErrorString, "ncclGetErrorString")
#undef BIND
  g_nccl.ok = true;
  return &g_nccl;
}

int nccl_status(const Nccl* n, ncclResult_t r, const char* what) {
  if (r == ncclSuccess) return SDCAB_OK;
  std::snprintf(g_comm_error, sizeof(g_comm_error), "%s: %s", what, n->GetErrorString(r));
  return SDCAB_ERR_NCCL;
}

}  // namespace
}  // namespace sdcab

extern "C" {

const char* sdcab_comm_last_error(void) { return sdcab::g_comm_error; }

int sdcab_comm_unique_id(void* id_out) {
  if (!id_out) return SDCAB_ERR_ARG;
  const sdcab::Nccl* n = sdcab::nccl();
  if (!n) return SDCAB_ERR_NCCL;
  ncclUniqueId id;
  int rc = sdcab::nccl_status(n, n->GetUniqueId(&id), "ncclGetUniqueId");
  if (rc) return rc;
  static_assert(sizeof(id) == SDCAB_COMM_ID_BYTES, "unique id size");
  std::memcpy(id_out, &id, sizeof(id));
  return SDCAB_OK;
}

int sdcab_comm_create(sdcab_comm** out, int nranks, int rank, const void* id_bytes) {
  if (!out || !id_bytes || nranks < 1 || rank < 0 || rank >= nranks) return SDCAB_ERR_ARG;
  const sdcab::Nccl* n = sdcab::nccl();
  if (!n) return SDCAB_ERR_NCCL;
  int dev = -1;
  SDCAB_CUDA_TRY(cudaGetDevice(&dev));
  ncclUniqueId id;
  std::memcpy(&id, id_bytes, sizeof(id));
  ncclComm_t comm = nullptr;
  int rc = sdcab::nccl_status(n, n->CommInitRank(&comm, nranks, id, rank), "ncclCommInitRank");
  if (rc) return rc;
  sdcab_comm* c = new sdcab_comm;
  c->comm = comm; c->rank = rank; c->size = nranks; c->device = dev;
  *out = c;
  return SDCAB_OK;
}

int sdcab_comm_create_local(sdcab_comm** out, int ngpus, const int* devices) {
  if (!out || ngpus < 1 || ngpus > 64) return SDCAB_ERR_ARG;
  const sdcab::Nccl* n = sdcab::nccl();
  if (!n) return SDCAB_ERR_NCCL;
  ncclComm_t comms[64];
  int devs[64];
  for (int i = 0; i < ngpus; ++i) devs[i] = devices ? devices[i] : i;
  int rc = sdcab::nccl_status(n, n->CommInitAll(comms, ngpus, devs), "ncclCommInitAll");
  if (rc) return rc;
  for (int i = 0; i < ngpus; ++i) {
    sdcab_comm* c = new sdcab_comm;
    c->comm = comms[i]; c->rank = i; c->size = ngpus; c->device = devs[i];
    out[i] = c;
  }
  return SDCAB_OK;
}

int sdcab_comm_destroy(sdcab_comm* c) {
  if (!c) return SDCAB_OK;
  const sdcab::Nccl* n = sdcab::nccl();
  int rc = SDCAB_OK;
  if (n && c->comm) rc = sdcab::nccl_status(n, n->CommDestroy(c->comm), "ncclCommDestroy");
  delete c;
  return rc;
}

int sdcab_comm_rank(const sdcab_comm* c) { return c ? c->rank : -1; }
int sdcab_comm_size(const sdcab_comm* c) { return c ? c->size : 0; }

int sdcab_comm_allreduce_f64(sdcab_comm* c, double* buf_dev, int64_t count, void* stream) {
  if (!c) return SDCAB_OK;   // no communicator: a single shard, nothing to add
  if (!buf_dev || count < 0) return SDCAB_ERR_ARG;
  const sdcab::Nccl* n = sdcab::nccl();
  if (!n) return SDCAB_ERR_NCCL;
  return sdcab::nccl_status(n, n->AllReduce(buf_dev, buf_dev, static_cast<size_t>(count), ncclFloat64, ncclSum,
                                            c->comm, static_cast<cudaStream_t>(stream)), "ncclAllReduce");
}

int sdcab_comm_allreduce_f32(sdcab_comm* c, float* buf_dev, int64_t count, void* stream) {
  if (!c) return SDCAB_OK;
  if (!buf_dev || count < 0) return SDCAB_ERR_ARG;
  const sdcab::Nccl* n = sdcab::nccl();
  if (!n) return SDCAB_ERR_NCCL;
  return sdcab::nccl_status(n, n->AllReduce(buf_dev, buf_dev, static_cast<size_t>(count), ncclFloat32, ncclSum,
                                            c->comm, static_cast<cudaStream_t>(stream)), "ncclAllReduce");
}

int sdcab_eval_sums_sharded_f32_dev(const sdcab_objective* obj, const sdcab_problem* p, double* sums_dev,
                                    void* workspace_dev, size_t workspace_bytes, sdcab_comm* comm,
                                    void* stream) {
  int rc = sdcab_eval_sums_f32_dev(obj, p, sums_dev, workspace_dev, workspace_bytes, stream);
  if (rc) return rc;
  return sdcab_comm_allreduce_f64(comm, sums_dev, SDCAB_EVAL_SUMS(p->m), stream);
}

int sdcab_eval_sums_sharded_f64_dev(const sdcab_objective* obj, const sdcab_problem* p, double* sums_dev,
                                    void* workspace_dev, size_t workspace_bytes, sdcab_comm* comm,
                                    void* stream) {
  int rc = sdcab_eval_sums_f64_dev(obj, p, sums_dev, workspace_dev, workspace_bytes, stream);
  if (rc) return rc;
  return sdcab_comm_allreduce_f64(comm, sums_dev, SDCAB_EVAL_SUMS(p->m), stream);
}

}  // extern "C"
