// Tensor-parallel exchange step of the path: one NCCL communicator per process and an
// in-place sum all-reduce, behind the C ABI.  Stands in for
// vllm.distributed.tensor_model_parallel_all_reduce as RowParallelLinear calls it after the
// o_proj GEMM (additional_designs/model_executor/layers/aptserve_linear.py:827-829).
//
// NCCL is not linked: the first call resolves the few functions it needs from the
// "libnccl.so.2" the process already has (the one PyTorch loaded) or, in a host without
// PyTorch, from the system's.  Only the stable 2.x entry points are used and the handful of
// types below are declared here, so no NCCL header is needed to build.
#include <dlfcn.h>

#include <cstdio>
#include <cstring>

#include <mutex>

#include "aps_common.cuh"

namespace {

// ---- the slice of NCCL's C interface this file uses ------------------------------------
struct NcclUniqueId { char internal[APS_TP_UNIQUE_ID_BYTES]; };
typedef struct ncclComm* NcclComm;
enum { kNcclSuccess = 0 };
enum { kNcclSum = 0 };
enum { kNcclFloat16 = 6, kNcclFloat32 = 7, kNcclBfloat16 = 9 };

struct NcclApi {
  int (*get_unique_id)(NcclUniqueId*) = nullptr;
  int (*comm_init_rank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
  int (*all_reduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*comm_destroy)(NcclComm) = nullptr;
  int (*comm_count)(NcclComm, int*) = nullptr;
  const char* (*get_error_string)(int) = nullptr;
  bool ok = false;
  char why[160] = {0};
};

NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (h == nullptr) {
      snprintf(api.why, sizeof(api.why), "NCCL library not found (%s)", dlerror());
      return;
    }
    api.get_unique_id = reinterpret_cast<decltype(api.get_unique_id)>(dlsym(h, "ncclGetUniqueId"));
    api.comm_init_rank = reinterpret_cast<decltype(api.comm_init_rank)>(dlsym(h, "ncclCommInitRank"));
    api.all_reduce = reinterpret_cast<decltype(api.all_reduce)>(dlsym(h, "ncclAllReduce"));
    api.comm_destroy = reinterpret_cast<decltype(api.comm_destroy)>(dlsym(h, "ncclCommDestroy"));
    api.comm_count = reinterpret_cast<decltype(api.comm_count)>(dlsym(h, "ncclCommCount"));
    api.get_error_string = reinterpret_cast<decltype(api.get_error_string)>(dlsym(h, "ncclGetErrorString"));
    api.ok = api.get_unique_id && api.comm_init_rank && api.all_reduce && api.comm_destroy &&
             api.comm_count && api.get_error_string;
    if (!api.ok) snprintf(api.why, sizeof(api.why), "NCCL library lacks an expected entry point");
  });
  return api;
}

int nccl_fail(const char* op, const char* call, int rc) {
  return aps::fail(APS_ERR_CUDA, "%s: %s failed: %s", op, call, nccl().get_error_string(rc));
}

#define APS_NCCL_READY(op)                                                                  \
  do {                                                                                      \
    if (!nccl().ok) return aps::fail(APS_ERR_UNSUPPORTED, "%s: %s", op, nccl().why);        \
  } while (0)

}  // namespace

extern "C" int aps_tp_unique_id(void* unique_id_out) {
  const char* op = "aps_tp_unique_id";
  APS_REQUIRE(unique_id_out != nullptr, APS_ERR_NULL_POINTER, "%s: null output", op);
  APS_NCCL_READY(op);
  NcclUniqueId id;
  const int rc = nccl().get_unique_id(&id);
  if (rc != kNcclSuccess) return nccl_fail(op, "ncclGetUniqueId", rc);
  memcpy(unique_id_out, &id, sizeof(id));
  return APS_OK;
}

extern "C" int aps_tp_init(void** comm_out, const void* unique_id, int rank, int world_size) {
  const char* op = "aps_tp_init";
  APS_REQUIRE(comm_out != nullptr && unique_id != nullptr, APS_ERR_NULL_POINTER, "%s: null argument", op);
  APS_REQUIRE(world_size >= 1 && rank >= 0 && rank < world_size, APS_ERR_SHAPE,
              "%s: rank %d of %d", op, rank, world_size);
  APS_NCCL_READY(op);
  NcclUniqueId id;
  memcpy(&id, unique_id, sizeof(id));
  NcclComm comm = nullptr;
  const int rc = nccl().comm_init_rank(&comm, world_size, id, rank);   // on the current device
  if (rc != kNcclSuccess) return nccl_fail(op, "ncclCommInitRank", rc);
  *comm_out = comm;
  return APS_OK;
}

extern "C" int aps_tp_allreduce(void* comm, void* buffer, int64_t count, int dtype, void* stream) {
  const char* op = "aps_tp_allreduce";
  APS_REQUIRE(comm != nullptr, APS_ERR_NULL_POINTER, "%s: null communicator", op);
  APS_REQUIRE(count >= 0, APS_ERR_SHAPE, "%s: negative count", op);
  if (count == 0) return APS_OK;
  APS_REQUIRE(buffer != nullptr, APS_ERR_NULL_POINTER, "%s: null buffer", op);
  int nccl_type;
  switch (dtype) {
    case APS_F32: nccl_type = kNcclFloat32; break;
    case APS_F16: nccl_type = kNcclFloat16; break;
    case APS_BF16: nccl_type = kNcclBfloat16; break;
    default: return aps::fail(APS_ERR_DTYPE, "%s: unsupported dtype %d", op, dtype);
  }
  APS_NCCL_READY(op);
  const int rc = nccl().all_reduce(buffer, buffer, (size_t)count, nccl_type, kNcclSum,
                                   static_cast<NcclComm>(comm), static_cast<cudaStream_t>(stream));
  if (rc != kNcclSuccess) return nccl_fail(op, "ncclAllReduce", rc);
  return APS_OK;
}

extern "C" int aps_tp_world_size(void* comm, int* world_size_out) {
  const char* op = "aps_tp_world_size";
  APS_REQUIRE(comm != nullptr && world_size_out != nullptr, APS_ERR_NULL_POINTER, "%s: null argument", op);
  APS_NCCL_READY(op);
  const int rc = nccl().comm_count(static_cast<NcclComm>(comm), world_size_out);
  if (rc != kNcclSuccess) return nccl_fail(op, "ncclCommCount", rc);
  return APS_OK;
}

extern "C" int aps_tp_destroy(void* comm) {
  const char* op = "aps_tp_destroy";
  if (comm == nullptr) return APS_OK;
  APS_NCCL_READY(op);
  const int rc = nccl().comm_destroy(static_cast<NcclComm>(comm));
  if (rc != kNcclSuccess) return nccl_fail(op, "ncclCommDestroy", rc);
  return APS_OK;
}
