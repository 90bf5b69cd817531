// Host-side helpers of the C ABI that are not arithmetic: device memory and
// copies for hosts that bring no allocator of their own (a ctypes harness, a
// test written in C), and the cross-GPU collectives of the row-sharded path
// (aqt_b200/distributed.py describes which quantities cross ranks and why).
//
// NCCL is not linked: libnccl.so.2 is opened on the first aqtb200_comm_* call,
// so a single-GPU host never needs it, and a process that already carries an
// NCCL (through another framework) shares that copy.
#include <dlfcn.h>

#include <cstring>
#include <mutex>

#include "common.cuh"

namespace aqtb200 {

// The slice of NCCL's C API used here, declared locally so that no NCCL header
// is needed to build. The types and enumerator values are those of nccl.h
// (stable across NCCL 2.x).
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclInt32 = 2, ncclFloat32 = 7, ncclBfloat16 = 9 };
enum { ncclSum = 0, ncclMax = 2 };

struct Nccl {
  void* handle = nullptr;
  int (*GetUniqueId)(ncclUniqueId*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
};

static Nccl g_nccl;
static std::mutex g_nccl_mu;

static int load_nccl() {
  std::lock_guard<std::mutex> lock(g_nccl_mu);
  if (g_nccl.handle != nullptr) return 0;
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  AQT_REQUIRE(h != nullptr, AQTB200_EDRIVER, "libnccl.so.2 could not be opened: %s", dlerror());
#define AQT_NCCL_SYM(field, name)                                                     \
  do {                                                                                \
    *(void**)(&g_nccl.field) = dlsym(h, name);                                        \
    AQT_REQUIRE(g_nccl.field != nullptr, AQTB200_EDRIVER, "libnccl lacks %s", name);  \
  } while (0)
  AQT_NCCL_SYM(GetUniqueId, "ncclGetUniqueId");
  AQT_NCCL_SYM(CommInitRank, "ncclCommInitRank");
  AQT_NCCL_SYM(CommDestroy, "ncclCommDestroy");
  AQT_NCCL_SYM(AllReduce, "ncclAllReduce");
  AQT_NCCL_SYM(ReduceScatter, "ncclReduceScatter");
  AQT_NCCL_SYM(AllGather, "ncclAllGather");
  AQT_NCCL_SYM(GetErrorString, "ncclGetErrorString");
#undef AQT_NCCL_SYM
  g_nccl.handle = h;
  return 0;
}

#define AQT_NCCL_OK(expr)                                                              \
  do {                                                                                 \
    int r_ = (expr);                                                                   \
    if (r_ != 0) {                                                                     \
      ::aqtb200::set_error("%s failed: %s", #expr, g_nccl.GetErrorString(r_));         \
      return AQTB200_EDRIVER;                                                          \
    }                                                                                  \
  } while (0)

static int nccl_dtype(int dt, int* out) {
  switch (dt) {
    case AQTB200_F32: *out = ncclFloat32; return 0;
    case AQTB200_S32: *out = ncclInt32; return 0;
    case AQTB200_BF16: *out = ncclBfloat16; return 0;
    default: set_error("collectives take f32, s32 or bf16 (got dtype %d)", dt); return AQTB200_EINVAL;
  }
}

}  // namespace aqtb200

using namespace aqtb200;

extern "C" {

// ---- device memory for hosts without an allocator of their own -------------
int aqtb200_dev_alloc(void** out, size_t bytes) {
  AQT_REQUIRE(out != nullptr, AQTB200_EINVAL, "null argument");
  AQT_CUDA_OK(cudaMalloc(out, bytes > 0 ? bytes : 1));
  return 0;
}
int aqtb200_dev_free(void* ptr) {
  AQT_CUDA_OK(cudaFree(ptr));
  return 0;
}
int aqtb200_dev_memset(void* ptr, int value, size_t bytes, void* stream) {
  AQT_CUDA_OK(cudaMemsetAsync(ptr, value, bytes, (cudaStream_t)stream));
  return 0;
}
int aqtb200_h2d(void* dst, const void* src, size_t bytes, void* stream) {
  AQT_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return 0;
}
int aqtb200_d2h(void* dst, const void* src, size_t bytes, void* stream) {
  AQT_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return 0;
}
int aqtb200_sync(void* stream) {
  AQT_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
  return 0;
}
int aqtb200_set_device(int device) {
  AQT_CUDA_OK(cudaSetDevice(device));
  return 0;
}

// ---- peer memory -----------------------------------------------------------
int aqtb200_ipc_export(const void* ptr, void* handle64) {
  AQT_REQUIRE(ptr != nullptr && handle64 != nullptr, AQTB200_EINVAL, "null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is documented as 64 bytes");
  cudaIpcMemHandle_t h;
  AQT_CUDA_OK(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)));
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
int aqtb200_ipc_open(const void* handle64, void** out) {
  AQT_REQUIRE(handle64 != nullptr && out != nullptr, AQTB200_EINVAL, "null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  AQT_CUDA_OK(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
int aqtb200_ipc_close(void* ptr) {
  AQT_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return 0;
}

// ---- collectives ---------------------------------------------------------
int aqtb200_comm_unique_id(void* id128) {
  AQT_REQUIRE(id128 != nullptr, AQTB200_EINVAL, "null argument");
  int rc = load_nccl();
  if (rc) return rc;
  AQT_NCCL_OK(g_nccl.GetUniqueId((ncclUniqueId*)id128));
  return 0;
}

int aqtb200_comm_init(int nranks, int rank, const void* id128, void** comm_out) {
  AQT_REQUIRE(id128 != nullptr && comm_out != nullptr && nranks >= 1 && rank >= 0 && rank < nranks,
              AQTB200_EINVAL, "bad communicator arguments");
  int rc = load_nccl();
  if (rc) return rc;
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  ncclComm_t comm = nullptr;
  AQT_NCCL_OK(g_nccl.CommInitRank(&comm, nranks, id, rank));
  *comm_out = (void*)comm;
  return 0;
}

int aqtb200_comm_destroy(void* comm) {
  if (comm == nullptr) return 0;
  int rc = load_nccl();
  if (rc) return rc;
  AQT_NCCL_OK(g_nccl.CommDestroy((ncclComm_t)comm));
  return 0;
}

int aqtb200_allreduce(void* comm, void* buf, int64_t count, int32_t dtype, int32_t op_max,
                      void* stream) {
  AQT_REQUIRE(comm != nullptr && (buf != nullptr || count == 0) && count >= 0, AQTB200_EINVAL,
              "bad all-reduce arguments");
  int dt = 0, rc = nccl_dtype(dtype, &dt);
  if (rc) return rc;
  if (count == 0) return 0;
  AQT_NCCL_OK(g_nccl.AllReduce(buf, buf, (size_t)count, dt, op_max ? ncclMax : ncclSum,
                               (ncclComm_t)comm, (cudaStream_t)stream));
  return 0;
}

int aqtb200_reduce_scatter_sum(void* comm, const void* send, void* recv, int64_t recv_count,
                               int32_t dtype, void* stream) {
  AQT_REQUIRE(comm != nullptr && send != nullptr && recv != nullptr && recv_count > 0,
              AQTB200_EINVAL, "bad reduce-scatter arguments");
  int dt = 0, rc = nccl_dtype(dtype, &dt);
  if (rc) return rc;
  AQT_NCCL_OK(g_nccl.ReduceScatter(send, recv, (size_t)recv_count, dt, ncclSum, (ncclComm_t)comm,
                                   (cudaStream_t)stream));
  return 0;
}

int aqtb200_all_gather(void* comm, const void* send, void* recv, int64_t send_count, int32_t dtype,
                       void* stream) {
  AQT_REQUIRE(comm != nullptr && send != nullptr && recv != nullptr && send_count > 0,
              AQTB200_EINVAL, "bad all-gather arguments");
  int dt = 0, rc = nccl_dtype(dtype, &dt);
  if (rc) return rc;
  AQT_NCCL_OK(g_nccl.AllGather(send, recv, (size_t)send_count, dt, (ncclComm_t)comm,
                               (cudaStream_t)stream));
  return 0;
}

}  // extern "C"
