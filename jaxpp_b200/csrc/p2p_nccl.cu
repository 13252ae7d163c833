// Point-to-point backend over NCCL for the pipeline runtime: one 2-rank communicator per directed pair of
// devices, all arrays of one transfer in one NCCL group, enqueued on a stream the caller names.
//
// Counterpart of the reference's cupy-based backend (src/jaxpp/dime2.py:72-105 communicator creation from an
// id exchanged through a key-value store, :258-345 grouped send / recv on a dedicated stream); here it is a
// C ABI over the NCCL library that the process has already loaded (resolved with dlopen / dlsym, so this
// library has no link-time dependency on NCCL).  Payloads are bytes: any dtype travels, fp8 included.
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace {

typedef void* nccl_comm_t;
struct nccl_unique_id { char internal[128]; };
typedef int nccl_result_t;        // ncclSuccess == 0
constexpr int kNcclInt8 = 0;      // ncclInt8 / ncclChar

typedef nccl_result_t (*fn_get_unique_id)(nccl_unique_id*);
typedef nccl_result_t (*fn_comm_init_rank)(nccl_comm_t*, int, nccl_unique_id, int);
typedef nccl_result_t (*fn_comm_destroy)(nccl_comm_t);
typedef nccl_result_t (*fn_group)(void);
typedef nccl_result_t (*fn_sendrecv)(void*, size_t, int, int, nccl_comm_t, cudaStream_t);
typedef const char* (*fn_error_string)(nccl_result_t);

struct NcclApi {
  void* handle = nullptr;
  fn_get_unique_id get_unique_id = nullptr;
  fn_comm_init_rank comm_init_rank = nullptr;
  fn_comm_destroy comm_destroy = nullptr;
  fn_group group_start = nullptr, group_end = nullptr;
  fn_sendrecv send = nullptr, recv = nullptr;
  fn_error_string error_string = nullptr;
  bool ok = false;
};

NcclApi g_api;
char g_error[512] = "";

void set_error(const char* what, nccl_result_t rc) {
  const char* msg = (g_api.error_string && rc > 0) ? g_api.error_string(rc) : "";
  snprintf(g_error, sizeof(g_error), "%s failed (%d) %s", what, rc, msg);
}

bool load_api() {
  if (g_api.ok) return true;
  if (g_api.handle == nullptr) {
    // the soname the framework's NCCL was loaded under; falls back to the unversioned name
    g_api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!g_api.handle) g_api.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!g_api.handle) {
      snprintf(g_error, sizeof(g_error), "libnccl not found: %s", dlerror());
      return false;
    }
  }
  void* h = g_api.handle;
  g_api.get_unique_id = reinterpret_cast<fn_get_unique_id>(dlsym(h, "ncclGetUniqueId"));
  g_api.comm_init_rank = reinterpret_cast<fn_comm_init_rank>(dlsym(h, "ncclCommInitRank"));
  g_api.comm_destroy = reinterpret_cast<fn_comm_destroy>(dlsym(h, "ncclCommDestroy"));
  g_api.group_start = reinterpret_cast<fn_group>(dlsym(h, "ncclGroupStart"));
  g_api.group_end = reinterpret_cast<fn_group>(dlsym(h, "ncclGroupEnd"));
  g_api.send = reinterpret_cast<fn_sendrecv>(dlsym(h, "ncclSend"));
  g_api.recv = reinterpret_cast<fn_sendrecv>(dlsym(h, "ncclRecv"));
  g_api.error_string = reinterpret_cast<fn_error_string>(dlsym(h, "ncclGetErrorString"));
  g_api.ok = g_api.get_unique_id && g_api.comm_init_rank && g_api.comm_destroy && g_api.group_start && g_api.group_end &&
             g_api.send && g_api.recv;
  if (!g_api.ok) snprintf(g_error, sizeof(g_error), "libnccl is missing a required symbol");
  return g_api.ok;
}

}  // namespace

struct JpbP2POp {
  void* ptr;
  long long bytes;
  int peer;      // rank inside the communicator
  int is_send;   // 1 send, 0 receive
};

JPB_API int jpb_p2p_available() { return load_api() ? 1 : 0; }
JPB_API const char* jpb_p2p_last_error() { return g_error; }

JPB_API int jpb_p2p_unique_id(unsigned char* out /* 128 bytes */) {
  if (!load_api()) return -1;
  nccl_unique_id id;
  const nccl_result_t rc = g_api.get_unique_id(&id);
  if (rc != 0) { set_error("ncclGetUniqueId", rc); return -2; }
  memcpy(out, id.internal, 128);
  return 0;
}

// Collective over the `nranks` processes that share `id`; returns when all of them have called it.
JPB_API int jpb_p2p_comm_create(const unsigned char* id_bytes, int nranks, int rank, void** comm_out) {
  if (!load_api()) return -1;
  nccl_unique_id id;
  memcpy(id.internal, id_bytes, 128);
  nccl_comm_t comm = nullptr;
  const nccl_result_t rc = g_api.comm_init_rank(&comm, nranks, id, rank);
  if (rc != 0) { set_error("ncclCommInitRank", rc); return -2; }
  *comm_out = comm;
  return 0;
}

JPB_API int jpb_p2p_comm_destroy(void* comm) {
  if (!load_api() || comm == nullptr) return 0;
  const nccl_result_t rc = g_api.comm_destroy(static_cast<nccl_comm_t>(comm));
  if (rc != 0) { set_error("ncclCommDestroy", rc); return -2; }
  return 0;
}

// All operations of one transfer as one NCCL group on `stream` (asynchronous with respect to the host).
JPB_API int jpb_p2p_batch(void* comm, const JpbP2POp* ops, int n, void* stream) {
  if (!load_api()) return -1;
  if (comm == nullptr || (n > 0 && ops == nullptr)) return -3;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  nccl_result_t rc = g_api.group_start();
  if (rc != 0) { set_error("ncclGroupStart", rc); return -2; }
  nccl_result_t first_bad = 0;
  for (int i = 0; i < n && first_bad == 0; ++i) {
    const JpbP2POp& op = ops[i];
    if (op.bytes <= 0) continue;
    rc = op.is_send ? g_api.send(op.ptr, size_t(op.bytes), kNcclInt8, op.peer, static_cast<nccl_comm_t>(comm), s)
                    : g_api.recv(op.ptr, size_t(op.bytes), kNcclInt8, op.peer, static_cast<nccl_comm_t>(comm), s);
    if (rc != 0) first_bad = rc;
  }
  rc = g_api.group_end();
  if (first_bad != 0) { set_error("ncclSend/ncclRecv", first_bad); return -2; }
  if (rc != 0) { set_error("ncclGroupEnd", rc); return -2; }
  return 0;
}
