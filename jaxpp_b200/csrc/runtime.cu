// Host-side runtime pieces shared by all kernels: the status word that device code reports bounded-wait
// time-outs through, TMA descriptor encoding (driver entry point looked up at run time, so the library
// links against the CUDA runtime only), and device queries.
#include "common.cuh"

#include <cstdio>
#include <cstring>
#include <mutex>

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PFN_encodeTiled g_encode = nullptr;
static std::once_flag g_encode_once;

static void load_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess)
    g_encode = reinterpret_cast<PFN_encodeTiled>(fn);
}

int jpb_make_tensor_map(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box, int swizzle_128b) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return -100;
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                         : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                           : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstrides[i] = strides_bytes[i];
  CUresult r = g_encode(out, dt, rank, const_cast<void*>(base), gdims, gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(1000 + int(r));
}

// ---- status word: one int per device in mapped pinned host memory --------------------------------------
static int* g_status_host[64] = {nullptr};
static int* g_status_dev[64] = {nullptr};
static std::mutex g_status_mutex;

int* jpb_status_device_ptr() {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (!g_status_dev[dev]) {
    int* h = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void**>(&h), 64, cudaHostAllocMapped) != cudaSuccess) return nullptr;
    for (int i = 0; i < 16; ++i) h[i] = 0;
    int* d = nullptr;
    cudaHostGetDevicePointer(reinterpret_cast<void**>(&d), h, 0);
    g_status_host[dev] = h;
    g_status_dev[dev] = d;
  }
  return g_status_dev[dev];
}

// Read (and optionally clear) the status word of the current device.  Non-zero = a kernel gave up on a
// bounded wait or rejected its arguments (see JpbStatus).  Call after a stream/device synchronise.
JPB_API int jpb_read_status(int clear) {
  int dev = 0;
  cudaGetDevice(&dev);
  jpb_status_device_ptr();
  int v = g_status_host[dev] ? *reinterpret_cast<volatile int*>(g_status_host[dev]) : 0;
  if (clear && g_status_host[dev]) *reinterpret_cast<volatile int*>(g_status_host[dev]) = 0;
  return v;
}

// ---- run-time wait budget ----------------------------------------------------------------------------------------
// Every .cu file of the library holds its own copy of the device variable (see common.cuh) and registers a setter
// for it during static initialisation; the table is a function-local static so that it exists before the first
// registration whatever the initialisation order of the object files.
struct BudgetSetters {
  JpbWaitBudgetSetter fn[32];
  int n = 0;
};
static BudgetSetters& budget_setters() {
  static BudgetSetters table;
  return table;
}
void jpb_register_wait_budget_setter(JpbWaitBudgetSetter fn) {
  BudgetSetters& t = budget_setters();
  if (t.n < 32) t.fn[t.n++] = fn;
}

// Longest time any device-side wait of this library may spin on the CURRENT device before its kernel gives up,
// records a status and returns (default 4 s).  Takes effect for kernels launched after the call; a value of 0 is
// rejected.  Returns 0 or the first CUDA error.
JPB_API int jpb_set_wait_budget_ns(unsigned long long ns) {
  if (ns == 0) return -JPB_ERR_BAD_ARGUMENT;
  BudgetSetters& t = budget_setters();
  for (int i = 0; i < t.n; ++i) {
    int rc = t.fn[i](ns);
    if (rc != 0) return rc;
  }
  return 0;
}

JPB_API int jpb_num_sms() {
  int dev = 0, n = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

JPB_API const char* jpb_build_info() { return "jaxpp_b200 native kernels, sm_100a, CUDA " JPB_STR(CUDART_VERSION); }

// ---- symmetric (peer-mapped) device memory through CUDA IPC ---------------------------------------------------
// Every rank allocates the same number of bytes, publishes the 64-byte handle, and opens its peers' handles;
// the kernels then address peers' buffers with plain pointers over NVLink.
// The buffer is zero-filled on `stream`: whatever the caller does to it next (guard-band patterns, staging copies,
// kernels) must be ordered after that fill, which holds for work on the same stream.  (A fill on the default stream
// is not ordered with a non-blocking stream: a later, smaller fill issued there could run first and be wiped out.)
JPB_API int jpb_ipc_alloc2(long long bytes, void** ptr, unsigned char* handle_out /* 64 bytes */, void* stream) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, size_t(bytes));
  if (e != cudaSuccess) return int(e);
  e = cudaMemsetAsync(p, 0, size_t(bytes), static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return int(e);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return int(e);
  static_assert(sizeof(h) == 64, "unexpected IPC handle size");
  memcpy(handle_out, &h, 64);
  *ptr = p;
  return 0;
}
JPB_API int jpb_ipc_alloc(long long bytes, void** ptr, unsigned char* handle_out) {
  return jpb_ipc_alloc2(bytes, ptr, handle_out, nullptr);
}

JPB_API int jpb_ipc_open(const unsigned char* handle, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  return int(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}

JPB_API int jpb_ipc_close(void* ptr) { return int(cudaIpcCloseMemHandle(ptr)); }
JPB_API int jpb_ipc_free(void* ptr) { return int(cudaFree(ptr)); }
JPB_API int jpb_memset_async(void* ptr, int value, long long bytes, void* stream) {
  return int(cudaMemsetAsync(ptr, value, size_t(bytes), static_cast<cudaStream_t>(stream)));
}
JPB_API int jpb_memcpy_async(void* dst, const void* src, long long bytes, void* stream) {
  return int(cudaMemcpyAsync(dst, src, size_t(bytes), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
}
