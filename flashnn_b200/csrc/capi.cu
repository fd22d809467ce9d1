// Status plumbing shared by every entry point of the C ABI: per-thread error
// text, the per-device status word that kernels write when a bounded wait runs
// out, and cached device properties.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "common.cuh"

namespace fnn {
namespace {

thread_local char g_error[512] = "";

// One status word per device that loads the library; kernels reach it through
// the address handed to them, host code through cudaMemcpyFromSymbol.
__device__ int g_device_status = 0;

constexpr int kMaxDevices = 64;
int* g_status_addr[kMaxDevices];
int g_sm_count[kMaxDevices];
std::once_flag g_once[kMaxDevices];

void init_device(int dev) {
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_device_status) == cudaSuccess) g_status_addr[dev] = static_cast<int*>(p);
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) g_sm_count[dev] = n;
}

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  std::call_once(g_once[dev], init_device, dev);
  return dev;
}

}  // namespace

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return status;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return FNN_OK;
  return fail(FNN_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

namespace {
std::atomic<int> g_opt_static_weights{0};
std::atomic<int> g_opt_test_stall_us{0};
std::atomic<int> g_opt_a8w8_pair_tile{0};
std::atomic<int> g_opt_a8w8_balanced{0};
}
int opt_a8w8_balanced() { return g_opt_a8w8_balanced.load(std::memory_order_relaxed); }
namespace { std::atomic<int> g_opt_a8w8_epilogue_warps{0}; }
int opt_a8w8_epilogue_warps() { return g_opt_a8w8_epilogue_warps.load(std::memory_order_relaxed); }
int opt_a8w8_pair_tile() { return g_opt_a8w8_pair_tile.load(std::memory_order_relaxed); }
bool opt_static_weights() { return g_opt_static_weights.load(std::memory_order_relaxed) != 0; }
int opt_test_stall_us() { return g_opt_test_stall_us.load(std::memory_order_relaxed); }

int* device_status_word() {
  const int dev = current_device();
  return dev < 0 ? nullptr : g_status_addr[dev];
}

namespace {
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}
}  // namespace

int make_tmap_2d(CUtensorMap* m, int elem_bytes, const void* base, int64_t rows, int64_t cols, int64_t pitch_bytes,
                 int box_cols, int box_rows, int swizzle) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return fail(FNN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(pitch_bytes)};
  const cuuint32_t box[2] = {cuuint32_t(box_cols), cuuint32_t(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
  const CUresult r = enc(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FNN_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", int(r));
  return FNN_OK;
}

int sm_count() {
  const int dev = current_device();
  return (dev < 0 || g_sm_count[dev] <= 0) ? 148 : g_sm_count[dev];
}

}  // namespace fnn

extern "C" int fnn_version(void) { return FNN_VERSION; }

extern "C" int fnn_set_option(int option, int value) {
  if (option == FNN_OPT_STATIC_WEIGHTS) {
    fnn::g_opt_static_weights.store(value != 0, std::memory_order_relaxed);
    return FNN_OK;
  }
  if (option == FNN_OPT_TEST_STALL_US) {
    if (value < 0 || value > 1000000)
      return fnn::fail(FNN_ERR_UNSUPPORTED, "fnn_set_option: FNN_OPT_TEST_STALL_US takes 0 .. 1000000 microseconds (got %d)", value);
    fnn::g_opt_test_stall_us.store(value, std::memory_order_relaxed);
    return FNN_OK;
  }
  if (option == FNN_OPT_A8W8_PAIR_TILE) {
    if (value != 0 && value != 256 && value != 224 && value != 192 && value != 160 && value != 128)
      return fnn::fail(FNN_ERR_UNSUPPORTED, "fnn_set_option: FNN_OPT_A8W8_PAIR_TILE takes 0, 128, 160, 192, 224 or 256 (got %d)", value);
    fnn::g_opt_a8w8_pair_tile.store(value, std::memory_order_relaxed);
    return FNN_OK;
  }
  if (option == FNN_OPT_A8W8_EPILOGUE_WARPS) {
    if (value != 0 && value != 4)
      return fnn::fail(FNN_ERR_UNSUPPORTED, "fnn_set_option: FNN_OPT_A8W8_EPILOGUE_WARPS takes 0 (by shape) or 4 (got %d)", value);
    fnn::g_opt_a8w8_epilogue_warps.store(value, std::memory_order_relaxed);
    return FNN_OK;
  }
  if (option == FNN_OPT_A8W8_BALANCED) {
    if (value < 0 || value > 2)
      return fnn::fail(FNN_ERR_UNSUPPORTED, "fnn_set_option: FNN_OPT_A8W8_BALANCED takes 0 (by shape), 1 (always) or 2 (never) (got %d)", value);
    fnn::g_opt_a8w8_balanced.store(value, std::memory_order_relaxed);
    return FNN_OK;
  }
  return fnn::fail(FNN_ERR_UNSUPPORTED, "fnn_set_option: unknown option %d", option);
}

extern "C" int fnn_get_option(int option) {
  if (option == FNN_OPT_STATIC_WEIGHTS) return fnn::g_opt_static_weights.load(std::memory_order_relaxed);
  if (option == FNN_OPT_TEST_STALL_US) return fnn::g_opt_test_stall_us.load(std::memory_order_relaxed);
  if (option == FNN_OPT_A8W8_PAIR_TILE) return fnn::g_opt_a8w8_pair_tile.load(std::memory_order_relaxed);
  if (option == FNN_OPT_A8W8_BALANCED) return fnn::g_opt_a8w8_balanced.load(std::memory_order_relaxed);
  if (option == FNN_OPT_A8W8_EPILOGUE_WARPS) return fnn::g_opt_a8w8_epilogue_warps.load(std::memory_order_relaxed);
  return -1;
}

extern "C" const char* fnn_last_error_string(void) { return fnn::g_error; }

extern "C" const char* fnn_status_string(int status) {
  switch (status) {
    case FNN_OK: return "ok";
    case FNN_ERR_NULL_POINTER: return "null pointer";
    case FNN_ERR_DTYPE: return "unsupported dtype";
    case FNN_ERR_SHAPE: return "bad shape";
    case FNN_ERR_ALIGNMENT: return "bad alignment";
    case FNN_ERR_UNSUPPORTED: return "unsupported combination";
    case FNN_ERR_WORKSPACE: return "workspace too small";
    case FNN_ERR_CUDA: return "CUDA error";
    case FNN_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}

extern "C" int fnn_device_status(int* device_code) {
  using namespace fnn;
  if (!device_code) return fail(FNN_ERR_NULL_POINTER, "device_status: null output pointer");
  int* word = device_status_word();
  if (!word) return fail(FNN_ERR_CUDA, "device_status: no current CUDA device");
  if (int e = check_cuda(cudaDeviceSynchronize(), "device_status: synchronize")) return e;
  int code = 0;
  if (int e = check_cuda(cudaMemcpy(&code, word, sizeof(int), cudaMemcpyDeviceToHost), "device_status: read")) return e;
  if (code != 0) {
    const int zero = 0;
    if (int e = check_cuda(cudaMemcpy(word, &zero, sizeof(int), cudaMemcpyHostToDevice), "device_status: clear")) return e;
  }
  *device_code = code;
  if (code != 0) return fail(FNN_ERR_DEVICE_TIMEOUT, "a kernel gave up on a bounded wait (device code %d)", code);
  return FNN_OK;
}
