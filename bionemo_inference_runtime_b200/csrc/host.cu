// Host-side plumbing shared by every entry point: status strings, per-device
// state, tensor-map encoding through the driver entry point (the library does
// not link libcuda, so it also loads on a machine without a driver).
#include <mutex>
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace b200ta {

namespace {
thread_local char g_error[512] = "";
std::mutex g_mutex;
constexpr int kMaxDevices = 64;
DeviceState g_devices[kMaxDevices];

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

// Written by a kernel that abandoned a bounded wait; read back by b200ta_device_status().
__device__ int g_status_word = 0;
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int get_device_state(DeviceState** out) {
  int dev = 0;
  B200TA_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(B200TA_ERR_INVALID, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState& st = g_devices[dev];
  if (st.device != dev) {
    cudaDeviceProp prop;
    B200TA_CHECK_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
      return fail(B200TA_ERR_UNSUPPORTED, "device %d is sm_%d%d; these kernels are built for sm_100a only",
                  dev, prop.major, prop.minor);
    // The status word is a file-scope device variable (one per device that loads the library), so creating
    // the state allocates nothing; its address is looked up once, with this device current.
    int* devp = nullptr;
    B200TA_CHECK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&devp), g_status_word));
    st.num_sms = prop.multiProcessorCount;
    st.status_dev = devp;
    st.device = dev;
  }
  *out = &st;
  return B200TA_OK;
}

int encode_tensor_map(CUtensorMap* map, const void* base, int elem_bytes, int rank,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      SwizzleMode swz, const char* what) {
  if (g_encode == nullptr) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
      if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr)
        return fail(B200TA_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from this driver");
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return fail(B200TA_ERR_INVALID, "%s: base address must be 16-byte aligned", what);
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (dims[i] == 0) return fail(B200TA_ERR_INVALID, "%s: dimension %d is empty", what, i);
    if (box[i] == 0 || box[i] > 256) return fail(B200TA_ERR_INVALID, "%s: box[%d]=%u out of range", what, i, box[i]);
  }
  for (int i = 0; i + 1 < rank; ++i) {
    gstrides[i] = strides_bytes[i];
    if ((strides_bytes[i] & 15u) != 0)
      return fail(B200TA_ERR_INVALID, "%s: stride %d (%llu bytes) must be a multiple of 16 bytes", what,
                  i + 1, (unsigned long long)strides_bytes[i]);
  }
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUtensorMapSwizzle sw = swz == SWZ_128  ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swz == SWZ_64 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swz == SWZ_32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                          : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = g_encode(map, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims, gstrides, gbox,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200TA_ERR_DRIVER, "%s: cuTensorMapEncodeTiled returned %d", what, (int)r);
  return B200TA_OK;
}

}  // namespace b200ta

extern "C" {

int b200ta_version(void) { return 100; }

const char* b200ta_last_error(void) { return b200ta::g_error; }

int b200ta_device_status(int* status) {
  if (status == nullptr) return b200ta::fail(B200TA_ERR_INVALID, "status must not be NULL");
  b200ta::DeviceState* st = nullptr;
  int rc = b200ta::get_device_state(&st);
  if (rc != B200TA_OK) return rc;
  B200TA_CHECK_CUDA(cudaMemcpy(status, st->status_dev, sizeof(int), cudaMemcpyDeviceToHost));
  return B200TA_OK;
}

int b200ta_reset_device_status(void) {
  b200ta::DeviceState* st = nullptr;
  int rc = b200ta::get_device_state(&st);
  if (rc != B200TA_OK) return rc;
  const int zero = 0;
  B200TA_CHECK_CUDA(cudaMemcpy(st->status_dev, &zero, sizeof(int), cudaMemcpyHostToDevice));
  return B200TA_OK;
}

}  // extern "C"
