// Library-wide host plumbing of the C ABI: thread-local error text, the device
// status word written by bounded waits, and the TMA tensor-map encoder.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"
#include "tensor_map.cuh"
#include "../../include/nano_omni_b200.h"

namespace nob200 {

static thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return code;
}

int check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    return fail(kCudaError, "%s: %s: %s", what, cudaGetErrorName(err), cudaGetErrorString(err));
  }
  return kOk;
}

// One status word per device that loads the library.
__device__ uint32_t g_status_word = 0;

uint32_t* status_word_device_ptr() {
  // The symbol's address differs per device; query it for the current one.
  static thread_local int cached_device = -1;
  static thread_local uint32_t* cached_ptr = nullptr;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return nullptr;
  if (device != cached_device) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    cached_ptr = static_cast<uint32_t*>(p);
    cached_device = device;
  }
  return cached_ptr;
}

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return static_cast<EncodeTiledFn>(nullptr);
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int make_tensor_map_3d(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t d0, uint64_t d1,
                       uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1,
                       uint32_t b2, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(kUnsupported, "cuTensorMapEncodeTiled is not available from this driver");
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0)
    return fail(kInvalidArgument, "tensor base %p is not 16-byte aligned", base);
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = fn(map, type, 3, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(kCudaError, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return kOk;
}

}  // namespace nob200

extern "C" const char* nob200_last_error(void) { return nob200::g_error; }

extern "C" int nob200_read_status(uint32_t* out, void* stream) {
  NOB_REQUIRE(out != nullptr, "nob200_read_status: out is NULL");
  uint32_t* dev = nob200::status_word_device_ptr();
  if (!dev) return nob200::fail(nob200::kCudaError, "status word address is unavailable");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err = cudaMemcpyAsync(out, dev, sizeof(uint32_t), cudaMemcpyDeviceToHost, s);
  if (err == cudaSuccess) err = cudaMemsetAsync(dev, 0, sizeof(uint32_t), s);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess)
    return nob200::fail(nob200::kCudaError, "nob200_read_status: %s", cudaGetErrorString(err));
  return nob200::kOk;
}

extern "C" int nob200_abi_version(void) { return NOB200_ABI_VERSION; }
