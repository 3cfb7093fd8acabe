// Host-side plumbing of libtgdn_b200: return codes, the device status word, tensor-map construction.
#include <stdio.h>

#include "tgdn_common.cuh"
#include "tgdn_host.h"
#include "tgdn_kernels.h"

namespace {

__device__ int g_status_word = 0;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

}  // namespace

int tgdn_cuda_error(cudaError_t e) { return e == cudaSuccess ? 0 : -(1000 + static_cast<int>(e)); }

int* tgdn_status_word() {
  static int* cached[64] = {nullptr};          // per device: the address never changes once the module is loaded
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  if (dev >= 0 && dev < 64 && cached[dev] != nullptr) return cached[dev];
  int* p = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status_word) != cudaSuccess) return nullptr;
  if (dev >= 0 && dev < 64) cached[dev] = p;
  return p;
}

int tgdn_check_device() {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  // Make the device's primary context current on the calling thread.  The tensor-map encoder is a driver call and
  // fails with "invalid context" on a thread that has not touched the runtime yet (an autograd worker whose tensors all
  // came out of the allocator's cache); setting the current device again is the documented way to bind the context.
  if (cudaSetDevice(dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return 0;
  return major == 10;
}

int tgdn_make_token_map(CUtensorMap* map, const void* base, int B, int T, int H, int box_cols, int box_rows,
                        int swizzle128) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return TGDN_ERR_DRIVER;
  if (reinterpret_cast<uintptr_t>(base) & 15) return TGDN_ERR_ALIGN;
  if (swizzle128 && box_cols != 64) return TGDN_ERR_SHAPE;
  const cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[3] = {256, static_cast<cuuint64_t>(H) * 256, static_cast<cuuint64_t>(T) * H * 256};
  const cuuint32_t box[4] = {static_cast<cuuint32_t>(box_cols), 1, static_cast<cuuint32_t>(box_rows), 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : TGDN_ERR_DRIVER;
}

int tgdn_make_gate_map(CUtensorMap* map, const float* base, int B, int T, int H, int E) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return TGDN_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || E % 4) return TGDN_ERR_ALIGN;
  const cuuint64_t row = static_cast<cuuint64_t>(E) * 4;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(E), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[3] = {row, static_cast<cuuint64_t>(H) * row, static_cast<cuuint64_t>(T) * H * row};
  const cuuint32_t box[4] = {static_cast<cuuint32_t>(E), 1, 64, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : TGDN_ERR_DRIVER;
}

int tgdn_make_rows_map(CUtensorMap* map, const void* base, int C, int T, int B, int64_t stride_t, int64_t stride_b, int box_cols,
                       int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return TGDN_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (stride_t % 8) || (stride_b % 8)) return TGDN_ERR_ALIGN;
  if (box_cols > 256 || box_rows > 256) return TGDN_ERR_SHAPE;
  // a single batch row needs no third stride; give it any valid multiple of 16 bytes
  const cuuint64_t sb = (B > 1) ? static_cast<cuuint64_t>(stride_b) * 2 : static_cast<cuuint64_t>(stride_t) * 2 * static_cast<cuuint64_t>(T);
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(stride_t) * 2, sb};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows), 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : TGDN_ERR_DRIVER;
}

int tgdn_check_core_shape(int B, int T, int H, int E, int NC, int packed) {
  if (B <= 0 || T <= 0 || H <= 0 || NC <= 0) return TGDN_ERR_SHAPE;
  if (E != 1 && E != 2 && E != 4 && E != 8 && E != 12 && E != 16) return TGDN_ERR_SHAPE;
  if (packed) {
    if (B != 1 || NC < (T + 63) / 64) return TGDN_ERR_SHAPE;
  } else if (T % 64 || NC != T / 64) {
    return TGDN_ERR_SHAPE;
  }
  if (static_cast<long long>(B) * NC * H > 0x7fffffffLL) return TGDN_ERR_SHAPE;
  if (!tgdn_check_device()) return TGDN_ERR_DEVICE;
  return 0;
}

// Number of SMs of the current device.  With one resident CTA per SM and blocks dispatched in index order, block
// i + count starts about when block i ends, which is what the per-item kernels use to warm L2 for their successor.
int tgdn_sm_count() {
  static int cached[64] = {0};
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
  if (dev >= 0 && dev < 64) cached[dev] = n;
  return n;
}

int tgdn_value_block(int E) { return E > 8 ? 16 : 32; }   // must match the dispatch in tgdn_bwd_rec.cu

extern "C" const char* tgdn_error_string(int code) {
  static thread_local char buf[160];
  switch (code) {
    case TGDN_OK: return "ok";
    case TGDN_ERR_SHAPE: return "unsupported or inconsistent sizes";
    case TGDN_ERR_NULL: return "a required pointer is NULL";
    case TGDN_ERR_ALIGN: return "a pointer or stride is not 16-byte aligned";
    case TGDN_ERR_DRIVER: return "cuTensorMapEncodeTiled is unavailable or rejected the tensor";
    case TGDN_ERR_SCRATCH: return "scratch buffer missing or too small";
    case TGDN_ERR_DEVICE: return "the current device is not compute capability 10.x (sm_100a kernels)";
    case TGDN_ERR_STATIC_LIMIT: return "the problem needs more scratch than the library's built-in static buffer holds";
    default: break;
  }
  if (code <= -1000) {
    snprintf(buf, sizeof(buf), "CUDA error %d: %s", -code - 1000, cudaGetErrorString(static_cast<cudaError_t>(-code - 1000)));
    return buf;
  }
  snprintf(buf, sizeof(buf), "unknown tgdn code %d", code);
  return buf;
}

extern "C" int tgdn_abi_version(void) { return 101; }
extern "C" int tgdn_gate_item_floats(int E) { return tgdn::gate_item_floats(E); }

extern "C" int tgdn_device_status(int* host_status) {
  if (!host_status) return TGDN_ERR_NULL;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  int v = 0, zero = 0;
  e = cudaMemcpyFromSymbol(&v, g_status_word, sizeof(int));
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  e = cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int));
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  *host_status = v;
  return 0;
}
