// Host helpers of the tensor-core kernels: TMA tensor-map construction (driver entry point resolved
// through the runtime, so libcuda is not a link-time dependency), the per-device abort word and the per-device
// record of kernels whose dynamic shared-memory limit has been raised.
#include <mutex>

#include "sm100.cuh"

namespace flexattn {

__device__ int g_abort_word = 0;

int* abort_flag_ptr() {
  static std::mutex mu;
  static int* cache[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_abort_word) != cudaSuccess) return nullptr;
    cache[dev] = static_cast<int*>(p);
  }
  return cache[dev];
}

int ensure_dynamic_smem(const void* kernel, int bytes, SmemAttrOnce* once) {
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FLEXATTN_ERR_CUDA;
  std::lock_guard<std::mutex> lock(mu);
  if (!once->done[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
      return FLEXATTN_ERR_CUDA;
    once->done[dev] = 1;
  }
  return FLEXATTN_OK;
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

int make_tile_map(CUtensorMap* out, const void* base, int slices, int rows, int cols) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return FLEXATTN_ERR_CUDA;
  const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)slices};
  const cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)cols * 2 * (cuuint64_t)rows};  // bytes, dims 1..2
  const cuuint32_t box[3] = {64, (cuuint32_t)kTile, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

}  // namespace flexattn
