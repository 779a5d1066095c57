// Forward entry point for callers that have no way to obtain scratch memory.
//
// flexattn_fwd needs a caller-owned workspace for the mask map.  Some hosts cannot provide one: a
// plugin that runs under a memory planner which fixed every device buffer before the program started
// and was given only the operands and results, or a process whose device memory is wholly owned by
// another allocator, so that any allocation made on their behalf would either fail or be invisible to
// that planner.  For them the mask map lives in a fixed array inside this library's device image.
//
// The array is file-scope `static __device__`: every GPU that loads the library holds
// kNoAllocScratchBytes of it until the process exits.  Host code may not use the array's name as a
// pointer (in host code it is only a handle); the device address is looked up once per device with
// cudaGetSymbolAddress, with that device current, and handed to the kernels like any workspace.
#include <mutex>

#include "common.cuh"

namespace flexattn {
namespace {

constexpr size_t kNoAllocScratchBytes = 1u << 20;  // 1 MiB: mask maps up to e.g. S = 32768 with 32 document rows
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// Device address of the array on the current device; nullptr (and *err set) if it cannot be resolved.
void* scratch_for_current_device(cudaError_t* err) {
  static std::mutex mu;
  static void* cache[64] = {};
  int dev = -1;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess) return nullptr;
  if (dev < 0 || dev >= 64) {
    *err = cudaErrorInvalidDevice;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev] == nullptr) {
    void* ptr = nullptr;
    *err = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (*err != cudaSuccess) return nullptr;
    cache[dev] = ptr;
  }
  return cache[dev];
}

}  // namespace
}  // namespace flexattn

using namespace flexattn;

extern "C" size_t flexattn_noalloc_scratch_bytes(void) { return kNoAllocScratchBytes; }

extern "C" int flexattn_fwd_noalloc(void* stream, const FlexAttnParams* p) {
  if (p == nullptr) return FLEXATTN_ERR_NULL_POINTER;
  FlexAttnParams local = *p;
  local.workspace = nullptr;
  local.workspace_bytes = 0;
  const size_t need = flexattn_workspace_bytes(&local);  // 0 = invalid shape / dtype / kinds
  if (need == 0) {
    // let the ordinary validation name the problem (it fails before touching the workspace)
    const int e = flexattn_fwd(stream, &local);
    return e != FLEXATTN_OK ? e : FLEXATTN_ERR_BAD_SHAPE;
  }
  if (need > kNoAllocScratchBytes) return FLEXATTN_ERR_NOALLOC_LIMIT;
  cudaError_t err = cudaSuccess;
  void* scratch = scratch_for_current_device(&err);
  if (scratch == nullptr) return FLEXATTN_ERR_CUDA;
  local.workspace = scratch;
  local.workspace_bytes = kNoAllocScratchBytes;
  // Every check the forward makes runs BEFORE anything is enqueued: a call that is going to be refused (null or
  // misaligned pointer, unsupported backend) must not have overwritten the shared array on its way out.
  bool tc = false;
  int e = validate_fwd_args(&local, &tc);
  if (e != FLEXATTN_OK) return e;
  // The map builder rewrites every word the kernels read (header, row map, column map, per-tile document
  // ranges, the work order of the q tiles and the row-map entries in that order), so nothing left in the
  // array by an earlier call has to be cleared.
  e = flexattn_build_mask_map(stream, &local);
  if (e != FLEXATTN_OK) return e;
  return flexattn_fwd(stream, &local);
}
