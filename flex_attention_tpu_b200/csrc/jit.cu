// Run-time compilation of the tensor-core kernels around a user score function.
//
// The reference lets a user pass any Python score function: make_jax_score_fn (util.py:150-189) rewrites it into
// code the Pallas kernels inline (flex_attention_kernel.py:248-255), and jax.vjp differentiates it inside the
// backward kernels (flex_attention_dq_bwd.py:340-345,373-380).  The counterpart here: the host side hands over the
// function and its derivative as two CUDA expressions (flexattn_user_score_create); the first launch that needs
// them compiles the SAME kernel source the ahead-of-time build uses - embedded in the library as text - with NVRTC,
// with the expressions substituted for the header user_score.cuh and the score kind fixed to FLEXATTN_SCORE_USER,
// loads the resulting cubin through the driver and caches the function per (handle, kernel, head_dim, mask kind,
// device).  NVRTC is opened with dlopen at first use and the driver entry points are resolved through the runtime,
// so the library links against neither.
#include <dlfcn.h>
#include <cuda.h>

#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "common.cuh"

namespace flexattn {

// kernel sources as text (generated at build time from the files of this directory)
extern const char* const kEmbeddedNames[];
extern const char* const kEmbeddedSources[];
extern const int kEmbeddedCount;

namespace {

// ------------------------------------------------------------------ NVRTC, opened at first use
struct Nvrtc {
  using Program = void*;
  int (*CreateProgram)(Program*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
  int (*DestroyProgram)(Program*) = nullptr;
  int (*CompileProgram)(Program, int, const char* const*) = nullptr;
  int (*GetProgramLogSize)(Program, size_t*) = nullptr;
  int (*GetProgramLog)(Program, char*) = nullptr;
  int (*GetCUBINSize)(Program, size_t*) = nullptr;
  int (*GetCUBIN)(Program, char*) = nullptr;
  int (*AddNameExpression)(Program, const char*) = nullptr;
  int (*GetLoweredName)(Program, const char*, const char**) = nullptr;
  bool ok = false;
};

const Nvrtc& nvrtc() {
  static Nvrtc n = [] {
    Nvrtc r;
    void* lib = nullptr;
    for (const char* name : {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                             "/usr/local/cuda/lib64/libnvrtc.so"}) {
      lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (lib != nullptr) break;
    }
    if (lib == nullptr) return r;
    bool all = true;
    auto sym = [&](auto& fn, const char* name) {
      fn = reinterpret_cast<std::remove_reference_t<decltype(fn)>>(dlsym(lib, name));
      all = all && fn != nullptr;
    };
    sym(r.CreateProgram, "nvrtcCreateProgram");
    sym(r.DestroyProgram, "nvrtcDestroyProgram");
    sym(r.CompileProgram, "nvrtcCompileProgram");
    sym(r.GetProgramLogSize, "nvrtcGetProgramLogSize");
    sym(r.GetProgramLog, "nvrtcGetProgramLog");
    sym(r.GetCUBINSize, "nvrtcGetCUBINSize");
    sym(r.GetCUBIN, "nvrtcGetCUBIN");
    sym(r.AddNameExpression, "nvrtcAddNameExpression");
    sym(r.GetLoweredName, "nvrtcGetLoweredName");
    r.ok = all;
    return r;
  }();
  return n;
}

// ------------------------------------------------------------------ driver entry points, through the runtime
struct Driver {
  CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*ModuleUnload)(CUmodule) = nullptr;
  CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                           void**, void**) = nullptr;
  bool ok = false;
};

const Driver& driver() {
  static Driver d = [] {
    Driver r;
    bool all = true;
    auto sym = [&](auto& fn, const char* name) {
      void* p = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
        p = nullptr;
      fn = reinterpret_cast<std::remove_reference_t<decltype(fn)>>(p);
      all = all && fn != nullptr;
    };
    sym(r.ModuleLoadData, "cuModuleLoadData");
    sym(r.ModuleUnload, "cuModuleUnload");
    sym(r.ModuleGetFunction, "cuModuleGetFunction");
    sym(r.FuncSetAttribute, "cuFuncSetAttribute");
    sym(r.LaunchKernel, "cuLaunchKernel");
    r.ok = all;
    return r;
  }();
  return d;
}

// ------------------------------------------------------------------ registry
struct Compiled {
  std::vector<char> cubin;
  std::string lowered;  // mangled name of the kernel inside the cubin
};
struct Loaded {
  CUmodule module = nullptr;
  CUfunction fn = nullptr;
  size_t smem_set = 0;
};
struct UserScore {
  std::string score, dscore, log;
  std::map<std::tuple<int, int, int>, Compiled> compiled;     // (which, head_dim, mask)
  std::map<std::tuple<int, int, int, int>, Loaded> loaded;    // (which, head_dim, mask, device)
  bool alive = true;
};

std::mutex g_mu;
std::vector<std::unique_ptr<UserScore>> g_scores;  // handle = index + 1

UserScore* find(int handle) {
  if (handle < 1 || handle > (int)g_scores.size()) return nullptr;
  UserScore* u = g_scores[handle - 1].get();
  return u->alive ? u : nullptr;
}

constexpr int kKernels = 4;  // forward (persistent), dQ, dK/dV, forward for long rows
const char* const kKernelFile[kKernels] = {"fwd_pipe_sm100.cu", "bwd_dq_sm100.cu", "bwd_dkv_sm100.cu", "fwd_pair_sm100.cu"};
const char* const kKernelName[kKernels] = {"fwd_pipe_sm100_kernel", "dq_sm100_kernel", "dkv_sm100_kernel", "fwd_pair_sm100_kernel"};

const char* embedded(const char* name) {
  for (int i = 0; i < kEmbeddedCount; ++i)
    if (std::string(kEmbeddedNames[i]) == name) return kEmbeddedSources[i];
  return nullptr;
}

// Compiles kernel `which` for (head_dim, mask) around the handle's expressions.  Caller holds g_mu.
int compile_locked(UserScore* u, int which, int head_dim, int mask, const Compiled** out) {
  const auto key = std::make_tuple(which, head_dim, mask);
  auto it = u->compiled.find(key);
  if (it != u->compiled.end()) {
    *out = &it->second;
    return FLEXATTN_OK;
  }
  const Nvrtc& n = nvrtc();
  if (!n.ok) return FLEXATTN_ERR_JIT_UNAVAILABLE;
  const char* src = embedded(kKernelFile[which]);
  if (src == nullptr) return FLEXATTN_ERR_JIT_UNAVAILABLE;
  const std::string user_header =
      "#pragma once\nnamespace flexattn {\n"
      "__device__ __forceinline__ float user_score(float s, int b, int h, int i, int j) { return (" + u->score + "); }\n"
      "__device__ __forceinline__ float user_dscore(float s, int b, int h, int i, int j) { return (" + u->dscore + "); }\n"
      "}  // namespace flexattn\n";
  // the headers the kernel files include, by the names they include them under
  const char* inc_names[] = {"sched.cuh", "sm100.cuh", "common.cuh", "../../include/flexattn.h", "user_score.cuh"};
  const char* inc_src[] = {embedded("sched.cuh"), embedded("sm100.cuh"), embedded("common.cuh"), embedded("flexattn.h"),
                           user_header.c_str()};
  for (const char* s : inc_src)
    if (s == nullptr) return FLEXATTN_ERR_JIT_UNAVAILABLE;
  Nvrtc::Program prog = nullptr;
  if (n.CreateProgram(&prog, src, kKernelFile[which], 5, inc_src, inc_names) != 0) return FLEXATTN_ERR_JIT_COMPILE;
  const std::string expr = std::string("flexattn::jit_tu::") + kKernelName[which] + "<" + std::to_string(head_dim) + ", " +
                           std::to_string((int)FLEXATTN_SCORE_USER) + ", " + std::to_string(mask) + ">";
#ifdef FLEXATTN_DEBUG
  const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-DFLEXATTN_JIT=1", "-default-device", "-DFLEXATTN_DEBUG=1"};
#else
  const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-DFLEXATTN_JIT=1", "-default-device"};
#endif
  int rc = n.AddNameExpression(prog, expr.c_str());
  if (rc == 0) rc = n.CompileProgram(prog, (int)(sizeof(opts) / sizeof(opts[0])), opts);
  size_t log_size = 0;
  u->log.clear();
  if (n.GetProgramLogSize(prog, &log_size) == 0 && log_size > 1) {
    u->log.resize(log_size);
    n.GetProgramLog(prog, &u->log[0]);
  }
  Compiled c;
  if (rc == 0) {
    const char* lowered = nullptr;
    size_t size = 0;
    if (n.GetLoweredName(prog, expr.c_str(), &lowered) == 0 && lowered != nullptr && n.GetCUBINSize(prog, &size) == 0 &&
        size > 0) {
      c.lowered = lowered;
      c.cubin.resize(size);
      if (n.GetCUBIN(prog, c.cubin.data()) != 0) rc = -1;
    } else {
      rc = -1;
    }
  }
  n.DestroyProgram(&prog);
  if (rc != 0) return FLEXATTN_ERR_JIT_COMPILE;
  *out = &(u->compiled[key] = std::move(c));
  return FLEXATTN_OK;
}

}  // namespace

int jit_launch(int which, int handle, int head_dim, int mask, unsigned grid_x, unsigned grid_y, unsigned threads,
               size_t smem_bytes, cudaStream_t st, void** args) {
  if (which < 0 || which >= kKernels) return FLEXATTN_ERR_UNSUPPORTED_MOD;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return FLEXATTN_ERR_CUDA;
  const Driver& d = driver();
  if (!d.ok) return FLEXATTN_ERR_JIT_UNAVAILABLE;
  CUfunction fn = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    UserScore* u = find(handle);
    if (u == nullptr) return FLEXATTN_ERR_UNSUPPORTED_MOD;
    Loaded& L = u->loaded[std::make_tuple(which, head_dim, mask, dev)];
    if (L.fn == nullptr) {
      const Compiled* c = nullptr;
      const int e = compile_locked(u, which, head_dim, mask, &c);
      if (e != FLEXATTN_OK) return e;
      if (cudaFree(nullptr) != cudaSuccess) return FLEXATTN_ERR_CUDA;  // the runtime's context is current from here on
      if (d.ModuleLoadData(&L.module, c->cubin.data()) != CUDA_SUCCESS) return FLEXATTN_ERR_CUDA;
      if (d.ModuleGetFunction(&L.fn, L.module, c->lowered.c_str()) != CUDA_SUCCESS) {
        d.ModuleUnload(L.module);
        L = Loaded{};
        return FLEXATTN_ERR_CUDA;
      }
    }
    if (L.smem_set < smem_bytes) {
      if (d.FuncSetAttribute(L.fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)smem_bytes) != CUDA_SUCCESS)
        return FLEXATTN_ERR_CUDA;
      L.smem_set = smem_bytes;
    }
    fn = L.fn;
  }
  const CUresult r = d.LaunchKernel(fn, grid_x, grid_y, 1, threads, 1, 1, (unsigned)smem_bytes,
                                    reinterpret_cast<CUstream>(st), args, nullptr);
  return r == CUDA_SUCCESS ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

}  // namespace flexattn

using namespace flexattn;

extern "C" int flexattn_user_score_create(const char* score_expr, const char* dscore_expr, int32_t* handle) {
  if (score_expr == nullptr || dscore_expr == nullptr || handle == nullptr) return FLEXATTN_ERR_NULL_POINTER;
  if (score_expr[0] == '\0' || dscore_expr[0] == '\0') return FLEXATTN_ERR_UNSUPPORTED_MOD;
  std::lock_guard<std::mutex> lock(g_mu);
  auto u = std::make_unique<UserScore>();
  u->score = score_expr;
  u->dscore = dscore_expr;
  g_scores.push_back(std::move(u));
  *handle = (int32_t)g_scores.size();
  return FLEXATTN_OK;
}

extern "C" int flexattn_user_score_destroy(int32_t handle) {
  std::lock_guard<std::mutex> lock(g_mu);
  UserScore* u = find(handle);
  if (u == nullptr) return FLEXATTN_ERR_UNSUPPORTED_MOD;
  const Driver& d = driver();
  for (auto& kv : u->loaded)
    if (kv.second.module != nullptr && d.ok) d.ModuleUnload(kv.second.module);
  u->loaded.clear();
  u->compiled.clear();
  u->alive = false;
  return FLEXATTN_OK;
}

extern "C" const char* flexattn_user_score_log(int32_t handle) {
  std::lock_guard<std::mutex> lock(g_mu);
  UserScore* u = find(handle);
  return u == nullptr ? "" : u->log.c_str();
}

extern "C" int flexattn_user_score_compile(int32_t handle, int which, int32_t head_dim, int32_t mask_kind) {
  if (which < 0 || which >= kKernels) return FLEXATTN_ERR_UNSUPPORTED_MOD;
  if (head_dim != 64 && head_dim != 128) return FLEXATTN_ERR_UNSUPPORTED_HEAD_DIM;
  if (mask_kind < FLEXATTN_MASK_NONE || mask_kind > FLEXATTN_MASK_S2) return FLEXATTN_ERR_UNSUPPORTED_MOD;
  std::lock_guard<std::mutex> lock(g_mu);
  UserScore* u = find(handle);
  if (u == nullptr) return FLEXATTN_ERR_UNSUPPORTED_MOD;
  const Compiled* c = nullptr;
  return compile_locked(u, which, head_dim, mask_kind, &c);
}
