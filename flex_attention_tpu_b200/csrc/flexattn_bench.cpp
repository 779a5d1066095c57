// Stand-alone C++ driver over the C ABI: the counterpart of the reference's only native file, GL_main.cpp
// (GL_main.cpp:12-44: random half-precision Q, K, V of shape B=1, H=4, L=2048, D=128 on the host, one call of
// a host wrapper that copies in, runs the attention kernel, copies out and reports the kernel time).  Here the
// inputs are bfloat16, the kernels are the tcgen05 ones behind libflexattn.so, and the time is the median of
// CUDA-event timings after warm-up.  No torch, no Python: plain CUDA runtime + include/flexattn.h.
//
//   flexattn_bench [--batch 1] [--heads 4] [--seq 2048] [--dim 128] [--causal 0|1] [--bwd 0|1]
//                  [--iters 20] [--warmup 5]
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "flexattn.h"

namespace {

#define CUDA_OK(call)                                                                        \
  do {                                                                                       \
    cudaError_t e_ = (call);                                                                 \
    if (e_ != cudaSuccess) {                                                                 \
      std::fprintf(stderr, "%s failed: %s\n", #call, cudaGetErrorString(e_));                \
      std::exit(2);                                                                          \
    }                                                                                        \
  } while (0)

#define FA_OK(call)                                                                          \
  do {                                                                                       \
    int e_ = (call);                                                                         \
    if (e_ != FLEXATTN_OK) {                                                                 \
      std::fprintf(stderr, "%s failed: %s\n", #call, flexattn_status_string(e_));            \
      std::exit(3);                                                                          \
    }                                                                                        \
  } while (0)

// float -> bfloat16 bits, round to nearest even
uint16_t to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

// uniform [0, 1) like the reference driver's rand() / RAND_MAX, from a fixed-seed generator
struct Lcg {
  uint64_t s;
  float next() {
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    return (float)((s >> 40) & 0xffffff) / 16777216.0f;
  }
};

void* upload_random(size_t n, Lcg& rng, float centre) {
  std::vector<uint16_t> h(n);
  for (size_t i = 0; i < n; ++i) h[i] = to_bf16(rng.next() - centre);
  void* d = nullptr;
  CUDA_OK(cudaMalloc(&d, n * 2));
  CUDA_OK(cudaMemcpy(d, h.data(), n * 2, cudaMemcpyHostToDevice));
  return d;
}

void* dev_alloc(size_t bytes) {
  void* d = nullptr;
  CUDA_OK(cudaMalloc(&d, bytes));
  CUDA_OK(cudaMemset(d, 0, bytes));
  return d;
}

int arg_int(int argc, char** argv, const char* name, int fallback) {
  for (int i = 1; i + 1 < argc; ++i)
    if (std::string(argv[i]) == name) return std::atoi(argv[i + 1]);
  return fallback;
}

template <class F>
float median_ms(F&& run, int warmup, int iters, cudaStream_t st) {
  cudaEvent_t a, b;
  CUDA_OK(cudaEventCreate(&a));
  CUDA_OK(cudaEventCreate(&b));
  for (int i = 0; i < warmup; ++i) run();
  std::vector<float> t(iters);
  for (int i = 0; i < iters; ++i) {
    CUDA_OK(cudaEventRecord(a, st));
    run();
    CUDA_OK(cudaEventRecord(b, st));
    CUDA_OK(cudaEventSynchronize(b));
    CUDA_OK(cudaEventElapsedTime(&t[i], a, b));
  }
  std::sort(t.begin(), t.end());
  CUDA_OK(cudaEventDestroy(a));
  CUDA_OK(cudaEventDestroy(b));
  return t[iters / 2];
}

}  // namespace

int main(int argc, char** argv) {
  const int B = arg_int(argc, argv, "--batch", 1), H = arg_int(argc, argv, "--heads", 4);
  const int L = arg_int(argc, argv, "--seq", 2048), D = arg_int(argc, argv, "--dim", 128);
  const int causal = arg_int(argc, argv, "--causal", 0), bwd = arg_int(argc, argv, "--bwd", 0);
  const int iters = std::max(1, arg_int(argc, argv, "--iters", 20)), warmup = arg_int(argc, argv, "--warmup", 5);
  if (flexattn_abi_version() != FLEXATTN_ABI_VERSION) {
    std::fprintf(stderr, "libflexattn.so ABI %d, header %d\n", flexattn_abi_version(), FLEXATTN_ABI_VERSION);
    return 1;
  }
  const size_t n = (size_t)B * H * L * D, rows = (size_t)B * H * L;
  Lcg rng{12345};
  FlexAttnParams p;
  std::memset(&p, 0, sizeof p);
  p.q = upload_random(n, rng, 0.f);  // the reference driver feeds uniform [0, 1) values
  p.k = upload_random(n, rng, 0.f);
  p.v = upload_random(n, rng, 0.f);
  p.d_o = upload_random(n, rng, 0.5f);
  p.o = dev_alloc(n * 2);
  p.dq = dev_alloc(n * 2);
  p.dk = dev_alloc(n * 2);
  p.dv = dev_alloc(n * 2);
  p.l = (float*)dev_alloc(rows * 4);
  p.m = (float*)dev_alloc(rows * 4);
  p.delta = (float*)dev_alloc(rows * 4);
  p.status = (int32_t*)dev_alloc(16);
  p.batch = B; p.heads = H; p.seq_q = L; p.seq_k = L; p.head_dim = D;
  p.dtype = FLEXATTN_BF16;
  p.sm_scale = 1.0f / std::sqrt((float)D);
  p.score_kind = FLEXATTN_SCORE_NONE;
  p.mask_kind = causal ? FLEXATTN_MASK_CAUSAL : FLEXATTN_MASK_NONE;
  p.backend = FLEXATTN_BACKEND_AUTO;
  p.workspace_bytes = flexattn_workspace_bytes(&p);
  if (p.workspace_bytes == 0) {
    std::fprintf(stderr, "unsupported problem\n");
    return 1;
  }
  p.workspace = dev_alloc(p.workspace_bytes);
  cudaStream_t st;
  CUDA_OK(cudaStreamCreate(&st));
  FA_OK(flexattn_build_mask_map(st, &p));

  const float fwd_ms = median_ms([&] { FA_OK(flexattn_fwd(st, &p)); }, warmup, iters, st);
  float bwd_ms = 0.f;
  if (bwd)
    bwd_ms = median_ms(
        [&] {
          FA_OK(flexattn_bwd_preprocess(st, &p));
          FA_OK(flexattn_bwd_dq(st, &p));
          FA_OK(flexattn_bwd_dkv(st, &p));
        },
        warmup, iters, st);
  CUDA_OK(cudaStreamSynchronize(st));
  int32_t status[4];
  CUDA_OK(cudaMemcpy(status, p.status, 16, cudaMemcpyDeviceToHost));
  if (status[0] != 0) {
    std::fprintf(stderr, "kernel status %d (%s), kernel %d block %d detail %d\n", status[0],
                 flexattn_status_string(status[0]), status[1], status[2], status[3]);
    return 4;
  }
  // a row of O is a convex combination of rows of V, and V is in [0, 1): check one value as a smoke test
  uint16_t o0;
  CUDA_OK(cudaMemcpy(&o0, p.o, 2, cudaMemcpyDeviceToHost));
  uint32_t bits = (uint32_t)o0 << 16;
  float o0f;
  std::memcpy(&o0f, &bits, 4);
  const double pairs = causal ? (double)L * (L + 1) / 2 : (double)L * L;
  const double fwd_flops = 4.0 * B * H * D * pairs, bwd_flops = 10.0 * B * H * D * pairs;
  std::printf("{\"driver\": \"flexattn_bench\", \"shape\": [%d, %d, %d, %d], \"dtype\": \"bf16\", \"causal\": %d, "
              "\"fwd_ms\": %.4f, \"fwd_tflops\": %.1f",
              B, H, L, D, causal, fwd_ms, fwd_flops / (fwd_ms * 1e-3) / 1e12);
  if (bwd) std::printf(", \"bwd_ms\": %.4f, \"bwd_tflops\": %.1f", bwd_ms, bwd_flops / (bwd_ms * 1e-3) / 1e12);
  std::printf(", \"o0\": %.4f}\n", o0f);
  return (o0f >= 0.f && o0f <= 1.f) ? 0 : 5;
}
