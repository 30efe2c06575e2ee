// Shared helpers for the sm_100a kernels of this package.
//
// Every launcher is an `extern "C"` function that takes raw device pointers, sizes and
// the stream to launch on, validates its arguments, and returns 0 or a negative code
// after recording a message that `ilb_last_error()` of the same library returns.
// Nothing here allocates device memory: callers own every buffer.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <stdlib.h>
#include <utility>

namespace ilb {

static thread_local char g_error[512] = "";

static inline int fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return -1;
}

static inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail("%s: launch failed: %s", what, cudaGetErrorString(e));
  return 0;
}

// Kernel attributes (shared-memory size, cluster size) are kept per device: a launcher asks
// `first()` with the launch's device current and sets them when it answers true.  A
// launcher that fails to set them calls `forget()` so that the next call tries again.
struct OncePerDevice {
  static constexpr int kMax = 64;
  bool done[kMax] = {};
  int last = -1;
  bool first() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMax) { last = -1; return true; }
    last = dev;
    if (done[dev]) return false;
    done[dev] = true;
    return true;
  }
  void forget() { if (last >= 0) done[last] = false; }
};

#define ILB_REQUIRE(cond, ...)            \
  do {                                    \
    if (!(cond)) return ilb::fail(__VA_ARGS__); \
  } while (0)

// Element type codes shared with the Python side.
enum DType : int { kF32 = 0, kBF16 = 1 };

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a thread block of up to 1024 threads; every thread gets the result.
// `scratch` must hold 33 floats of shared memory.  The order of additions is fixed
// by the block size alone.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const int nwarps = (blockDim.x + 31) >> 5;
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// ---------------------------------------------------------------- dependent launches
// Every kernel of this package is launched with programmatic stream serialization: it
// may become resident while the kernel before it in the stream is still running.  The
// contract each kernel keeps: it calls pdl_wait() before it reads or writes anything in
// global memory that an earlier kernel may write or read (kernel parameters and weights
// are free), and it calls pdl_launch_dependents() once letting the next kernel start
// cannot hurt.  pdl_wait() returns when the preceding kernel has completed and its
// writes are visible, so chains of such kernels stay ordered.  ILB_PDL=0 in the
// environment launches everything the ordinary, fully serialized way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("ILB_PDL");
    on = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return on != 0;
}

// cluster_x > 1 launches thread-block clusters of that many consecutive CTAs (grid.x must be
// a multiple of it).
template <typename... KArgs, typename... Args>
static inline void launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  int cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

template <typename... KArgs, typename... Args>
static inline void launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args&&... args) {
  launch_cluster(kernel, grid, block, smem, stream, 1, std::forward<Args>(args)...);
}

}  // namespace ilb

#define ILB_EXPORT extern "C" __attribute__((visibility("default")))

// One copy per library.
#define ILB_DEFINE_LAST_ERROR() \
  ILB_EXPORT const char* ilb_last_error() { return ilb::g_error; }
