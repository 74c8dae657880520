// Shared by every kernel file: element types, widening and narrowing, warp and
// block reductions, and the launch-error convention of the exported functions.
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes and
// a stream, launches without synchronising, and returns a cudaError_t as int
// (0 = launched). Sizes a kernel cannot take are refused with
// cudaErrorInvalidValue before anything is launched; the Python side turns a
// non-zero code into an exception that names the function.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SAKV_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side (ops/_lib.py)
enum : int { SAKV_F32 = 0, SAKV_BF16 = 1 };

constexpr int kCacheBlock = 64;  // tokens per cache block; the Python side asserts the same

__device__ __forceinline__ float widen(float v) { return v; }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T narrow(float v);
template <> __device__ __forceinline__ float narrow<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16>(float v) {
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

// Sum over a block of up to 1024 threads; every thread gets the result. The
// order of the additions depends on the block size only.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int w = 0; w < warps; ++w) total += scratch[w];
    scratch[32] = total;
  }
  __syncthreads();
  return scratch[32];
}

static inline int launch_status() { return static_cast<int>(cudaGetLastError()); }

// Programmatic dependent launch: a kernel launched with `launch_overlapped` may begin
// (set up its shared memory, prefetch constants such as weights) while the kernel before
// it on the stream is still running. It must call `wait_for_previous_kernel()` before it
// reads anything that kernel wrote and before it writes global memory at all; it calls
// `let_next_kernel_start()` at its top so that its own successor can do the same.
__device__ __forceinline__ void wait_for_previous_kernel() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void let_next_kernel_start() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// `cluster`: the thread-block cluster's shape, (1, 1, 1) for none.
template <typename... KernelArgs, typename... Args>
static inline int launch_overlapped_cluster(void (*kernel)(KernelArgs...), dim3 grid, dim3 block,
                                            size_t smem, cudaStream_t stream, dim3 cluster,
                                            Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[3];
  int n = 0;
  attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[n].val.programmaticStreamSerializationAllowed = 1;
  ++n;
  if (cluster.x * cluster.y * cluster.z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster.x;
    attr[n].val.clusterDim.y = cluster.y;
    attr[n].val.clusterDim.z = cluster.z;
    ++n;
    // (the blocks of a cluster are there to pull weights through as many SMs as possible)
    attr[n].id = cudaLaunchAttributeClusterSchedulingPolicyPreference;
    attr[n].val.clusterSchedulingPolicyPreference = cudaClusterSchedulingPolicySpread;
    ++n;
  }
  config.attrs = attr;
  config.numAttrs = n;
  const cudaError_t e = cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
  return e != cudaSuccess ? static_cast<int>(e) : launch_status();
}

template <typename... KernelArgs, typename... Args>
static inline int launch_overlapped(void (*kernel)(KernelArgs...), dim3 grid, dim3 block,
                                    size_t smem, cudaStream_t stream, int cluster_z,
                                    Args&&... args) {
  return launch_overlapped_cluster(kernel, grid, block, smem, stream,
                                   dim3(1, 1, cluster_z > 1 ? cluster_z : 1),
                                   static_cast<Args&&>(args)...);
}

// The number of SMs of the current device, asked once per device (148 on a B200; fewer on
// a part with SMs masked off). Grids and the one-wave reasoning of the launchers use it.
static inline int sm_count() {
  constexpr int kDevices = 64;
  static int known[kDevices] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kDevices) return 148;
  if (known[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0)
      n = 148;
    known[device] = n;
  }
  return known[device];
}

// A kernel's attributes (its opt-in to large dynamic shared memory) belong to a device: a
// launcher keeps one of these per kernel and configures the kernel once on EACH device that
// launches it. `needs()` is true until `done()` was called on the current device.
struct PerDeviceOnce {
  static constexpr int kDevices = 64;
  bool set[kDevices] = {};
  static int current() {
    int device = 0;
    return cudaGetDevice(&device) == cudaSuccess ? device : -1;
  }
  bool needs() const {
    const int d = current();
    return d < 0 || d >= kDevices || !set[d];
  }
  void done() {
    const int d = current();
    if (d >= 0 && d < kDevices) set[d] = true;
  }
};

static inline int grid_for(long long work, int threads, int per_sm = 16) {
  const int cap = sm_count() * per_sm;
  long long blocks = (work + threads - 1) / threads;
  if (blocks < 1) blocks = 1;
  if (blocks > cap) blocks = cap;
  return static_cast<int>(blocks);
}
