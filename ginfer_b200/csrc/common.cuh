// Shared device helpers for the hand-written sm_100a kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#define GF_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes used across the C interface
#define GF_F32 0
#define GF_BF16 1

namespace gf {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
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

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();                      // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

inline int launch_status() { return (int)cudaGetLastError(); }

// ---- programmatic dependent launch -------------------------------------------------------------
// A kernel launched with the attribute may start while its predecessor in the stream still runs;
// it must call pdl_wait() before it reads (or overwrites) anything the predecessor touches, and
// may do independent work first (set-up, loading weights).  pdl_trigger() lets the successor start.
// Launched without the attribute, both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

inline int& pdl_flag() {
  static int enabled = 1;
  return enabled;
}

// cluster > 1 launches thread-block clusters of (1, 1, cluster), or (cluster, 1, 1) with along_x.
template <typename... KArgs, typename... Args>
inline int launch_kernel_cluster_dims(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, int cluster_z, bool along_x,
                                      Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl_flag()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = along_x ? (unsigned)cluster_z : 1;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = along_x ? 1 : (unsigned)cluster_z;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename... KArgs, typename... Args>
inline int launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, int cluster_z, Args... args) {
  return launch_kernel_cluster_dims(kernel, grid, block, smem, stream, cluster_z, false, args...);
}

template <typename... KArgs, typename... Args>
inline int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                         cudaStream_t stream, Args... args) {
  return launch_kernel_cluster_dims(kernel, grid, block, smem, stream, 1, false, args...);
}

}  // namespace gf

// Every library exports this switch for programmatic dependent launch (on by default).
// A kernel's attributes (dynamic shared memory, cluster sizes) belong to a device: `set` runs once
// on each device a launcher is used on.  Returns `set`'s error, -9 for a device that cannot be
// told, else 0.  One object per launcher and attribute set (a function-local static).
struct OncePerDevice {
  static constexpr int kMaxDevices = 64;
  std::mutex lock;
  bool done[kMaxDevices] = {};
  template <typename F>
  int run(F&& set) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -9;
    std::lock_guard<std::mutex> hold(lock);
    if (done[dev]) return 0;
    const cudaError_t e = set();
    if (e != cudaSuccess) return (int)e;
    done[dev] = true;
    return 0;
  }
};

#define GF_DEFINE_PDL_SWITCH \
  GF_EXPORT void gf_set_pdl(int on) { gf::pdl_flag() = on ? 1 : 0; }
