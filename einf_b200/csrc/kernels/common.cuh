// Shared helpers of the sm_100a kernels: element types, reductions, launch checks.
//
// Every launcher in this directory is an `extern "C"` function that takes raw
// device pointers, sizes and a stream, launches on that stream and returns the
// cudaError_t of the launch (0 on success).  Shapes are validated by the Python
// wrappers in einf_b200/ops; launchers re-check only what would corrupt memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

namespace einf {

// dtype codes shared with einf_b200/ops/__init__.py (FLOAT32, BFLOAT16)
enum DType : int { kFloat32 = 0, kBFloat16 = 1 };

// Bits of the device status word that kernels set instead of faulting.
enum Status : int {
  kStatusBadToken = 1,      // a token id outside the embedding table
  kStatusBadPage = 2,       // a block-table entry outside the page pool
  kStatusWaitExpired = 4,   // a bounded wait on a barrier gave up
};

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats of shared memory.  The order of additions depends
// only on the block size, never on other rows of the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < warps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < warps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Programmatic dependent launch: a kernel launched with the attribute may become resident
// while kernels before it on the stream still run.  The rules every kernel here keeps:
//  - Before pdl_wait() a thread reads only what no kernel of the step writes (weights, the
//    step's own inputs such as positions and block tables, keys and values of earlier steps)
//    and writes nothing to global memory.
//  - Every kernel calls pdl_wait() (at least one thread, before anything is written), so that
//    "the kernel before me is complete" carries back along the whole chain.
//  - pdl_launch_dependents() comes as early as possible, so that the next kernel's launch
//    latency and prologue hide behind this kernel; but a kernel that allocates tensor memory
//    calls it only after the allocation: a resident kernel holds its columns until it ends,
//    and an earlier kernel must never wait for columns that a later one holds.  A kernel that
//    writes step inputs in place (advance_decode) does not call it at all: its successors read
//    those inputs before their own wait.
// Both calls are no-ops for an ordinary launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Launch with the programmatic-dependent-launch attribute: the grid may be scheduled
// while the kernel before it on the stream drains.  Every kernel launched this way
// calls pdl_wait() before it touches memory another kernel may have written.
// EINF_B200_PDL=0 in the environment turns the attribute off.
inline bool pdl_enabled() {
  static const bool enabled = [] {
    const char* value = getenv("EINF_B200_PDL");
    return !(value && value[0] == '0');
  }();
  return enabled;
}

template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

// The same with the CTAs along x grouped into thread-block clusters of `cluster` (a divisor of grid.x).
template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, int cluster,
                                      cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = cluster;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

// Thread-block clusters: rank and size along x, a barrier over the whole cluster, and a read of a
// float at the same shared-memory offset in another CTA of the cluster.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_peer(float* local, uint32_t rank, float v) {
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(local));
  uint32_t peer;
  asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(addr), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(peer), "f"(v) : "memory");
}

#define EINF_DISPATCH_2(code, NAME, ...)                         \
  if ((code) == einf::kFloat32) {                                \
    using NAME = float;                                          \
    __VA_ARGS__                                                  \
  } else {                                                       \
    using NAME = __nv_bfloat16;                                  \
    __VA_ARGS__                                                  \
  }

}  // namespace einf
