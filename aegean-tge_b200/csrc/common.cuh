// Shared helpers for the sm_100a kernels of this engine.
//
// Conventions every kernel file follows:
//  * entry points are extern "C", take raw device pointers plus a cudaStream_t,
//    validate their arguments on the host and return 0 or a negative code after
//    storing a message readable through tge_last_error();
//  * a kernel that can meet a bad index (token id, page id) does not touch
//    memory with it: it records the fault in a caller-supplied status word and
//    skips the access, so a bad input never becomes a memory fault;
//  * statistics (norm sums, softmax, rotation, residual sums) are float32.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TGE_API extern "C" __attribute__((visibility("default")))

// Status word bits set by kernels (one int32 in device memory, owned by the caller).
enum TgeStatusBits : int {
  TGE_STATUS_BAD_TOKEN = 1,      // token id outside the vocabulary
  TGE_STATUS_BAD_PAGE = 2,       // page id outside the pool
  TGE_STATUS_BAD_ROW = 4,        // row index outside the batch
  TGE_STATUS_WAIT_TIMEOUT = 8,   // a bounded device-side wait gave up
};

void tge_set_error(const char* fmt, ...);
// 0 when the last launch was accepted, a negative code (message stored) otherwise
int tge_check_launch(const char* what);
// Entry points return the number of kernels they launched (>= 0) or a negative code.
inline int tge_launched(const char* what, int kernels) {
  const int rc = tge_check_launch(what);
  return rc != 0 ? rc : kernels;
}
constexpr int TGE_UNSUPPORTED = -100;  // shape outside what the kernel takes; nothing was touched

#define TGE_REQUIRE(cond, ...)            \
  do {                                    \
    if (!(cond)) {                        \
      tge_set_error(__VA_ARGS__);         \
      return -1;                          \
    }                                     \
  } while (0)

// Programmatic dependent launch.  A kernel calls pdl_trigger() as its first statement (the next kernel in
// the stream may then be scheduled and run its own set-up) and pdl_wait() before it first touches global
// memory that an earlier kernel writes or reads: the wait returns once the preceding kernel has finished
// and its writes are visible.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// True in exactly one lane of a converged warp.  A role that one thread plays is entered through this and
// not through `lane == 0`: the compiler then knows the region to be uniform and keeps the addresses and
// descriptors of the TMA and tcgen05 instructions in uniform registers (measured: the one-SM products of a
// 2,048-token prefill 2-9 % faster, the decode products 3-4 %, the two-SM products 4-13 %).
__device__ __forceinline__ bool elect_one() {
  uint32_t chosen;
  asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(chosen));
  return chosen != 0;
}

// The index of the calling warp in its block, in a form the compiler knows to be the same in all its lanes
// (a broadcast from lane 0), so that branches on a warp's role and addresses derived from it stay uniform.
__device__ __forceinline__ int uniform_warp_index() { return __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0); }

bool tge_pdl_enabled();
// Streaming multiprocessors of the current device (asked once).
int tge_sm_count();

// Launches `kernel` so that it may start while its predecessor in the stream drains (see above).
template <typename... KernelArgs, typename... Args>
inline cudaError_t tge_launch(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = tge_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, KernelArgs(args)...);
}

// The same for a kernel whose blocks run as clusters of `cluster` along x (the grid a multiple of it).
template <typename... KernelArgs, typename... Args>
inline cudaError_t tge_launch_clusters(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, int cluster,
                                       cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = cluster;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = tge_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&config, kernel, KernelArgs(args)...);
}

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
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Sum over a block in a fixed order: a butterfly inside each warp, then the
// warp totals added in warp order by every thread.  `scratch` holds 32 floats.
// Sum over the block (up to 32 warps; scratch holds 32 floats).  Every thread gets the same value: the warps'
// sums are combined by one butterfly in every warp, in an order that depends on nothing but the block size.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  return warp_sum(lane < warps ? scratch[lane] : 0.0f);
}
