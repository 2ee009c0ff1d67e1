// The bfloat16 product for callers that cannot allocate device memory.
//
// Who that is: a host program that has handed every byte of device memory it
// is allowed to use to its own pools before it loads this library (an
// inference server that sizes its page pool from "all that is free"), or one
// that runs under a memory quota where any further cudaMalloc fails; and code
// that must not synchronise the device, since cudaMalloc and cudaFree do.  The
// regular entry point tge_gemm_tcgen05 expects such a caller to bring a float32
// scratch buffer for the partial sums of its k-splits.  This variant brings its
// own: a fixed array inside the library image, so the call allocates nothing -
// no cudaMalloc, no cudaFree, no allocating library routine.
//
// The price and the rules:
//  * every GPU that loads the library holds the array (16 MiB) until the
//    process exits, whether or not this entry point is ever called;
//  * a product whose k-splits would need more than TGE_STATIC_SCRATCH_FLOATS
//    partial sums is refused with a message that names both numbers; nothing is
//    launched in that case.  (The regular entry point is the one to use for
//    larger shapes.)
//  * the first call on a device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current) and keeps it; make that
//    first call before any stream capture begins, because the look-up is not
//    a stream operation.  Host threads that make their first calls at the same
//    moment each look the address up and store the same value, which is
//    harmless; nothing else about the entry point is shared between threads;
//  * all calls share the one array and it keeps whatever the last call left in
//    it.  Nothing in it has to start at zero: every partial sum that the
//    reduction reads was written by the same call's product kernel first.  Two
//    calls that overlap on the GPU (different streams, or graph branches that
//    run side by side) would write the same array and race: keep calls in
//    stream order.
#include "gemm_static_scratch.h"

#include "common.cuh"

extern "C" int tge_gemm_tcgen05(const void* x, long long ldx, const void* w, long long ldw, const float* bias,
                                void* out, long long ldo, int M, int N, int K, int epilogue, float* scratch,
                                long long scratch_floats, int force_bn, int force_splits, int* status,
                                const float* x_ss, int x_ss_slices, int x_ss_width, float x_ss_eps,
                                cudaStream_t stream);
extern "C" long long tge_gemm_tcgen05_scratch_floats(int M, int N, int K);

// The scratch itself.  In host code this name is only a handle for the runtime's symbol
// table, not a device address: the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_static_scratch[TGE_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_scratch_address[MAX_DEVICES] = {nullptr};
}  // namespace

TGE_API int tge_gemm_tcgen05_static_scratch(const void* x, long long ldx, const void* w, long long ldw,
                                            const float* bias, void* out, long long ldo, int M, int N, int K,
                                            int epilogue, int* status, cudaStream_t stream) {
  TGE_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm (static scratch): bad sizes M=%d N=%d K=%d", M, N, K);
  const long long need = tge_gemm_tcgen05_scratch_floats(M, N, K);
  TGE_REQUIRE(need <= (long long)TGE_STATIC_SCRATCH_FLOATS,
              "gemm (static scratch): M=%d N=%d K=%d would keep %lld partial sums, the built-in buffer holds %lld; "
              "use tge_gemm_tcgen05 with a buffer of your own",
              M, N, K, need, (long long)TGE_STATIC_SCRATCH_FLOATS);
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  TGE_REQUIRE(err == cudaSuccess, "gemm (static scratch): cudaGetDevice failed: %s", cudaGetErrorString(err));
  TGE_REQUIRE(device >= 0 && device < MAX_DEVICES, "gemm (static scratch): device index %d out of range", device);
  if (g_scratch_address[device] == nullptr) {
    // once per device, with that device current
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, g_static_scratch);
    TGE_REQUIRE(err == cudaSuccess && address != nullptr,
                "gemm (static scratch): cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
    g_scratch_address[device] = static_cast<float*>(address);
  }
  return tge_gemm_tcgen05(x, ldx, w, ldw, bias, out, ldo, M, N, K, epilogue, g_scratch_address[device],
                          (long long)TGE_STATIC_SCRATCH_FLOATS, 0, 0, status, nullptr, 0, 0, 0.0f, stream);
}
