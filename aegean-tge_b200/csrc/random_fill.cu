// Random weights drawn on the device: one thread per pair of neighbouring elements, values from
// random_weights.h, so a 32B-parameter model is filled in the time it takes to write it.
// The same values come from the host loop in runtime.cpp and from the tests' own restatement.
#include "common.cuh"
#include "random_weights.h"

template <typename T>
__global__ void random_fill_kernel(T* __restrict__ out, long long count, long long first, uint64_t key, int kind,
                                   float scale, int base, unsigned int span) {
  const long long pairs = (count + 1) / 2;
  for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < pairs; p += (long long)gridDim.x * blockDim.x) {
    float value[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint64_t index = (uint64_t)(first + 2 * p + j);
      value[j] = kind == TGE_RANDOM_NORMAL
                     ? __fmul_rn(__int2float_rn(tge_rw_normal_int(key, index)), scale)
                     : __fmul_rn(__int2float_rn(tge_rw_uniform_int(key, index, base, span)), 5.9604644775390625e-08f);
    }
    const long long i = 2 * p;
    if (i + 1 < count && (reinterpret_cast<uintptr_t>(out + i) % (2 * sizeof(T))) == 0) {
      if constexpr (sizeof(T) == 2) {
        *reinterpret_cast<__nv_bfloat162*>(out + i) = __floats2bfloat162_rn(value[0], value[1]);
      } else {
        *reinterpret_cast<float2*>(out + i) = make_float2(value[0], value[1]);
      }
    } else {
      out[i] = from_float<T>(value[0]);
      if (i + 1 < count) out[i + 1] = from_float<T>(value[1]);
    }
  }
}

// Fills out[0..count) with elements first..first+count of the tensor whose key is `key`.
// kind 0: normal, value = float(int) * scale.  kind 1: uniform, value = float(base + (u32 * span >> 32)) * 2^-24.
TGE_API int tge_random_fill(void* out, int is_bf16, long long count, long long first, unsigned long long key, int kind,
                            float scale, int base, unsigned int span, cudaStream_t stream) {
  TGE_REQUIRE(count >= 0 && first >= 0, "random_fill: bad range first=%lld count=%lld", first, count);
  TGE_REQUIRE(kind == TGE_RANDOM_NORMAL || kind == TGE_RANDOM_UNIFORM, "random_fill: unknown kind %d", kind);
  if (count == 0) return 0;
  const long long pairs = (count + 1) / 2;
  const int threads = 256;
  const long long want = (pairs + threads - 1) / threads;
  const long long most = (long long)tge_sm_count() * 16;
  const int blocks = (int)(want < most ? want : most);
  if (is_bf16)
    random_fill_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16*)out, count, first, key, kind, scale, base, span);
  else
    random_fill_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, count, first, key, kind, scale, base, span);
  return tge_launched("random_fill", 1);
}
