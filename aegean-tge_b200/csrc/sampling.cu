// Greedy and temperature sampling over float32 logits, one block per row.
//
// Rules of the reference sampler (src/models/sampling.cpp:183-228, :72-93;
// src/cpu/scalar/norm_rope_scalar.cpp:53-72):
//  * temperature <= 0: the first index holding the maximum (strict '>' scan);
//  * otherwise e_i = exp((z_i - max) / T), Z = sum e_i, target = u * Z, walk the
//    indices in order subtracting e_i and return the first index where the
//    remainder is <= 0 (the last index if none; index 0 if Z is not positive).
// The uniform u comes from the caller (the request's xorshift32 stream lives
// on the host).  The sum and the walk run in a fixed order: the vocabulary is
// cut into 32 contiguous segments, one per warp; segment totals are added in
// segment order, and inside the chosen segment the walk advances 32 indices
// at a time with a warp prefix sum.
#include "common.cuh"

namespace {

__device__ __forceinline__ float warp_inclusive_scan(float v, int lane) {
#pragma unroll
  for (int offset = 1; offset < 32; offset <<= 1) {
    const float other = __shfl_up_sync(0xffffffffu, v, offset);
    if (lane >= offset) v += other;
  }
  return v;
}

__global__ void __launch_bounds__(1024) sample_kernel(const float* __restrict__ logits, long long row_stride,
                                                      const float* __restrict__ temperature,
                                                      const float* __restrict__ uniform, int* __restrict__ out,
                                                      int vocab) {
  __shared__ float best_value[32];
  __shared__ int best_index[32];
  __shared__ float segment_sum[32];
  __shared__ int chosen_segment;
  __shared__ float chosen_target;
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* z = logits + (size_t)row * row_stride;

  // first maximal index
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  // (a thread meets its indices in ascending order, four at a time where the row allows 16-byte loads)
  auto visit = [&](float v, int i) {
    if (v > bv || bi == 0x7fffffff) { bv = v; bi = i; }
  };
  if ((reinterpret_cast<uintptr_t>(z) & 15u) == 0) {
    const int quads = vocab >> 2;
#pragma unroll 4
    for (int q = tid; q < quads; q += 1024) {
      const float4 v = reinterpret_cast<const float4*>(z)[q];
      visit(v.x, 4 * q);
      visit(v.y, 4 * q + 1);
      visit(v.z, 4 * q + 2);
      visit(v.w, 4 * q + 3);
    }
    for (int i = 4 * quads + tid; i < vocab; i += 1024) visit(z[i], i);
  } else {
#pragma unroll 8
    for (int i = tid; i < vocab; i += 1024) visit(z[i], i);
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, offset);
    if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
  }
  if (lane == 0) { best_value[warp] = bv; best_index[warp] = bi; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < 32; ++w) {
      const float ov = best_value[w];
      const int oi = best_index[w];
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    best_value[0] = bv;
    best_index[0] = bi;
  }
  __syncthreads();
  const float maximum = best_value[0];
  const int arg_max = best_index[0];
  const float temp = temperature[row];
  if (!(temp > 0.0f)) {
    if (tid == 0) out[row] = arg_max;
    return;
  }

  const float inverse = 1.0f / temp;
  const int segment = ((vocab + 31) / 32 + 31) / 32 * 32;  // indices per warp, a multiple of 32
  const int begin = warp * segment;
  const int end = min(begin + segment, vocab);
  float partial = 0.0f;
#pragma unroll 8
  for (int i = begin + lane; i < end; i += 32) partial += expf((z[i] - maximum) * inverse);
  partial = warp_sum(partial);
  if (lane == 0) segment_sum[warp] = partial;
  __syncthreads();
  if (tid == 0) {
    float total = 0.0f;
    for (int w = 0; w < 32; ++w) total += segment_sum[w];
    int pick = -1;
    float target = 0.0f;
    if (total > 0.0f) {
      target = uniform[row] * total;
      for (int w = 0; w < 32; ++w) {
        if (w * segment >= vocab) break;
        if (target - segment_sum[w] <= 0.0f) { pick = w; break; }
        target -= segment_sum[w];
      }
      if (pick < 0) pick = 32;  // ran off the end: last index
    }
    chosen_segment = pick;
    chosen_target = target;
  }
  __syncthreads();
  const int pick = chosen_segment;
  if (pick < 0) {
    if (tid == 0) out[row] = 0;
    return;
  }
  if (pick == 32) {
    if (tid == 0) out[row] = vocab - 1;
    return;
  }
  if (warp != pick) return;
  float target = chosen_target;
  int result = -1;
  for (int base = begin; base < end; base += 32) {
    const int i = base + lane;
    const float e = i < end ? expf((z[i] - maximum) * inverse) : 0.0f;
    const float scan = warp_inclusive_scan(e, lane);
    const bool hit = i < end && target - scan <= 0.0f;
    const unsigned mask = __ballot_sync(0xffffffffu, hit);
    if (mask) {
      result = base + __ffs(mask) - 1;
      break;
    }
    target -= __shfl_sync(0xffffffffu, scan, 31);
  }
  if (result < 0) result = end - 1;
  if (lane == 0) out[row] = result;
}

}  // namespace

TGE_API int tge_sample(const float* logits, long long row_stride, const float* temperature, const float* uniform,
                       int* out, int rows, int vocab, cudaStream_t stream) {
  TGE_REQUIRE(rows >= 0 && vocab > 0, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
  TGE_REQUIRE(row_stride >= vocab, "sample: row stride %lld shorter than the vocabulary %d", row_stride, vocab);
  if (rows == 0) return 0;
  tge_launch(sample_kernel, rows, 1024, 0, stream, logits, row_stride, temperature, uniform, out, vocab);
  return tge_launched("sample", 1);
}
