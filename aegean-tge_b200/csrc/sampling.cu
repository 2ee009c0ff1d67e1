// Greedy and temperature sampling over float32 logits: one block per row, or for a large vocabulary a
// cluster of up to eight blocks that exchange their maxima and sums through distributed shared memory.
//
// Rules of the reference sampler (src/models/sampling.cpp:183-228, :72-93;
// src/cpu/scalar/norm_rope_scalar.cpp:53-72):
//  * temperature <= 0: the first index holding the maximum (strict '>' scan);
//  * otherwise e_i = exp((z_i - max) / T), Z = sum e_i, target = u * Z, walk the
//    indices in order subtracting e_i and return the first index where the
//    remainder is <= 0 (the last index if none; index 0 if Z is not positive).
// The uniform u comes from the caller (the request's xorshift32 stream lives
// on the host).  The sum and the walk run in a fixed order that depends on the vocabulary only: the row is
// cut into contiguous ranges, one per block of the cluster, and each range into 32 contiguous segments, one
// per warp; segment totals are added in segment order, and inside the chosen segment the walk advances 32
// indices at a time with a warp prefix sum.
#include <cooperative_groups.h>

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

constexpr int MAX_CLUSTER = 8;

__global__ void __launch_bounds__(1024) sample_kernel(const float* __restrict__ logits, long long row_stride,
                                                      const float* __restrict__ temperature,
                                                      const float* __restrict__ uniform, int* __restrict__ out,
                                                      int vocab, int span) {
  namespace cg = cooperative_groups;
  // what the other blocks of the cluster read: this block's maximum and its 32 segment sums
  __shared__ float best_value[32];
  __shared__ int best_index[32];
  __shared__ float segment_sum[32];
  __shared__ float block_best_value;
  __shared__ int block_best_index;
  __shared__ int chosen_block, chosen_segment;
  __shared__ float chosen_target;
  cg::cluster_group cluster = cg::this_cluster();
  const int blocks = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x / blocks;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* z = logits + (size_t)row * row_stride;
  const int lo = min(rank * span, vocab), hi = min(lo + span, vocab);        // this block's indices (span % 4 == 0)

  // first maximal index of the range
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  // (a thread meets its indices in ascending order, four at a time where the row allows 16-byte loads)
  auto visit = [&](float v, int i) {
    if (v > bv || bi == 0x7fffffff) { bv = v; bi = i; }
  };
  if ((reinterpret_cast<uintptr_t>(z) & 15u) == 0) {
    const int quads = (hi - lo) >> 2;
    const float4* z4 = reinterpret_cast<const float4*>(z + lo);
#pragma unroll 4
    for (int q = tid; q < quads; q += 1024) {
      const float4 v = z4[q];
      visit(v.x, lo + 4 * q);
      visit(v.y, lo + 4 * q + 1);
      visit(v.z, lo + 4 * q + 2);
      visit(v.w, lo + 4 * q + 3);
    }
    for (int i = lo + 4 * quads + tid; i < hi; i += 1024) visit(z[i], i);
  } else {
#pragma unroll 8
    for (int i = lo + tid; i < hi; i += 1024) visit(z[i], i);
  }
  auto better = [](float ov, int oi, float v, int i) {       // (ov, oi) goes before (v, i)
    return oi != 0x7fffffff && (i == 0x7fffffff || ov > v || (ov == v && oi < i));
  };
  auto warp_best = [&]() {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, offset);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
  };
  warp_best();
  if (lane == 0) { best_value[warp] = bv; best_index[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = best_value[lane];
    bi = best_index[lane];
    warp_best();
    if (lane == 0) { block_best_value = bv; block_best_index = bi; }
  }
  cluster.sync();
  // every block works the row's maximum out of all blocks' (the order "larger value, then lower index" is total,
  // so the order of the comparisons does not matter)
  if (warp == 0) {
    bv = -INFINITY;
    bi = 0x7fffffff;
    if (lane < blocks) {
      bv = *cluster.map_shared_rank(&block_best_value, lane);
      bi = *cluster.map_shared_rank(&block_best_index, lane);
    }
    warp_best();
    if (lane == 0) { best_value[0] = bv; best_index[0] = bi; }
  }
  __syncthreads();
  const float maximum = best_value[0];
  const int arg_max = best_index[0];
  const float temp = temperature[row];
  if (!(temp > 0.0f)) {
    if (tid == 0 && rank == 0) out[row] = arg_max;
    cluster.sync();                       // nobody leaves while its shared memory may still be read
    return;
  }

  const float inverse = 1.0f / temp;
  const int segment = ((hi - lo + 31) / 32 + 31) / 32 * 32;  // indices per warp, a multiple of 32
  const int begin = min(lo + warp * segment, hi);
  const int end = min(begin + segment, hi);
  float partial = 0.0f;
#pragma unroll 8
  for (int i = begin + lane; i < end; i += 32) partial += expf((z[i] - maximum) * inverse);
  partial = warp_sum(partial);
  if (lane == 0) segment_sum[warp] = partial;
  cluster.sync();
  if (warp == 0) {
    // All segments of the row, blocks * 32 of them, shared out over the lanes of one warp in order: lane l takes
    // the `per_lane` segments from l * per_lane on.  A lane adds its segments' sums in order, a prefix sum over
    // the lanes gives the total and the lane in which the target falls, and that lane walks its segments.
    const int per_lane = blocks;                              // blocks * 32 segments over 32 lanes
    const float* sums = cluster.map_shared_rank(segment_sum, (lane * per_lane) / 32) + (lane * per_lane) % 32;
    float mine[MAX_CLUSTER];
    float local = 0.0f;
#pragma unroll
    for (int k = 0; k < MAX_CLUSTER; ++k) {
      mine[k] = k < per_lane ? sums[k] : 0.0f;
      local += mine[k];
    }
    const float scan = warp_inclusive_scan(local, lane);
    const float up = __shfl_up_sync(0xffffffffu, scan, 1);
    const float before = lane > 0 ? up : 0.0f;                // the sum of the lanes before this one
    const float total = __shfl_sync(0xffffffffu, scan, 31);
    const float target = uniform[row] * total;
    const bool here = total > 0.0f && target - scan <= 0.0f;
    const unsigned mask = __ballot_sync(0xffffffffu, here);
    if (!(total > 0.0f)) {
      if (lane == 0) { chosen_block = -1; chosen_segment = -1; chosen_target = 0.0f; }
    } else if (mask == 0) {
      if (lane == 0) { chosen_block = blocks; chosen_segment = -1; chosen_target = 0.0f; }      // ran off the end
    } else if (lane == __ffs(mask) - 1) {
      float rest = target - before;                           // what is left when this lane's segments begin
      int pick = -1;
#pragma unroll
      for (int k = 0; k < MAX_CLUSTER; ++k) {
        if (k < per_lane && pick < 0) {
          if (rest - mine[k] <= 0.0f) pick = lane * per_lane + k;
          else rest -= mine[k];
        }
      }
      if (pick < 0) pick = lane * per_lane + per_lane - 1;    // rounding: the lane's last segment
      chosen_block = pick / 32;
      chosen_segment = pick % 32;
      chosen_target = rest;
    }
  }
  cluster.sync();                         // the sums were read; after this nobody reads another block's memory
  const int pick_block = chosen_block, pick = chosen_segment;
  if (pick_block < 0) {
    if (tid == 0 && rank == 0) out[row] = 0;
    return;
  }
  if (pick_block == blocks) {
    if (tid == 0 && rank == 0) out[row] = vocab - 1;
    return;
  }
  if (rank != pick_block || warp != pick) return;
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
  // blocks per row: as many (a power of two, eight at most) as leave each at least 8,192 indices
  int blocks = 1;
  while (blocks < MAX_CLUSTER && vocab / (2 * blocks) >= 8192) blocks *= 2;
  const int span = ((vocab + blocks - 1) / blocks + 3) / 4 * 4;
  const cudaError_t err = tge_launch_clusters(sample_kernel, dim3(rows * blocks), dim3(1024), 0, blocks, stream, logits,
                                              row_stride, temperature, uniform, out, vocab, span);
  TGE_REQUIRE(err == cudaSuccess, "sample: launch failed: %s", cudaGetErrorString(err));
  return tge_launched("sample", 1);
}
