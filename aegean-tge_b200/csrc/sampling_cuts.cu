// Repetition penalty and the top-k / min-p / top-p cuts of the reference sampler
// (src/models/sampling.cpp:32-54, :183-410), one block per row.
//
// Penalty: every distinct token in the recent history window has its score divided by the
// penalty when positive and multiplied when negative, once however often it occurs.  The kernel
// writes f(original score) for every history position, so duplicates write the same value.
//
// Cuts, in the reference's order: probabilities e_i = exp((z_i - max) / T); candidates ordered by
// probability, highest first (ties: lower index first); top-k keeps the first k; min-p drops what
// is below min_p times the best; the total is what survived; top-p keeps the shortest prefix whose
// share of the total reaches top_p; the draw u scales the kept mass and the walk over the kept
// prefix returns the first candidate at which the running remainder is <= 0.
//
// The order is produced by a bitonic sort of (probability, index) pairs in scratch memory in
// global memory (a power of two >= vocab entries per row, padded with -1); sums over the sorted
// prefix are formed per thread over contiguous chunks and combined in chunk order.
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;

__global__ void penalty_kernel(const float* __restrict__ src, float* __restrict__ dst, long long row_stride,
                               const int* __restrict__ history, const int* __restrict__ history_start,
                               const float* __restrict__ penalty, int vocab) {
  const int row = blockIdx.x;
  const float factor = penalty[row];
  if (!(factor > 0.0f) || factor == 1.0f) return;
  const int begin = history_start[row], end = history_start[row + 1];
  for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const int token = history[i];
    if (token < 0 || token >= vocab) continue;
    const float value = src[(size_t)row * row_stride + token];
    dst[(size_t)row * row_stride + token] = value > 0.0f ? value / factor : value * factor;
  }
}

// (probability desc, index asc): true when a must come before b
__device__ __forceinline__ bool before(float pa, int ia, float pb, int ib) {
  return pa > pb || (pa == pb && ia < ib);
}

__global__ void __launch_bounds__(THREADS) sample_cuts_kernel(
    const float* __restrict__ scores, long long row_stride, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
    const float* __restrict__ uniform, float* __restrict__ sort_prob, int* __restrict__ sort_index, int padded,
    int* __restrict__ out, int vocab) {
  __shared__ float red_value[32];
  __shared__ int red_index[32];
  __shared__ float chunk_sum[THREADS];
  __shared__ float shared_f[4];
  __shared__ int shared_i[4];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* z = scores + (size_t)row * row_stride;
  float* prob = sort_prob + (size_t)row * padded;
  int* index = sort_index + (size_t)row * padded;

  // maximum (first index on ties), as in the plain kernel
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = tid; i < vocab; i += THREADS) {
    const float v = z[i];
    if (v > bv || bi == 0x7fffffff) { bv = v; bi = i; }
  }
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, offset);
    if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
  }
  if (lane == 0) { red_value[warp] = bv; red_index[warp] = bi; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < 32; ++w) {
      const float ov = red_value[w];
      const int oi = red_index[w];
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    shared_f[0] = bv;
    shared_i[0] = bi;
  }
  __syncthreads();
  const float maximum = shared_f[0];
  const int arg_max = shared_i[0];
  const float temp = temperature[row];
  if (!(temp > 0.0f)) {
    if (tid == 0) out[row] = arg_max;
    return;
  }
  const float inverse = 1.0f / temp;
  for (int i = tid; i < padded; i += THREADS) {
    prob[i] = i < vocab ? expf((z[i] - maximum) * inverse) : -1.0f;
    index[i] = i;
  }
  __syncthreads();

  // bitonic sort, descending by (probability, -index)
  for (int size = 2; size <= padded; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = tid; t < (padded >> 1); t += THREADS) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool descending = (lo & size) == 0;
        const float pa = prob[lo], pb = prob[hi];
        const int ia = index[lo], ib = index[hi];
        const bool ordered = before(pa, ia, pb, ib);
        if (ordered != descending) {
          prob[lo] = pb; prob[hi] = pa;
          index[lo] = ib; index[hi] = ia;
        }
      }
      __syncthreads();
    }
  }

  // how many candidates survive top-k and min-p (a prefix of the sorted order)
  int keep = top_k[row] > 0 ? min(top_k[row], vocab) : vocab;
  const float floor_value = min_p[row] > 0.0f ? min_p[row] * prob[0] : -1.0f;
  if (tid == 0) shared_i[1] = keep;
  __syncthreads();
  if (min_p[row] > 0.0f) {
    // first position in [0, keep) whose probability is below the floor
    for (int i = tid; i < keep; i += THREADS)
      if (prob[i] < floor_value && (i == 0 || prob[i - 1] >= floor_value)) atomicMin(&shared_i[1], i);
    __syncthreads();
  }
  keep = shared_i[1];
  if (keep <= 0) {
    if (tid == 0) out[row] = index[0];
    return;
  }

  // chunked prefix sums over the kept prefix, in chunk order
  const int chunk = (keep + THREADS - 1) / THREADS;
  const int begin = min(tid * chunk, keep), end = min(begin + chunk, keep);
  float local = 0.0f;
  for (int i = begin; i < end; ++i) local += prob[i];
  chunk_sum[tid] = local;
  __syncthreads();
  if (tid == 0) {
    float total = 0.0f;
    for (int c = 0; c < THREADS; ++c) total += chunk_sum[c];
    shared_f[1] = total;
    // nucleus: shortest prefix whose share of the total reaches top_p
    int limit = keep;
    const float nucleus = top_p[row];
    if (nucleus < 1.0f && total > 0.0f) {
      float cumulative = 0.0f;
      bool found = false;
      for (int c = 0; c < THREADS && !found; ++c) {
        const int cb = min(c * chunk, keep), ce = min(cb + chunk, keep);
        if ((cumulative + chunk_sum[c]) / total < nucleus && c + 1 < THREADS && ce < keep) {
          cumulative += chunk_sum[c];
          continue;
        }
        for (int i = cb; i < ce; ++i) {
          cumulative += prob[i];
          if (cumulative / total >= nucleus) { limit = i + 1; found = true; break; }
        }
      }
    }
    shared_i[2] = limit;
  }
  __syncthreads();
  const float total = shared_f[1];
  const int limit = shared_i[2];
  if (!(total > 0.0f) || limit <= 0) {
    if (tid == 0) out[row] = index[0];
    return;
  }
  // kept mass and the walk over the kept prefix
  const int chunk2 = (limit + THREADS - 1) / THREADS;
  const int b2 = min(tid * chunk2, limit), e2 = min(b2 + chunk2, limit);
  local = 0.0f;
  for (int i = b2; i < e2; ++i) local += prob[i];
  __syncthreads();
  chunk_sum[tid] = local;
  __syncthreads();
  if (tid == 0) {
    float kept = 0.0f;
    for (int c = 0; c < THREADS; ++c) kept += chunk_sum[c];
    int result = index[0];
    if (kept > 0.0f) {
      float target = uniform[row] * kept;
      result = index[limit - 1];
      bool found = false;
      for (int c = 0; c < THREADS && !found; ++c) {
        const int cb = min(c * chunk2, limit), ce = min(cb + chunk2, limit);
        if (cb >= ce) break;
        if (target - chunk_sum[c] > 0.0f) { target -= chunk_sum[c]; continue; }
        for (int i = cb; i < ce; ++i) {
          target -= prob[i];
          if (target <= 0.0f) { result = index[i]; found = true; break; }
        }
        if (!found) { result = index[ce - 1]; found = true; }
      }
    }
    out[row] = result;
  }
}

}  // namespace

// dst must already hold a copy of src; history is the concatenation of every row's window,
// history_start [rows + 1] its offsets; penalty [rows] (1.0 = off).
TGE_API int tge_apply_penalty(const float* src, float* dst, long long row_stride, const int* history,
                              const int* history_start, const float* penalty, int rows, int vocab,
                              cudaStream_t stream) {
  TGE_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "penalty: bad sizes");
  if (rows == 0) return 0;
  penalty_kernel<<<rows, 256, 0, stream>>>(src, dst, row_stride, history, history_start, penalty, vocab);
  return tge_launched("apply_penalty", 1);
}

TGE_API long long tge_sample_cuts_padded(int vocab) {
  long long padded = 2;
  while (padded < vocab) padded <<= 1;
  return padded;
}

// scratch: sort_prob float32 [rows, padded], sort_index int32 [rows, padded] with padded from tge_sample_cuts_padded.
TGE_API int tge_sample_cuts(const float* scores, long long row_stride, const float* temperature, const int* top_k,
                            const float* top_p, const float* min_p, const float* uniform, float* sort_prob,
                            int* sort_index, int* out, int rows, int vocab, cudaStream_t stream) {
  TGE_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "sample_cuts: bad sizes rows=%d vocab=%d", rows, vocab);
  TGE_REQUIRE(sort_prob != nullptr && sort_index != nullptr, "sample_cuts: needs scratch for the sort");
  if (rows == 0) return 0;
  sample_cuts_kernel<<<rows, THREADS, 0, stream>>>(scores, row_stride, temperature, top_k, top_p, min_p, uniform,
                                                   sort_prob, sort_index, (int)tge_sample_cuts_padded(vocab), out,
                                                   vocab);
  return tge_launched("sample_cuts", 1);
}
