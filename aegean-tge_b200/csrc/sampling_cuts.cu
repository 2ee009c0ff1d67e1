// Repetition penalty and the top-k / min-p / top-p cuts of the reference sampler
// (src/models/sampling.cpp:32-54, :183-410): one block per row, or for a large vocabulary a cluster of up to
// eight blocks that share the passes over the row and hand their candidates to the first of them.
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
// Only a prefix of the order is ever walked, and with the distributions a language model makes it is short
// (a top-k of tens, a nucleus of hundreds among 150,000 tokens).  So the kernel first narrows a threshold on the
// probabilities' bit patterns in three counting passes (ten coarse levels 2^-4, 2^-8, ... of the best while the
// probabilities are computed; then the four exponents of the level; then eight steps of the mantissa), each time
// taking the highest threshold whose candidates are certain to contain the prefix (they hold the top k; or their
// mass reaches the nucleus's share of the total; or they are all that min-p keeps), gathers the candidates, at
// most 16,384, into shared memory and sorts those.  A row whose prefix cannot be bounded that way (a flat distribution under
// top-p) takes the old way: a bitonic sort of all (probability, index) pairs in scratch memory in global memory
// (a power of two >= vocab entries per row, padded with -1).  Sums over the sorted prefix are formed per thread
// over contiguous chunks of sixteen candidates and combined in chunk order, whatever the number of candidates;
// the total that top-p's share refers to is added as integers (see Units); the float32 masses of the counting
// passes only bound the candidates, with a hair to spare.  So a row's token depends on nothing but its inputs:
// not on the batch, and not on how many blocks shared the row.
//
// With several blocks per row each scans a contiguous range of the row; after a pass every block leaves its
// counts and masses in shared memory, a cluster barrier follows, and every block adds all blocks' figures
// through distributed shared memory, so that all of them take the same decisions without a word from anybody.
// The candidates are gathered per block and copied into the first block, which sorts and walks.
#include <cooperative_groups.h>

#include "common.cuh"

namespace {

constexpr int THREADS = 1024;
constexpr int LEVELS = 10;              // coarse thresholds 2^-4, 2^-8, ... 2^-40 of the best probability
constexpr int BINS = 8;                 // bins of a refinement pass
constexpr int CANDIDATES = 16384;       // most candidates sorted in shared memory (128 KB)
constexpr int MAX_CLUSTER = 8;

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

// A probability is at most 1, so its bit pattern orders like its value.  exponents_below(pr) = d with pr in
// [2^-d, 2^(1-d)); the coarse level of d is 0 for d <= 4, 1 for d <= 8, ...
__device__ __forceinline__ int exponents_below(float pr) { return 127 - (int)((__float_as_uint(pr) >> 23) & 255u); }
__device__ __forceinline__ int level_of_exponent(int d) { return d <= 0 ? 0 : (d - 1) / 4; }

// Calls visit(value, index) for every element of data[0, n), each thread of the block taking every 1024th group of
// four (16-byte loads when the row starts on a 16-byte boundary, which keeps four times as many bytes in flight).
template <typename Visit>
__device__ __forceinline__ void for_each_element(const float* __restrict__ data, int n, Visit visit) {
  const int tid = threadIdx.x;
  if ((reinterpret_cast<uintptr_t>(data) & 15u) == 0) {
    const int quads = n >> 2;
#pragma unroll 4
    for (int q = tid; q < quads; q += THREADS) {
      const float4 v = reinterpret_cast<const float4*>(data)[q];
      visit(v.x, 4 * q);
      visit(v.y, 4 * q + 1);
      visit(v.z, 4 * q + 2);
      visit(v.w, 4 * q + 3);
    }
    for (int i = 4 * quads + tid; i < n; i += THREADS) visit(data[i], i);
  } else {
#pragma unroll 8
    for (int i = tid; i < n; i += THREADS) visit(data[i], i);
  }
}

// What the walk needs of the candidates above a threshold: enough of them for the top-k, or enough mass for the
// nucleus's share of the total (with a hair to spare: the sums here and in the walk are formed in different orders).
// The mass of everything min-p keeps is the total that top-p's share refers to, so it must not depend on who added
// what in which order: it is added as integers, in units of 2^-40 of the best probability (which is 1).  What a
// probability below 2^-16 loses in the conversion is below 2^-40, 1.4e-7 of the best for a whole vocabulary of
// 150,000.  (The masses of levels and bins only bound the candidates, with a hair to spare; they stay float32.)
typedef unsigned long long Units;
__device__ __forceinline__ Units units_of(float pr) { return __float2ull_rz(pr * 1099511627776.0f); }
__device__ __forceinline__ float units_value(Units m) { return (float)m * (1.0f / 1099511627776.0f); }

struct Need {
  int k_wanted;          // 0: no top-k
  float share;           // top-p (>= 1: none)
  float kept_mass;       // of everything min-p keeps
  int kept_count;
  __device__ bool met(int count, float mass) const {
    if (count == kept_count) return true;                  // everything that is kept at all
    if (k_wanted > 0) return count >= k_wanted;
    return share < 1.0f && mass >= share * kept_mass * 1.00001f;
  }
};

// Block-wide sums of BINS (or LEVELS) counts and masses in a fixed order: a butterfly in each warp, then the
// warps in warp order.  Results land in row 0 of the two arrays.
template <int N>
__device__ __forceinline__ void block_sums(float (&mass)[N], int (&count)[N], float (*red_mass)[LEVELS + 1],
                                           int (*red_count)[LEVELS + 1]) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __syncthreads();                                   // earlier readers of the arrays are done
#pragma unroll
  for (int l = 0; l < N; ++l) {
    mass[l] = warp_sum(mass[l]);
    count[l] = __reduce_add_sync(0xffffffffu, count[l]);
  }
  if (lane == 0) {
#pragma unroll
    for (int l = 0; l < N; ++l) { red_mass[warp][l] = mass[l]; red_count[warp][l] = count[l]; }
  }
  __syncthreads();
  if (tid < N) {
    float m = 0.0f;
    int c = 0;
    for (int w = 0; w < THREADS / 32; ++w) { m += red_mass[w][tid]; c += red_count[w][tid]; }
    red_mass[0][tid] = m;                            // thread t touches only column t
    red_count[0][tid] = c;
  }
  __syncthreads();
}

__global__ void __launch_bounds__(THREADS, 1) sample_cuts_kernel(
    const float* __restrict__ scores, long long row_stride, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
    const float* __restrict__ uniform, float* __restrict__ sort_prob, int* __restrict__ sort_index, int padded,
    int* __restrict__ out, int vocab, int skip_uncut, int span) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int blocks = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  const int row = blockIdx.x / blocks;
  // a row with every cut switched off keeps the id it was given (the kernel without cuts drew it)
  if (skip_uncut && !(top_k[row] > 0 || top_p[row] < 1.0f || min_p[row] > 0.0f)) return;
  extern __shared__ float few_prob[];                 // [CANDIDATES], then int few_index[CANDIDATES]
  int* few_index = reinterpret_cast<int*>(few_prob + CANDIDATES);
  __shared__ float red_value[32];
  __shared__ int red_index[32];
  __shared__ float chunk_sum[THREADS];
  __shared__ float group_sum[32];
  __shared__ float shared_f[4];
  __shared__ int shared_i[8];
  __shared__ float red_mass[THREADS / 32][LEVELS + 1];
  __shared__ int red_count[THREADS / 32][LEVELS + 1];
  // what the other blocks of the cluster read: this block's maximum, its figures of each pass, its candidates' count
  __shared__ float block_best_value;
  __shared__ int block_best_index;
  __shared__ float pass_mass[3][LEVELS + 1];
  __shared__ Units kept_units;                        // of this block's range
  __shared__ Units warp_units[THREADS / 32];
  __shared__ int pass_count[3][LEVELS + 1];
  __shared__ int gathered;
  // the row's figures of the current pass, the same in every block
  __shared__ float row_mass[LEVELS + 1];
  __shared__ int row_count[LEVELS + 1];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* z = scores + (size_t)row * row_stride;
  float* prob = sort_prob + (size_t)row * padded;     // (prob, index and padded move to shared memory below
  int* index = sort_index + (size_t)row * padded;     //  when few candidates suffice)
  const int lo = min(rank * span, vocab), hi = min(lo + span, vocab);       // this block's indices (span % 4 == 0)

  // Adds every block's figures of a pass (left in row 0 of red_mass / red_count by block_sums) in block order.
  auto row_sums = [&](int pass, int n) {
    if (tid < n) { pass_mass[pass][tid] = red_mass[0][tid]; pass_count[pass][tid] = red_count[0][tid]; }
    cluster.sync();
    if (tid < n) {
      float m = 0.0f;
      int c = 0;
      for (int b = 0; b < blocks; ++b) {
        m += cluster.map_shared_rank(&pass_mass[pass][0], b)[tid];
        c += cluster.map_shared_rank(&pass_count[pass][0], b)[tid];
      }
      row_mass[tid] = m;
      row_count[tid] = c;
    }
    __syncthreads();
  };

  // maximum (first index on ties), as in the plain kernel
  float bv = -INFINITY;
  int bi = 0x7fffffff;
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
  for_each_element(z + lo, hi - lo, [&](float v, int i) {   // (a thread meets its elements in ascending order)
    if (v > bv || bi == 0x7fffffff) { bv = v; bi = lo + i; }
  });
  warp_best();
  if (lane == 0) { red_value[warp] = bv; red_index[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = red_value[lane];
    bi = red_index[lane];
    warp_best();
    if (lane == 0) { block_best_value = bv; block_best_index = bi; }
  }
  cluster.sync();
  if (warp == 0) {
    bv = -INFINITY;
    bi = 0x7fffffff;
    if (lane < blocks) {
      bv = *cluster.map_shared_rank(&block_best_value, lane);
      bi = *cluster.map_shared_rank(&block_best_index, lane);
    }
    warp_best();
    if (lane == 0) { shared_f[0] = bv; shared_i[0] = bi; }
  }
  __syncthreads();
  const float maximum = shared_f[0];
  const int arg_max = shared_i[0];
  const float temp = temperature[row];
  if (!(temp > 0.0f)) {
    if (tid == 0 && rank == 0) out[row] = arg_max;
    cluster.sync();                       // nobody leaves while its shared memory may still be read
    return;
  }
  const float inverse = 1.0f / temp;
  const float floor_value = min_p[row] > 0.0f ? min_p[row] : -1.0f;      // times the best probability, which is exp(0) = 1
  Need need;
  need.k_wanted = top_k[row] > 0 ? min(top_k[row], vocab) : 0;
  need.share = top_p[row];

  // ---- pass 1: probabilities; counts and masses of the coarse levels and of everything min-p keeps ----
  {
    // every thread keeps its level sums in a column of its own in the shared memory that later holds the candidates
    float* const level_mass = few_prob;                                    // [LEVELS][THREADS]
    int* const level_count = reinterpret_cast<int*>(few_prob + LEVELS * THREADS);
#pragma unroll
    for (int l = 0; l < LEVELS; ++l) { level_mass[l * THREADS + tid] = 0.0f; level_count[l * THREADS + tid] = 0; }
    Units kept = 0;
    int kept_count = 0;
    float* const prob_out = prob + lo;
    for_each_element(z + lo, hi - lo, [&](float v, int i) {
      const float pr = expf((v - maximum) * inverse);
      prob_out[i] = pr;
      if (pr >= floor_value) {
        kept += units_of(pr);
        ++kept_count;
        const int level = level_of_exponent(exponents_below(pr));
        if (level < LEVELS) {
          level_mass[level * THREADS + tid] += pr;
          level_count[level * THREADS + tid] += 1;
        }
      }
    });
    float mass[LEVELS + 1];
    int count[LEVELS + 1];
#pragma unroll
    for (int l = 0; l < LEVELS; ++l) { mass[l] = level_mass[l * THREADS + tid]; count[l] = level_count[l * THREADS + tid]; }
    mass[LEVELS] = 0.0f;
    count[LEVELS] = kept_count;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) kept += __shfl_xor_sync(0xffffffffu, kept, offset);
    if (lane == 0) warp_units[warp] = kept;
    block_sums<LEVELS + 1>(mass, count, red_mass, red_count);
    if (tid == 0) {
      Units sum = 0;
      for (int w = 0; w < THREADS / 32; ++w) sum += warp_units[w];
      kept_units = sum;
    }
    row_sums(0, LEVELS + 1);
    if (tid == 0) {
      Units sum = 0;
      for (int b = 0; b < blocks; ++b) sum += *cluster.map_shared_rank(&kept_units, b);
      shared_f[3] = units_value(sum);
    }
    __syncthreads();
  }
  need.kept_mass = shared_f[3];
  need.kept_count = row_count[LEVELS];
  // Thread 0 of every block narrows the threshold, all from the same figures; its block follows through shared_i:
  //   [1] state: 0 searching, 1 found, -1 the full sort   [2] exponent range top   [3] candidates so far
  //   [4] threshold bits (found)   shared_f[2]: mass so far
  if (tid == 0) {
    int state = -1, running_count = 0, level = 0;
    float running_mass = 0.0f;
    if (need.kept_count <= CANDIDATES) {             // all that is kept fits: no threshold beyond the floor
      state = 1;
      shared_i[4] = 0;
    } else {
      for (; level < LEVELS; ++level) {
        if (need.met(running_count + row_count[level], running_mass + row_mass[level])) { state = 0; break; }
        running_count += row_count[level];
        running_mass += row_mass[level];
      }
      if (running_count > CANDIDATES) state = -1;
    }
    shared_i[1] = state;
    shared_i[2] = level;
    shared_i[3] = running_count;
    shared_f[2] = running_mass;
  }
  __syncthreads();
  if (shared_i[1] == 0) {
    // ---- pass 2: the four exponents of the chosen coarse level (bins 0..3; level 0 also holds exponent 0) ----
    const int level = shared_i[2];
    // bin = d - (4 level + 1); the one probability with d = 0 (the best: exactly 1) goes with d = 1
    float mass[BINS];
    int count[BINS];
#pragma unroll
    for (int l = 0; l < BINS; ++l) { mass[l] = 0.0f; count[l] = 0; }
    for_each_element(prob + lo, hi - lo, [&](float pr, int) {
      const int d = exponents_below(pr);
      const bool inside = pr >= floor_value && level_of_exponent(d) == level;
      const int bin = inside ? max(d - (4 * level + 1), 0) : -1;
#pragma unroll
      for (int l = 0; l < 4; ++l) {
        mass[l] += bin == l ? pr : 0.0f;
        count[l] += bin == l ? 1 : 0;
      }
    });
    block_sums<BINS>(mass, count, red_mass, red_count);
    row_sums(1, BINS);
    if (tid == 0) {
      int running_count = shared_i[3], bin = 0;
      float running_mass = shared_f[2];
      for (; bin < 3; ++bin) {
        if (need.met(running_count + row_count[bin], running_mass + row_mass[bin])) break;
        running_count += row_count[bin];
        running_mass += row_mass[bin];
      }
      shared_i[2] = 4 * level + 1 + bin;                               // the exponent d (>= 1) in which the threshold lies
      shared_i[3] = running_count;
      shared_f[2] = running_mass;
      if (running_count > CANDIDATES) shared_i[1] = -1;
    }
    __syncthreads();
  }
  if (shared_i[1] == 0) {
    // ---- pass 3: eight bins of the mantissa within that exponent, highest first ----
    const int d_in = shared_i[2];
    float mass[BINS];
    int count[BINS];
#pragma unroll
    for (int l = 0; l < BINS; ++l) { mass[l] = 0.0f; count[l] = 0; }
    for_each_element(prob + lo, hi - lo, [&](float pr, int) {
      const int d = exponents_below(pr);
      const bool inside = pr >= floor_value && max(d, 1) == d_in;
      const int bin = !inside ? -1 : (d <= 0 ? 0 : 7 - (int)((__float_as_uint(pr) >> 20) & 7u));
#pragma unroll
      for (int l = 0; l < BINS; ++l) {
        mass[l] += bin == l ? pr : 0.0f;
        count[l] += bin == l ? 1 : 0;
      }
    });
    block_sums<BINS>(mass, count, red_mass, red_count);
    row_sums(2, BINS);
    if (tid == 0) {
      int running_count = shared_i[3], bin = 0;
      float running_mass = shared_f[2];
      for (; bin < BINS - 1; ++bin) {
        if (need.met(running_count + row_count[bin], running_mass + row_mass[bin])) break;
        running_count += row_count[bin];
        running_mass += row_mass[bin];
      }
      running_count += row_count[bin];
      // candidates: every kept probability whose bits reach those of the chosen bin's lower edge
      const unsigned int exponent_field = (unsigned int)max(127 - d_in, 0);
      shared_i[4] = (int)((exponent_field << 23) | ((unsigned int)(7 - bin) << 20));
      shared_i[1] = running_count <= CANDIDATES ? 1 : -1;
    }
    __syncthreads();
  }
  const bool few = shared_i[1] == 1;
  const float kept_total = need.kept_mass;
  int count_here = vocab;               // entries of the sorted arrays that are real
  if (few) {
    // ---- gather the candidates into shared memory, all of them into the first block's, and sort them there ----
    const unsigned int threshold_bits = (unsigned int)shared_i[4];
    if (tid == 0) shared_i[5] = 0;
    __syncthreads();
    for_each_element(prob + lo, hi - lo, [&](float pr, int i) {
      if (pr >= floor_value && __float_as_uint(pr) >= threshold_bits) {
        const int slot = atomicAdd(&shared_i[5], 1);
        if (slot < CANDIDATES) {
          few_prob[slot] = pr;
          few_index[slot] = lo + i;
        }
      }
    });
    __syncthreads();
    count_here = min(shared_i[5], CANDIDATES);
    if (tid == 0) gathered = count_here;
    cluster.sync();
    if (rank == 0) {
      for (int b = 1; b < blocks; ++b) {
        const int more = min(*cluster.map_shared_rank(&gathered, b), CANDIDATES - count_here);
        const float* their_prob = cluster.map_shared_rank(few_prob, b);
        const int* their_index = cluster.map_shared_rank(few_index, b);
        for (int i = tid; i < more; i += THREADS) {
          few_prob[count_here + i] = their_prob[i];
          few_index[count_here + i] = their_index[i];
        }
        count_here += more;
      }
    }
    cluster.sync();                       // the candidates were copied: the other blocks are done
    if (rank != 0) return;
    int padded_few = 2;
    while (padded_few < count_here) padded_few <<= 1;
    for (int i = count_here + tid; i < padded_few; i += THREADS) { few_prob[i] = -1.0f; few_index[i] = 0x7fffffff; }
    __syncthreads();
    prob = few_prob;
    index = few_index;
    padded = padded_few;
  } else {
    // the full sort, by the first block alone (every block's probabilities are in global memory after the barrier)
    cluster.sync();
    if (rank != 0) return;
    for (int i = tid; i < padded; i += THREADS) {
      if (i >= vocab) prob[i] = -1.0f;
      index[i] = i;
    }
    __syncthreads();
  }

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
  int keep = need.k_wanted > 0 ? min(need.k_wanted, count_here) : count_here;
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
  // Without a top-k the total is the mass of everything min-p keeps, which the candidates need not all be:
  // it was summed in the first pass.
  const bool total_known = few && need.k_wanted == 0;

  // Sums over the kept prefix in a fixed order: every thread adds a contiguous chunk, 32 threads add 32 chunk sums
  // each (a group), one thread adds the 32 group sums; the walks below skip whole groups and chunks the same way.
  // Candidates in shared memory are added in chunks of sixteen whatever their number, so that a threshold that
  // let a few more of them in changes no sum over the prefix that is walked.
  constexpr int GROUP = 32;
  const int chunk = few ? CANDIDATES / THREADS : (keep + THREADS - 1) / THREADS;
  const int begin = min(tid * chunk, keep), end = min(begin + chunk, keep);
  float local = 0.0f;
  for (int i = begin; i < end; ++i) local += prob[i];
  chunk_sum[tid] = local;
  __syncthreads();
  if (tid < GROUP) {
    float sum = 0.0f;
    for (int c = 0; c < THREADS / GROUP; ++c) sum += chunk_sum[tid * (THREADS / GROUP) + c];
    group_sum[tid] = sum;
  }
  __syncthreads();
  if (tid == 0) {
    float total = 0.0f;
    for (int g = 0; g < GROUP; ++g) total += group_sum[g];
    if (total_known) total = kept_total;
    shared_f[1] = total;
    // nucleus: shortest prefix whose share of the total reaches top_p
    int limit = keep;
    const float nucleus = need.share;
    if (nucleus < 1.0f && total > 0.0f) {
      float cumulative = 0.0f;
      bool found = false;
      for (int g = 0; g < GROUP && !found; ++g) {
        const int first_chunk = g * (THREADS / GROUP);
        if (first_chunk * chunk >= keep) break;
        if ((cumulative + group_sum[g]) / total < nucleus && (first_chunk + THREADS / GROUP) * chunk < keep) {
          cumulative += group_sum[g];
          continue;
        }
        for (int c = first_chunk; c < first_chunk + THREADS / GROUP && !found; ++c) {
          const int cb = min(c * chunk, keep), ce = min(cb + chunk, keep);
          if (cb >= ce) break;
          if ((cumulative + chunk_sum[c]) / total < nucleus && ce < keep) {
            cumulative += chunk_sum[c];
            continue;
          }
          for (int i = cb; i < ce; ++i) {
            cumulative += prob[i];
            if (cumulative / total >= nucleus) { limit = i + 1; found = true; break; }
          }
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
  const int chunk2 = few ? CANDIDATES / THREADS : (limit + THREADS - 1) / THREADS;
  const int b2 = min(tid * chunk2, limit), e2 = min(b2 + chunk2, limit);
  local = 0.0f;
  for (int i = b2; i < e2; ++i) local += prob[i];
  __syncthreads();
  chunk_sum[tid] = local;
  __syncthreads();
  if (tid < GROUP) {
    float sum = 0.0f;
    for (int c = 0; c < THREADS / GROUP; ++c) sum += chunk_sum[tid * (THREADS / GROUP) + c];
    group_sum[tid] = sum;
  }
  __syncthreads();
  if (tid == 0) {
    float kept = 0.0f;
    for (int g = 0; g < GROUP; ++g) kept += group_sum[g];
    int result = index[0];
    if (kept > 0.0f) {
      float target = uniform[row] * kept;
      result = index[limit - 1];
      bool found = false;
      for (int g = 0; g < GROUP && !found; ++g) {
        const int first_chunk = g * (THREADS / GROUP);
        if (first_chunk * chunk2 >= limit) break;
        if (target - group_sum[g] > 0.0f) { target -= group_sum[g]; continue; }
        for (int c = first_chunk; c < first_chunk + THREADS / GROUP && !found; ++c) {
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
// skip_uncut: rows whose cuts are all switched off (top_k 0, top_p >= 1, min_p <= 0) are left untouched in `out`.
TGE_API int tge_sample_cuts(const float* scores, long long row_stride, const float* temperature, const int* top_k,
                            const float* top_p, const float* min_p, const float* uniform, float* sort_prob,
                            int* sort_index, int* out, int rows, int vocab, int skip_uncut, cudaStream_t stream) {
  TGE_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "sample_cuts: bad sizes rows=%d vocab=%d", rows, vocab);
  TGE_REQUIRE(sort_prob != nullptr && sort_index != nullptr, "sample_cuts: needs scratch for the sort");
  if (rows == 0) return 0;
  const size_t smem = (size_t)CANDIDATES * (sizeof(float) + sizeof(int));
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(sample_cuts_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) {
      tge_set_error("sample_cuts: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
      return -2;
    }
    configured = true;
  }
  // Blocks per row: a power of two, eight at most, each with at least 8,192 scores, and no more blocks in all
  // than the GPU runs at once: a block holds 128 KB of shared memory, so an SM takes one, and a cluster of four
  // or eight needs its SMs in one part of the GPU, so that only three quarters of the SMs are counted on (16
  // rows of eight blocks took 91 us, of four 51 us).  The choice changes no result (see the head of this file).
  int blocks = 1;
  while (blocks < MAX_CLUSTER && vocab / (2 * blocks) >= 8192 &&
         (long long)rows * 2 * blocks <= (blocks == 1 ? tge_sm_count() : 3 * tge_sm_count() / 4))
    blocks *= 2;
  const int span = ((vocab + blocks - 1) / blocks + 3) / 4 * 4;
  const cudaError_t err = tge_launch_clusters(sample_cuts_kernel, dim3(rows * blocks), dim3(THREADS), smem, blocks, stream,
                                              scores, row_stride, temperature, top_k, top_p, min_p, uniform, sort_prob,
                                              sort_index, (int)tge_sample_cuts_padded(vocab), out, vocab, skip_uncut, span);
  TGE_REQUIRE(err == cudaSuccess, "sample_cuts: launch failed: %s", cudaGetErrorString(err));
  return tge_launched("sample_cuts", 1);
}
