// bfloat16 matrix product on the 5th-generation tensor cores: out = x . w^T (+ epilogue).
//
// Shape of the kernel (one persistent block per SM, 320 threads):
//   warp 0     one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle)
//              of a 128-row weight tile and a BN-row activation tile per k-block
//              of 64 into a ring of shared-memory stages;
//   warp 1     allocates tensor memory; one lane issues tcgen05.mma (M=128, N=BN,
//              K=16, float32 accumulators in tensor memory) and commits each
//              stage back to the loader and each finished tile to the epilogue;
//   warps 2-9  read the accumulator with tcgen05.ld (two warps per 32-lane quarter,
//              half the columns each) and apply the epilogue, while the MMA warp
//              already fills the second accumulator buffer with the next tile.
// The weight rows are the M side of the instruction ("swap-AB"): a decode step
// with 1..64 tokens still fills all 128 lanes with useful rows and streams each
// weight byte exactly once; the token tile BN is 16..256.  Narrow outputs with
// few tiles are additionally cut along k; the partial sums go to a float32
// scratch buffer and a second kernel adds them in split order and applies the
// epilogue, so the result does not depend on which block ran when.
//
// Epilogues: +bias -> run dtype; +bias -> float32; += into the float32 residual
// stream; SiLU(gate)*up over interleaved weight rows (row 2i = gate_i, 2i+1 =
// up_i), exchanged between neighbouring lanes.  Formulas as in gemm_simt.cu.
//
// Every wait on an mbarrier is bounded: after about two seconds a waiter sets
// TGE_STATUS_WAIT_TIMEOUT in the status word, all roles leave their loops, the
// loader waits (bounded) for its copies in flight, tensor memory is freed and
// the kernel returns.
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"

enum GemmEpilogue : int { GEMM_STORE = 0, GEMM_STORE_F32 = 1, GEMM_ADD_F32 = 2, GEMM_SWIGLU = 3 };

namespace {

constexpr int BM = 128;                  // weight rows per tile = tensor-memory lanes
constexpr int BK = 64;                   // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int MAX_STAGES = 8;
constexpr int EPI_WARPS = 8;              // two per 32-lane quarter of tensor memory, each taking half the columns
constexpr int NUM_THREADS = (2 + EPI_WARPS) * 32;
constexpr int SMEM_LIMIT = 227 * 1024;

struct GemmParams {
  int n_w, m_tok, K;
  int bn, stages, splits;
  int k_blocks, tiles_w, tiles_t;
  int epilogue;
  int acc_cols;        // tensor-memory columns allocated (power of two >= 32)
  int to_partial;      // write float32 partial sums to `partial` instead of applying the epilogue
  const float* bias;
  void* out;
  long long ldo;
  float* partial;
  int* status;
  // Rows of x that still lack their RMSNorm factor: 1 / sqrt(sum over slices of ss[slice][token] / ss_width + ss_eps)
  // multiplies the product's column of that token (null: x is complete).  At most DEFER_MAX_TOKENS tokens.
  const float* ss;
  int ss_slices, ss_width;
  float ss_eps;
};
constexpr int DEFER_MAX_TOKENS = 128;

// ---- PTX wrappers ----------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}

// Bounded wait.  Returns false when it gave up (after `limit_ns` nanoseconds) or when another role already did.
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, volatile int* abort_flag,
                                          unsigned long long limit_ns = WAIT_LIMIT_NS) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long start = global_timer();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 1023u) == 0) {
      if (*abort_flag) return false;
      if (global_timer() - start > limit_ns) {
        *abort_flag = 1;
        atomicOr(status, TGE_STATUS_WAIT_TIMEOUT);
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T, both operands K-major, bf16 in, f32 out
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

// 32 lanes x 16 consecutive columns of 32-bit accumulators
__device__ __forceinline__ void tc_load16(uint32_t taddr, uint32_t r[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

// Shared-memory operand descriptor: K-major tile of 128-byte rows, 128-byte
// swizzle, 8-row groups 1024 bytes apart, descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);   // start address, 16-byte units
  desc |= (uint64_t)1 << 16;                         // leading byte offset (unused for swizzled K-major)
  desc |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset between 8-row groups
  desc |= (uint64_t)1 << 46;                         // descriptor version
  desc |= (uint64_t)2 << 61;                         // SWIZZLE_128B
  return desc;
}

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

// 1 / sqrt(mean square of the row + eps) from the row's sums of squares in slices (added in slice order; the
// loads of eight slices are in flight together)
__device__ __forceinline__ float row_factor_of(const float* __restrict__ ss, int slices, int width, float eps, int m_tok, int m) {
  if (ss == nullptr) return 1.0f;
  float sum = 0.0f;
  for (int first = 0; first < slices; first += 8) {
    float part[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) part[i] = first + i < slices ? ss[(size_t)(first + i) * m_tok + m] : 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) sum += part[i];
  }
  return 1.0f / sqrtf(sum / (float)width + eps);
}

// The epilogue of one finished tile: this warp's 32 lanes (weight rows n) by its columns [c_begin, c_end)
// of the accumulator buffer `acc`.
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t tmem_base, int acc, int quarter, int lane,
                                              int c_begin, int c_end, int n, int tile_t, int split,
                                              const float* row_factor = nullptr) {
  const bool n_ok = n < p.n_w;
  const float bias = (p.bias && n_ok && !p.to_partial) ? p.bias[n] : 0.0f;
  for (int c0 = c_begin; c0 < c_end; c0 += 16) {
    uint32_t r[16];
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * p.bn + c0);
    tc_load16(taddr, r);
    const int m0 = tile_t * p.bn + c0;
    if (m0 >= p.m_tok) continue;                              // uniform over the warp
    if (row_factor != nullptr && !p.to_partial) {             // partial sums stay as they are: who adds them scales
#pragma unroll
      for (int j = 0; j < 16; ++j)
        r[j] = __float_as_uint(__uint_as_float(r[j]) * row_factor[min(m0 + j, DEFER_MAX_TOKENS - 1)]);
    }
    if (!p.to_partial && p.epilogue == GEMM_ADD_F32) {
      // read all sixteen old values before the first store, so the loads overlap
      float* dst = reinterpret_cast<float*>(p.out) + (size_t)m0 * p.ldo + n;
      float old[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) old[j] = (n_ok && m0 + j < p.m_tok) ? dst[(size_t)j * p.ldo] : 0.0f;
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (n_ok && m0 + j < p.m_tok) dst[(size_t)j * p.ldo] = old[j] + __uint_as_float(r[j]) + bias;
      continue;
    }
    if (!p.to_partial && p.epilogue == GEMM_SWIGLU) {
      // Even lanes hold gate rows, odd lanes the matching up rows.  Per pair of token columns one
      // exchange gives the even lane (gate, up) of the first column and the odd lane those of the second.
      const bool odd = lane & 1;
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        const float a = __uint_as_float(r[j]) + bias, b = __uint_as_float(r[j + 1]) + bias;
        const float got = __shfl_xor_sync(0xffffffffu, odd ? a : b, 1);
        const float g = odd ? got : a, u = odd ? b : got;
        const int m = m0 + j + (odd ? 1 : 0);
        if (n_ok && m < p.m_tok)
          reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + (n >> 1)] =
              __float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g)) * u);
      }
      continue;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int m = m0 + j;
      float v = __uint_as_float(r[j]) + bias;
      if (p.to_partial) {
        if (n_ok && m < p.m_tok) p.partial[((size_t)split * p.m_tok + m) * p.n_w + n] = v;
      } else if (n_ok && m < p.m_tok) {
        if (p.epilogue == GEMM_STORE) reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + n] = __float2bfloat16_rn(v);
        else reinterpret_cast<float*>(p.out)[(size_t)m * p.ldo + n] = v;
      }
    }
  }
}

// ---- the kernel ------------------------------------------------------------
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  // stages first (1024-byte aligned for the swizzle), barriers after them
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t b_stage_bytes = (uint32_t)p.bn * BK * 2;
  const uint32_t stage_bytes = A_STAGE_BYTES + b_stage_bytes;
  const uint32_t bars = base + (uint32_t)p.stages * stage_bytes;
  // barrier layout: full[stages], empty[stages], tmem_full[2], tmem_empty[2], then tmem base, abort flag
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (p.stages + s); };
  auto tfull_bar = [&](int s) { return bars + 8u * (2 * p.stages + s); };
  auto tempty_bar = [&](int s) { return bars + 8u * (2 * p.stages + 2 + s); };
  const uint32_t tmem_slot = bars + 8u * (2 * p.stages + 4);
  unsigned char* generic_base = smem_raw + (base - raw);
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(generic_base + (size_t)p.stages * stage_bytes + 8u * (2 * p.stages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot_ptr + 1);

  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), EPI_WARPS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tmem_slot), "r"((uint32_t)p.acc_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // Only now may the next kernel be scheduled: this block already holds its tensor memory, so a block of
  // the next kernel that lands on the same SM can at worst wait for it, never starve it.
  pdl_trigger();
  // Set-up above overlapped the previous kernel; from here on its results are read.  The loading warp
  // waits later: weights are nobody's result, so it first asks for a ring-full of weight tiles.
  if (warp != 0) pdl_wait();

  const int total_work = p.tiles_w * p.tiles_t * p.splits;
  float* row_factor = nullptr;
  if (p.ss != nullptr && !p.to_partial && warp >= 2) {
    // the epilogue warps work out every token's factor once, while the first tile is being multiplied
    // (partial sums are left unscaled: the kernel that adds them applies the factor)
    row_factor = reinterpret_cast<float*>(const_cast<int*>(abort_flag) + 3);
    const int m = (int)threadIdx.x - 64;
    if (m < DEFER_MAX_TOKENS)
      row_factor[m] = m < p.m_tok ? row_factor_of(p.ss, p.ss_slices, p.ss_width, p.ss_eps, p.m_tok, m) : 0.0f;
    asm volatile("bar.sync 1, %0;\n" ::"n"(EPI_WARPS * 32) : "memory");
  }

  if (warp == 0) {
    // ------------------------------ TMA loader ------------------------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      int ahead = 0;      // stages of the first item whose weight tile is already on its way
      if ((int)blockIdx.x < total_work) {
        const int split = (int)blockIdx.x % p.splits;
        const int tile_w = ((int)blockIdx.x / p.splits) / p.tiles_t;
        const int kb_begin = (int)((long long)split * p.k_blocks / p.splits);
        const int kb_end = (int)((long long)(split + 1) * p.k_blocks / p.splits);
        ahead = kb_end - kb_begin < p.stages ? kb_end - kb_begin : p.stages;
        for (int s = 0; s < ahead; ++s) {
          mbar_expect_tx(full_bar(s), stage_bytes);
          tma_load_2d(base + (uint32_t)s * stage_bytes, &map_w, full_bar(s), (kb_begin + s) * BK, tile_w * BM);
        }
      }
      pdl_wait();
      for (int work = blockIdx.x; work < total_work && ok; work += gridDim.x) {
        const int split = work % p.splits;
        const int rest = work / p.splits;
        const int tile_t = rest % p.tiles_t, tile_w = rest / p.tiles_t;
        const int kb_begin = (int)((long long)split * p.k_blocks / p.splits);
        const int kb_end = (int)((long long)(split + 1) * p.k_blocks / p.splits);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          const uint32_t a_dst = base + (uint32_t)stage * stage_bytes;
          if (ahead > 0) {
            --ahead;      // first pass over the ring: the stage is free and its weight tile was requested above
          } else {
            if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, abort_flag)) { ok = false; break; }
            mbar_expect_tx(full_bar(stage), stage_bytes);
            tma_load_2d(a_dst, &map_w, full_bar(stage), kb * BK, tile_w * BM);
          }
          tma_load_2d(a_dst + A_STAGE_BYTES, &map_x, full_bar(stage), kb * BK, tile_t * p.bn);
          ++issued;
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok || *abort_flag) {
        // wait (bounded) for the copies already issued, newest phase of every stage used
        const int used = issued < p.stages ? issued : p.stages;
        for (int back = 1; back <= used; ++back) {
          int s = stage - back;
          uint32_t ph = phase;
          if (s < 0) { s += p.stages; ph ^= 1u; }
          const unsigned long long start = global_timer();
          while (!mbar_try_wait(full_bar(s), ph) && global_timer() - start < 100000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (elect_one()) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < total_work && ok; work += gridDim.x) {
        const int split = work % p.splits;
        const int kb_begin = (int)((long long)split * p.k_blocks / p.splits);
        const int kb_end = (int)((long long)(split + 1) * p.k_blocks / p.splits);
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, p.status, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.bn);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, p.status, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = base + (uint32_t)stage * stage_bytes;
          const uint32_t b_addr = a_addr + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t desc_a = make_smem_desc(a_addr + k * UMMA_K * 2);
            const uint64_t desc_b = make_smem_desc(b_addr + k * UMMA_K * 2);
            tc_mma(d_tmem, desc_a, desc_b, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(tfull_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------- epilogue -------------------------------
    const int quarter = warp & 3;            // tensor-memory lanes this warp may read
    const int column_half = (warp - 2) >> 2; // which half of the token columns it takes
    const int first_half = ((p.bn / 16 + 1) / 2) * 16;   // groups of 16 columns, the odd one to the first half
    const int c_begin = column_half == 0 ? 0 : first_half;
    const int c_end = column_half == 0 ? first_half : p.bn;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int work = blockIdx.x; work < total_work && ok; work += gridDim.x) {
      const int split = work % p.splits;
      const int rest = work / p.splits;
      const int tile_t = rest % p.tiles_t, tile_w = rest / p.tiles_t;
      if (!mbar_wait(tfull_bar(acc), acc_phase, p.status, abort_flag)) { ok = false; break; }
      tc_fence_after();
      epilogue_tile(p, tmem_base, acc, quarter, lane, c_begin, c_end, tile_w * BM + quarter * 32 + lane, tile_t, split,
                    row_factor);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)p.acc_cols) : "memory");
  }
}

// ---- two SMs on one tile ------------------------------------------------------
// A pair of blocks (a cluster of two) owns a tile of 256 weight rows by BN tokens.  Each block copies its
// own 128 weight rows and its own half of the token rows into its own shared memory; one thread of the
// even block issues tcgen05.mma.cta_group::2 (M = 256), which reads the weight rows of each block for that
// block's accumulator lanes and the token rows of both for all of them, so every SM fetches half as many
// token rows per product as when it works alone.  Each block's tensor memory ends up holding its 128 rows
// by BN columns, in the layout of the one-SM kernel, and each block runs the same epilogue on it.
// Barriers: the copies of both blocks complete on the even block's full barrier; a commit of the issuing
// thread arrives on the empty (and accumulator-full) barrier at the same offset in both blocks; the epilogue
// warps of both blocks arrive on the even block's accumulator-empty barrier.  Waits are bounded as above;
// both blocks meet at a cluster barrier before tensor memory is freed, so neither leaves while the other may
// still signal it.
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
// the address, in the cluster's shared window, of `addr` of this block as seen in block `rank`
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.aligned;\nbarrier.cluster.wait.aligned;\n" ::: "memory");
}
// copy into this block's shared memory, bytes counted on a barrier that may live in the other block of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// arrives on the barrier at this offset in both blocks of the pair once the products issued so far are done
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  const uint32_t zero = 0;      // no output lane is switched off
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}\n"
      ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(zero) : "memory");
}

constexpr int PAIR_BM = 2 * BM;          // weight rows per tile of a pair

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                         const GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t b_half_bytes = (uint32_t)(p.bn / 2) * BK * 2;          // this block's half of the token rows
  const uint32_t stage_bytes = A_STAGE_BYTES + b_half_bytes;
  const uint32_t bars = base + (uint32_t)p.stages * stage_bytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (p.stages + s); };
  auto tfull_bar = [&](int s) { return bars + 8u * (2 * p.stages + s); };
  auto tempty_bar = [&](int s) { return bars + 8u * (2 * p.stages + 2 + s); };
  const uint32_t tmem_slot = bars + 8u * (2 * p.stages + 4);
  unsigned char* generic_base = smem_raw + (base - raw);
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(generic_base + (size_t)p.stages * stage_bytes + 8u * (2 * p.stages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot_ptr + 1);

  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();                                 // 0: issues the products; 1: its partner

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full_bar(s), 1);                                        // used in the even block only
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), 2 * EPI_WARPS);                          // used in the even block only
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) {
    // one warp of each block, the same warp in both, the same place for the address in both
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tmem_slot), "r"((uint32_t)p.acc_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
  }
  __syncwarp();
  tc_fence_before();
  cluster_sync_all();             // both blocks' barriers exist before either signals the other
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  pdl_trigger();
  pdl_wait();

  const int total_work = p.tiles_w * p.tiles_t * p.splits;
  const int pair = (int)blockIdx.x >> 1, pairs = (int)gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------ TMA loader (both blocks) ------------------------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int work = pair; work < total_work && ok; work += pairs) {
        const int split = work % p.splits;
        const int rest = work / p.splits;
        const int tile_t = rest % p.tiles_t, tile_w = rest / p.tiles_t;
        const int kb_begin = (int)((long long)split * p.k_blocks / p.splits);
        const int kb_end = (int)((long long)(split + 1) * p.k_blocks / p.splits);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, abort_flag)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2u * stage_bytes);
          const uint32_t leader_full = map_to_rank(full_bar(stage), 0);
          const uint32_t a_dst = base + (uint32_t)stage * stage_bytes;
          tma_load_2d_pair(a_dst, &map_w, leader_full, kb * BK, tile_w * PAIR_BM + (int)rank * BM);
          tma_load_2d_pair(a_dst + A_STAGE_BYTES, &map_x, leader_full, kb * BK, tile_t * p.bn + (int)rank * (p.bn / 2));
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok || *abort_flag) {
        // copies may still be on their way into this block's shared memory: give them time
        const unsigned long long start = global_timer();
        while (global_timer() - start < 1000000ull) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even block) ------------------------------
    if (rank == 0 && elect_one()) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)(PAIR_BM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int work = pair; work < total_work && ok; work += pairs) {
        const int split = work % p.splits;
        const int kb_begin = (int)((long long)split * p.k_blocks / p.splits);
        const int kb_end = (int)((long long)(split + 1) * p.k_blocks / p.splits);
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, p.status, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.bn);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, p.status, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = base + (uint32_t)stage * stage_bytes;
          const uint32_t b_addr = a_addr + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t desc_a = make_smem_desc(a_addr + k * UMMA_K * 2);
            const uint64_t desc_b = make_smem_desc(b_addr + k * UMMA_K * 2);
            tc_mma_pair(d_tmem, desc_a, desc_b, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
          }
          tc_commit_pair(empty_bar(stage));
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit_pair(tfull_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------- epilogue (both blocks) -------------------------------
    const int quarter = warp & 3;
    const int column_half = (warp - 2) >> 2;
    const int first_half = ((p.bn / 16 + 1) / 2) * 16;
    const int c_begin = column_half == 0 ? 0 : first_half;
    const int c_end = column_half == 0 ? first_half : p.bn;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int work = pair; work < total_work && ok; work += pairs) {
      const int split = work % p.splits;
      const int rest = work / p.splits;
      const int tile_t = rest % p.tiles_t, tile_w = rest / p.tiles_t;
      if (!mbar_wait(tfull_bar(acc), acc_phase, p.status, abort_flag)) { ok = false; break; }
      tc_fence_after();
      epilogue_tile(p, tmem_base, acc, quarter, lane, c_begin, c_end,
                    tile_w * PAIR_BM + (int)rank * BM + quarter * 32 + lane, tile_t, split);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_rank(tempty_bar(acc), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  __syncwarp();
  tc_fence_before();
  cluster_sync_all();             // nobody of the pair is still computing, copying or signalling
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)p.acc_cols) : "memory");
  }
}

// Adds the k-splits in split order and applies the epilogue.
__global__ void splitk_epilogue_kernel(const float* __restrict__ partial, const float* __restrict__ bias, void* out,
                                       long long ldo, int m_tok, int n_w, int splits, int epilogue,
                                       const float* __restrict__ ss, int ss_slices, int ss_width, float ss_eps) {
  pdl_trigger();
  pdl_wait();
  const size_t plane = (size_t)m_tok * n_w;
  if (epilogue == GEMM_SWIGLU) {
    const size_t count = plane / 2;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
      const int m = (int)(i / (n_w / 2)), c = (int)(i % (n_w / 2));
      float g = 0.0f, u = 0.0f;
      for (int s = 0; s < splits; ++s) {
        const float2 v = *reinterpret_cast<const float2*>(partial + s * plane + (size_t)m * n_w + 2 * c);
        g += v.x;
        u += v.y;
      }
      const float factor = row_factor_of(ss, ss_slices, ss_width, ss_eps, m_tok, m);
      g *= factor;
      u *= factor;
      if (bias) { g += bias[2 * c]; u += bias[2 * c + 1]; }
      reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + c] = __float2bfloat16_rn(silu_mul(g, u));
    }
    return;
  }
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < plane; i += (size_t)gridDim.x * blockDim.x) {
    const int m = (int)(i / n_w), n = (int)(i % n_w);
    float v = 0.0f;
    for (int s = 0; s < splits; ++s) v += partial[s * plane + i];
    v *= row_factor_of(ss, ss_slices, ss_width, ss_eps, m_tok, m);
    if (bias) v += bias[n];
    if (epilogue == GEMM_STORE) reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(v);
    else if (epilogue == GEMM_STORE_F32) reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = v;
    else reinterpret_cast<float*>(out)[(size_t)m * ldo + n] += v;
  }
}

// ---- host side ---------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// rows x K bf16 matrix, row stride `ld` elements; box = box_rows x 64 elements, 128-byte swizzle
int make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows,
             CUtensorMapL2promotion promo) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    tge_set_error("gemm_tcgen05: the driver does not export cuTensorMapEncodeTiled");
    return -3;
  }
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    tge_set_error("gemm_tcgen05: cuTensorMapEncodeTiled failed with code %d (rows=%lld K=%lld ld=%lld box=%d)", (int)rc,
                  rows, K, ld, box_rows);
    return -3;
  }
  return 0;
}

int sm_count() { return tge_sm_count(); }

struct Plan {
  int bn, stages, splits;
};

// Sums of squares of the rows of x, in slices, when x still lacks its RMSNorm factor (ss null: it does not).
struct RowSums {
  const float* ss = nullptr;
  int slices = 0, width = 0;
  float eps = 0.0f;
};

// What a k-block (64 of k) of one work item costs, in cycles at about 1.9 GHz, by the width of the token tile.
// Measured with both operands in L2, one item per SM (or per pair of SMs), as the difference between two lengths of
// k.  An SM alone needs 2.6 to 3 cycles per token column whatever the width (the tensor core alone 2), so narrow
// tiles that fill the last wave better cost it nothing; a pair has a floor of about 440 cycles per k-block (its
// signals cross between two SMs) and is at its best, 2.4 to 2.6 cycles per column, from 176 columns on.  (The
// 2,048-token products of the 7B shape by width of the pair's tile, 176 / 192 / 208 / 224 / 256 columns: gate and
// up 342 / 340 / 334 / 352 / 324 us, down 219 / 236 / 180 / 188 / 205 us, q/k/v 55 / 57 / 61 / 66 / 55 us, o 53 / 55 / 47 /
// 49 / 55 us: the order this table gives.)
int interpolate(const int (*table)[2], int entries, int bn) {
  if (bn <= table[0][0]) return table[0][1];
  for (int i = 1; i < entries; ++i)
    if (bn <= table[i][0])
      return table[i - 1][1] + (table[i][1] - table[i - 1][1]) * (bn - table[i - 1][0]) / (table[i][0] - table[i - 1][0]);
  return table[entries - 1][1];
}
int one_sm_kblock_cycles(int bn) {
  static const int table[][2] = {{32, 290}, {64, 345}, {128, 368}, {160, 428}, {192, 536}, {224, 581}, {256, 757}};
  return interpolate(table, 7, bn);
}
int pair_kblock_cycles(int bn) {
  static const int table[][2] = {{176, 440}, {192, 482}, {208, 543}, {224, 589}, {240, 640}, {256, 620}};
  return interpolate(table, 6, bn);
}

// What a plan costs, in the same cycles: waves of the grid x (k-blocks per item + a fixed cost per item of about
// six k-blocks) x the cost of a k-block at this tile width.  A cut along k adds a kernel that sums the partial sums
// (about 3 us) and their way to memory and back (8 bytes per partial sum at about 4 TB/s).
long long plan_cost(long long items, int places, int k_blocks, int splits, int kblock_cycles, long long outputs) {
  const long long waves = (items * splits + places - 1) / places;
  long long cost = waves * ((k_blocks + splits - 1) / splits + 6) * kblock_cycles;
  if (splits > 1) cost += 5700 + (long long)((double)splits * outputs * 8.0 / 4.0e12 * 1.9e9);
  return cost;
}

Plan make_plan(int M, int N, int K, long long scratch_floats, int force_bn, int force_splits) {
  Plan plan;
  const int sms = sm_count();
  const int tiles_w = (N + BM - 1) / BM;
  int bn, wide_splits = 0;                 // wide_splits: the cut chosen together with the width (more than 128 tokens)
  if (force_bn > 0) bn = force_bn;
  else if (M <= 16) bn = 16;
  else if (M <= 32) bn = 32;
  else if (M <= 64) bn = 64;
  else if (M <= 128) bn = 128;
  else {
    // More than 128 tokens: every width of the token tile (a multiple of 16 in 128..256, the tokens shared out
    // evenly) with every cut along k that the scratch holds, by the cost above; ties go to the wider tile and
    // the fewer splits.
    const int k_blocks_here = (K + BK - 1) / BK;
    long long best = -1;
    bn = 256;
    for (int count = (M + 255) / 256;; ++count) {
      const int width = ((M + count - 1) / count + 15) / 16 * 16;
      if (width < 128) break;
      const long long items = (long long)tiles_w * ((M + width - 1) / width);
      const int most = force_splits > 0 ? force_splits : (items >= sms || k_blocks_here < 8 ? 1 : (k_blocks_here / 4 < 32 ? k_blocks_here / 4 : 32));
      for (int s = force_splits > 0 ? force_splits : 1; s <= most; ++s) {
        if (s > 1 && (long long)s * M * N > scratch_floats) break;
        const long long cost = plan_cost(items, sms, k_blocks_here, s, one_sm_kblock_cycles(width), (long long)M * N);
        if (best < 0 || cost < best) { best = cost; bn = width; wide_splits = s; }
      }
    }
  }
  plan.bn = bn;
  const int stage_bytes = A_STAGE_BYTES + bn * BK * 2;
  int stages = (SMEM_LIMIT - 2048) / stage_bytes;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  const int k_blocks = (K + BK - 1) / BK;
  if (stages > k_blocks) stages = k_blocks < 2 ? 2 : k_blocks;
  plan.stages = stages;
  const long long tiles = (long long)tiles_w * ((M + bn - 1) / bn);
  int splits = 1;
  if (force_splits > 0) splits = force_splits;
  else if (wide_splits > 0) splits = wide_splits;
  else if (tiles < sms && k_blocks >= 8) {
    // Few tiles: cut k so that the work items fill whole waves of the persistent grid.  The cost of a
    // choice is waves x (k-blocks per item + a fixed per-item overhead, in k-blocks); ties go to fewer splits.
    const int overhead = 6;
    long long best_cost = -1;
    const int most = k_blocks / 4 < 32 ? k_blocks / 4 : 32;
    for (int s = 1; s <= most; ++s) {
      if ((long long)s * M * N > scratch_floats && s > 1) break;
      const long long items = tiles * s;
      const long long waves = (items + sms - 1) / sms;
      const long long cost = waves * ((k_blocks + s - 1) / s + overhead);
      if (best_cost < 0 || cost < best_cost) { best_cost = cost; splits = s; }
    }
  }
  if (splits > k_blocks) splits = k_blocks;
  while (splits > 1 && (long long)splits * M * N > scratch_floats) --splits;
  if (splits < 1) splits = 1;
  plan.splits = splits;
  return plan;
}

// ---- pairs of SMs ----
int g_pair_mode = 1;      // 0: never; 1: where it is expected to be faster; 2: wherever the kernel can run

// How many pairs of blocks of the pair kernel the GPU holds at once; 0 when it cannot be launched.
int pair_capacity() {
  static int capacity = -1;
  if (capacity >= 0) return capacity;
  capacity = 0;
  if (getenv("TGE_NO_PAIR_GEMM") != nullptr) return capacity;
  if (cudaFuncSetAttribute(gemm_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT) != cudaSuccess) {
    cudaGetLastError();
    return capacity;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(sm_count() / 2 * 2);
  config.blockDim = dim3(NUM_THREADS);
  config.dynamicSmemBytes = SMEM_LIMIT;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = 2;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tcgen05_pair_kernel, &config) == cudaSuccess && clusters > 0)
    capacity = clusters < sm_count() / 2 ? clusters : sm_count() / 2;
  else
    cudaGetLastError();
  return capacity;
}

// Token tile and cut along k of the pair kernel: the widest tiles first, then enough splits to fill the pairs.
Plan make_pair_plan(int M, int N, int K, int pairs, long long scratch_floats, long long* cost_out) {
  Plan plan;
  const int tiles_w = (N + PAIR_BM - 1) / PAIR_BM;
  const int k_blocks = (K + BK - 1) / BK;
  int first_width;
  if (M <= 16) first_width = 16;
  else if (M <= 32) first_width = 32;
  else if (M <= 64) first_width = 64;
  else if (M <= 128) first_width = 128;
  else first_width = 0;
  long long best = -1;
  plan.bn = 256;
  plan.splits = 1;
  for (int count = (M + 255) / 256;; ++count) {
    const int width = first_width ? first_width : ((M + count - 1) / count + 15) / 16 * 16;
    if (!first_width && width < 128) break;
    const long long items = (long long)tiles_w * ((M + width - 1) / width);
    const int most = items >= pairs || k_blocks < 8 ? 1 : (k_blocks / 4 < 32 ? k_blocks / 4 : 32);
    for (int splits = 1; splits <= most; ++splits) {
      if (splits > 1 && (long long)splits * M * N > scratch_floats) break;
      const long long cost = plan_cost(items, pairs, k_blocks, splits, pair_kblock_cycles(width), (long long)M * N);
      if (best < 0 || cost < best) { best = cost; plan.bn = width; plan.splits = splits; }
    }
    if (first_width) break;
  }
  const int stage_bytes = A_STAGE_BYTES + (plan.bn / 2) * BK * 2;
  int stages = (SMEM_LIMIT - 2048) / stage_bytes;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages > k_blocks) stages = k_blocks < 2 ? 2 : k_blocks;
  plan.stages = stages;
  *cost_out = best;
  return plan;
}

// Whether the pair kernel takes this product, and with which plan.
bool choose_pair(int M, int N, int K, long long scratch_floats, const Plan& single, int force_bn, int force_splits,
                 Plan* pair_plan) {
  if (g_pair_mode <= 0 || force_bn != 0 || force_splits != 0 || (M <= 128 && g_pair_mode != 2)) return false;
  const int pairs = pair_capacity();
  if (pairs <= 0) return false;
  long long pair_cost = 0;
  *pair_plan = make_pair_plan(M, N, K, pairs, scratch_floats, &pair_cost);
  const long long single_items = (long long)((N + BM - 1) / BM) * ((M + single.bn - 1) / single.bn);
  long long single_cost = plan_cost(single_items, sm_count(), (K + BK - 1) / BK, single.splits,
                                    one_sm_kblock_cycles(single.bn), (long long)M * N);
  // From about a thousand tokens on the pair does better than these figures say (every SM fetches half as many
  // token rows, which counts once the operands no longer sit in L2: o at 4,096 tokens 78 us against 92, down 375
  // against 420, where the figures put the SM alone ahead by a few per cent), so it is given 15 % there.
  if (M >= 1024) single_cost += single_cost * 15 / 100;
  return g_pair_mode == 2 || pair_cost <= single_cost;
}

}  // namespace

// 0: never pair two SMs on a tile; 1: where it is expected to be faster (the default); 2: wherever possible.
TGE_API void tge_gemm_tcgen05_pair_mode(int mode) { g_pair_mode = mode; }

// One thread waits, through the product kernels' own bounded wait, on a barrier at which nothing ever arrives:
// the wait must give up after `limit_ns`, set the status bit and let the kernel return.  outcome[0] = 1 if the
// wait reported success (it must not), outcome[1] = the nanoseconds it took.
__global__ void wait_gives_up_kernel(int* status, unsigned long long limit_ns, long long* outcome) {
  __shared__ __align__(8) unsigned long long barrier;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&barrier), 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    const unsigned long long start = global_timer();
    const bool arrived = mbar_wait(smem_u32(&barrier), 0, status, &abort_flag, limit_ns);
    outcome[0] = arrived ? 1 : 0;
    outcome[1] = (long long)(global_timer() - start);
  }
}

// For tests of the status word: limits above 10 ms are refused, so nothing launched here can wait for long.
TGE_API int tge_wait_gives_up(int* status, long long limit_ns, long long* outcome, cudaStream_t stream) {
  TGE_REQUIRE(status != nullptr && outcome != nullptr, "wait_gives_up: null pointer");
  TGE_REQUIRE(limit_ns > 0 && limit_ns <= 10000000ll, "wait_gives_up: the limit must lie in (0, 10 ms], got %lld ns", limit_ns);
  wait_gives_up_kernel<<<1, 32, 0, stream>>>(status, (unsigned long long)limit_ns, outcome);
  return tge_launched("wait_gives_up", 1);
}
// What the product of these sizes would run as: out = {two SMs per tile?, token tile, stages, k-splits}.
TGE_API void tge_gemm_tcgen05_describe(int M, int N, int K, int* out) {
  const Plan plan = make_plan(M, N, K, (long long)1 << 60, 0, 0);
  Plan pair_plan;
  const bool pair = choose_pair(M, N, K, (long long)1 << 60, plan, 0, 0, &pair_plan);
  const Plan& used = pair ? pair_plan : plan;
  out[0] = pair ? 1 : 0; out[1] = used.bn; out[2] = used.stages; out[3] = used.splits;
}
// How many pairs of SMs the pair kernel occupies at once (0: it cannot run here or is switched off).
TGE_API int tge_gemm_tcgen05_pair_capacity() { return pair_capacity(); }

// How many float32 of scratch the product would like (0 when it will not split along k).
TGE_API long long tge_gemm_tcgen05_scratch_floats(int M, int N, int K) {
  const Plan plan = make_plan(M, N, K, (long long)1 << 60, 0, 0);
  int splits = plan.splits;
  Plan pair_plan;
  if (choose_pair(M, N, K, (long long)1 << 60, plan, 0, 0, &pair_plan) && pair_plan.splits > splits) splits = pair_plan.splits;
  return splits > 1 ? (long long)splits * M * N : 0;
}

namespace {

// Launches the product kernel.  With `partial_always` (or when the plan cuts k) the kernel leaves
// float32 partial sums [splits, M, N] in `scratch` and *splits_out tells how many; the caller then
// runs the kernel that adds them up.  Returns 1 (one kernel launched), TGE_UNSUPPORTED, or an error.
int launch_product(const void* x, long long ldx, const void* w, long long ldw, const float* bias, void* out,
                   long long ldo, int M, int N, int K, int epilogue, float* scratch, long long scratch_floats,
                   int force_bn, int force_splits, bool partial_always, int* status, cudaStream_t stream,
                   int* splits_out, const RowSums& sums = RowSums()) {
  if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || (uintptr_t)x % 16 != 0 || (uintptr_t)w % 16 != 0) return TGE_UNSUPPORTED;
  if (scratch == nullptr) scratch_floats = 0;
  const Plan plan = make_plan(M, N, K, scratch_floats, force_bn, force_splits);
  const bool to_partial = partial_always || plan.splits > 1;
  TGE_REQUIRE(!to_partial || (long long)plan.splits * M * N <= scratch_floats,
              "gemm_tcgen05: %d k-splits need %lld floats of scratch, have %lld", plan.splits,
              (long long)plan.splits * M * N, scratch_floats);

  CUtensorMap map_w, map_x;
  int rc = make_map(&map_w, w, N, K, ldw, BM, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
  if (rc != 0) return rc;

  TGE_REQUIRE(sums.ss == nullptr || (M <= DEFER_MAX_TOKENS && sums.slices > 0 && sums.width > 0),
              "gemm_tcgen05: rows without their norm factor: at most %d tokens, got %d", DEFER_MAX_TOKENS, M);
  Plan pair_plan;
  if (sums.ss == nullptr && choose_pair(M, N, K, scratch_floats, plan, force_bn, force_splits, &pair_plan)) {
    const bool pair_partial = partial_always || pair_plan.splits > 1;
    TGE_REQUIRE(!pair_partial || (long long)pair_plan.splits * M * N <= scratch_floats,
                "gemm_tcgen05: %d k-splits need %lld floats of scratch, have %lld", pair_plan.splits,
                (long long)pair_plan.splits * M * N, scratch_floats);
    rc = make_map(&map_x, x, M, K, ldx, pair_plan.bn / 2, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != 0) return rc;
    GemmParams p;
    p.n_w = N; p.m_tok = M; p.K = K;
    p.bn = pair_plan.bn; p.stages = pair_plan.stages; p.splits = pair_plan.splits;
    p.k_blocks = (K + BK - 1) / BK;
    p.tiles_w = (N + PAIR_BM - 1) / PAIR_BM;
    p.tiles_t = (M + pair_plan.bn - 1) / pair_plan.bn;
    p.epilogue = epilogue;
    int cols = 32;
    while (cols < 2 * pair_plan.bn) cols *= 2;
    p.acc_cols = cols;
    p.to_partial = pair_partial ? 1 : 0;
    p.bias = bias; p.out = out; p.ldo = ldo; p.partial = scratch; p.status = status;
    p.ss = nullptr; p.ss_slices = 0; p.ss_width = 0; p.ss_eps = 0.0f;
    const size_t smem = 1024 + (size_t)pair_plan.stages * (A_STAGE_BYTES + (pair_plan.bn / 2) * BK * 2) +
                        8 * (2 * pair_plan.stages + 4) + 16;
    const long long total = (long long)p.tiles_w * p.tiles_t * p.splits;
    const int pairs = pair_capacity();
    const int grid = 2 * (int)(total < pairs ? total : pairs);
    tge_launch_clusters(gemm_tcgen05_pair_kernel, grid, NUM_THREADS, smem, 2, stream, map_w, map_x, p);
    rc = tge_check_launch("gemm_tcgen05_pair");
    if (rc != 0) return rc;
    *splits_out = pair_partial ? pair_plan.splits : 0;
    return 1;
  }

  rc = make_map(&map_x, x, M, K, ldx, plan.bn, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
  if (rc != 0) return rc;

  GemmParams p;
  p.n_w = N; p.m_tok = M; p.K = K;
  p.bn = plan.bn; p.stages = plan.stages; p.splits = plan.splits;
  p.k_blocks = (K + BK - 1) / BK;
  p.tiles_w = (N + BM - 1) / BM;
  p.tiles_t = (M + plan.bn - 1) / plan.bn;
  p.epilogue = epilogue;
  int cols = 32;
  while (cols < 2 * plan.bn) cols *= 2;
  p.acc_cols = cols;
  p.to_partial = to_partial ? 1 : 0;
  p.bias = bias; p.out = out; p.ldo = ldo; p.partial = scratch; p.status = status;
  p.ss = sums.ss; p.ss_slices = sums.slices; p.ss_width = sums.width; p.ss_eps = sums.eps;

  const size_t smem = 1024 + (size_t)plan.stages * (A_STAGE_BYTES + plan.bn * BK * 2) + 8 * (2 * plan.stages + 4) + 16 +
                      DEFER_MAX_TOKENS * sizeof(float);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t err = cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
    if (err != cudaSuccess) {
      tge_set_error("gemm_tcgen05: cannot reserve shared memory: %s", cudaGetErrorString(err));
      return -2;
    }
    configured = SMEM_LIMIT;
  }
  const long long total = (long long)p.tiles_w * p.tiles_t * p.splits;
  const int grid = (int)(total < sm_count() ? total : sm_count());
  tge_launch(gemm_tcgen05_kernel, grid, NUM_THREADS, smem, stream, map_w, map_x, p);
  rc = tge_check_launch("gemm_tcgen05");
  if (rc != 0) return rc;
  *splits_out = to_partial ? plan.splits : 0;
  return 1;
}

// One block per token adds the k-split partial sums (+ bias) into the float32 stream and writes
// RMSNorm(row) * weight for the next product.  (Eight blocks per row as a cluster that met through
// distributed shared memory took 8.8 us after the o projection at batch 8, two 7.5 us, one block 7 us:
// the cluster's barriers cost more than the parallelism gave.)
constexpr int NORM_THREADS = 1024;
constexpr int NORM_PER_THREAD = 8;               // columns per thread: rows up to 1024 * 8 = 8192 wide

__global__ void __launch_bounds__(NORM_THREADS)
splitk_add_norm_kernel(const float* __restrict__ partial, const float* __restrict__ bias, float* __restrict__ stream,
                       long long ld_stream, const float* __restrict__ norm_weight, float eps,
                       __nv_bfloat16* __restrict__ norm_out, long long ld_norm, int m_tok, int n_w, int splits) {
  __shared__ float scratch[32];
  pdl_trigger();
  const int t = blockIdx.x;
  const size_t plane = (size_t)m_tok * n_w;
  // constants of the model first: they do not depend on the previous kernel
  float gain[NORM_PER_THREAD], add[NORM_PER_THREAD], value[NORM_PER_THREAD];
#pragma unroll
  for (int i = 0; i < NORM_PER_THREAD; ++i) {
    const int n = threadIdx.x + i * NORM_THREADS;
    gain[i] = n < n_w ? norm_weight[n] : 0.0f;
    add[i] = (bias && n < n_w) ? bias[n] : 0.0f;
  }
  pdl_wait();
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < NORM_PER_THREAD; ++i) {
    const int n = threadIdx.x + i * NORM_THREADS;
    value[i] = 0.0f;
    if (n < n_w) {
      const float* src = partial + (size_t)t * n_w + n;
      float acc = 0.0f;
#pragma unroll 4
      for (int s = 0; s < splits; ++s) acc += src[s * plane];
      const float v = stream[(size_t)t * ld_stream + n] + (acc + add[i]);
      stream[(size_t)t * ld_stream + n] = v;
      value[i] = v;
      sum = fmaf(v, v, sum);
    }
  }
  sum = block_sum(sum, scratch);
  const float scale = 1.0f / sqrtf(sum / (float)n_w + eps);
#pragma unroll
  for (int i = 0; i < NORM_PER_THREAD; ++i) {
    const int n = threadIdx.x + i * NORM_THREADS;
    if (n < n_w) norm_out[(size_t)t * ld_norm + n] = __float2bfloat16_rn(value[i] * scale * gain[i]);
  }
}

// One block per (token, head): the head's q, k or v values = sum of the partial sums + bias; a query head is
// rotated into the qkv buffer, a key head rotated into its page, a value head copied into its page
// (formulas as in the stand-alone rotate-and-store kernel).
__global__ void splitk_qkv_rope_store_kernel(const float* __restrict__ partial, const float* __restrict__ bias,
                                             __nv_bfloat16* __restrict__ qkv, long long ld_qkv, int m_tok, int n_w,
                                             int splits, const float* __restrict__ cos_table,
                                             const float* __restrict__ sin_table, int table_rows, int rotary,
                                             const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                             const int* __restrict__ block_table, int max_pages,
                                             __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                                             int num_pages, int page_size, int heads, int kv_heads, int head_dim,
                                             int* status, const float* __restrict__ ss, int ss_slices, int ss_width,
                                             float ss_eps) {
  extern __shared__ float head_values[];
  pdl_trigger();
  const int t = blockIdx.x, unit = blockIdx.y;     // unit: query heads, then key heads, then value heads
  const size_t plane = (size_t)m_tok * n_w;
  const int column0 = unit * head_dim;
  // What the step was given and the model's constants are read while the product before this kernel still
  // runs: the position and its angles, the page; only the partial sums (and the sums of squares) are its work.
  const int pos = positions[t];
  const int half = rotary / 2;
  const bool is_value = unit >= heads + kv_heads;
  const bool pos_ok = is_value || half == 0 || (pos >= 0 && pos < table_rows);
  int page = 0, page_index = 0;
  if (unit >= heads) {
    const int seq = seq_of_token[t];
    page_index = pos / page_size;
    page = (pos >= 0 && page_index < max_pages) ? block_table[(size_t)seq * max_pages + page_index] : -1;
  }
  // the angle of every dimension this thread will write (two dimensions per thread at most: head sizes up to 256)
  float angle_cos[2] = {1.0f, 1.0f}, angle_sin[2] = {0.0f, 0.0f};
  if (!is_value && pos_ok) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int d = (int)threadIdx.x + i * (int)blockDim.x;
      if (d < rotary) {
        const int j = d < half ? d : d - half;
        angle_cos[i] = cos_table[(size_t)pos * half + j];
        angle_sin[i] = sin_table[(size_t)pos * half + j];
      }
    }
  }
  pdl_wait();
  // the first sixteen slices' sums are asked for before the partial sums and used after them: one round trip
  float early[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) early[i] = (ss != nullptr && i < ss_slices) ? ss[(size_t)i * m_tok + t] : 0.0f;
  float factor = 1.0f;
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    const float* src = partial + (size_t)t * n_w + column0 + d;
    float acc = 0.0f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) acc += src[s * plane];
    if (ss != nullptr && d == (int)threadIdx.x) {
      float sum = 0.0f;
#pragma unroll
      for (int i = 0; i < 16; ++i) sum += early[i];
      for (int slice = 16; slice < ss_slices; ++slice) sum += ss[(size_t)slice * m_tok + t];
      factor = 1.0f / sqrtf(sum / (float)ss_width + ss_eps);
    }
    acc *= factor;
    if (bias) acc += bias[column0 + d];
    head_values[d] = acc;
  }
  __syncthreads();
  if (!pos_ok) {
    if (threadIdx.x == 0) atomicOr(status, TGE_STATUS_BAD_ROW);
    return;
  }
  auto rotated = [&](int d, int i) -> float {
    if (is_value || d >= rotary) return head_values[d];
    if (d < half) return head_values[d] * angle_cos[i] - head_values[d + half] * angle_sin[i];
    return head_values[d - half] * angle_sin[i] + head_values[d] * angle_cos[i];
  };
  __nv_bfloat16* dst;
  if (unit < heads) {
    dst = qkv + (size_t)t * ld_qkv + column0;
  } else {
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, TGE_STATUS_BAD_PAGE);
      return;
    }
    const int h = is_value ? unit - heads - kv_heads : unit - heads;
    dst = (is_value ? v_pages : k_pages) +
          (((size_t)page * kv_heads + h) * page_size + (pos - page_index * page_size)) * head_dim;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int d = (int)threadIdx.x + i * (int)blockDim.x;
    if (d < head_dim) dst[d] = __float2bfloat16_rn(rotated(d, i));
  }
}

// The add+norm kernel without the norm's factor: the stream takes the sums, the next product's input is
// stream * weight, and each block leaves the sum of squares of its slice of the row; whoever multiplies that
// input works the factor out of the slices' sums (always in slice order) and applies it to its result.  No
// block waits for another, so a row is spread over many SMs: 4 us in a step where the kernel above takes 7.
constexpr int SCALE_SLICE = 256;

__global__ void __launch_bounds__(SCALE_SLICE)
splitk_add_scale_kernel(const float* __restrict__ partial, const float* __restrict__ bias, float* __restrict__ stream,
                        long long ld_stream, const float* __restrict__ norm_weight, __nv_bfloat16* __restrict__ scaled_out,
                        long long ld_scaled, float* __restrict__ ss_out, int m_tok, int n_w, int splits) {
  __shared__ float scratch[32];
  pdl_trigger();
  const int t = blockIdx.y, n = blockIdx.x * SCALE_SLICE + threadIdx.x;
  const bool inside = n < n_w;
  const float gain = inside ? norm_weight[n] : 0.0f;
  const float add = (bias && inside) ? bias[n] : 0.0f;
  pdl_wait();
  float v = 0.0f;
  if (inside) {
    const size_t plane = (size_t)m_tok * n_w;
    const float* src = partial + (size_t)t * n_w + n;
    float acc = 0.0f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) acc += src[s * plane];
    v = stream[(size_t)t * ld_stream + n] + (acc + add);
    stream[(size_t)t * ld_stream + n] = v;
    scaled_out[(size_t)t * ld_scaled + n] = __float2bfloat16_rn(v * gain);
  }
  const float sum = block_sum(v * v, scratch);
  if (threadIdx.x == 0) ss_out[(size_t)blockIdx.x * m_tok + t] = sum;
}

constexpr int FUSED_MAX_TOKENS = 256;   // above this the product's own epilogue is the better path

}  // namespace

// x [M, K] bf16 (row stride ldx), w [N, K] bf16 (row stride ldw); bias float32 [N] or null;
// out per epilogue (row stride ldo elements).  scratch: float32 buffer of scratch_floats
// elements for split-k partial sums (may be null: no split).  force_bn / force_splits: 0 = automatic.
// Returns TGE_UNSUPPORTED (and touches nothing) when the shape cannot go through TMA: K not a
// multiple of 8, misaligned pointers or strides.  The caller then uses the CUDA-core product.
// x_ss (null, or float32 [x_ss_slices, M]): the rows of x still lack their RMSNorm factor
// 1 / sqrt(sum over slices / x_ss_width + x_ss_eps), which then multiplies the product before the bias.
TGE_API int tge_gemm_tcgen05(const void* x, long long ldx, const void* w, long long ldw, const float* bias, void* out,
                             long long ldo, int M, int N, int K, int epilogue, float* scratch,
                             long long scratch_floats, int force_bn, int force_splits, int* status,
                             const float* x_ss, int x_ss_slices, int x_ss_width, float x_ss_eps, cudaStream_t stream) {
  TGE_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
  TGE_REQUIRE(epilogue >= GEMM_STORE && epilogue <= GEMM_SWIGLU, "gemm: unknown epilogue %d", epilogue);
  TGE_REQUIRE(epilogue != GEMM_SWIGLU || N % 2 == 0, "gemm: the gated epilogue needs an even number of weight rows, got %d", N);
  TGE_REQUIRE(force_bn == 0 || (force_bn % 16 == 0 && force_bn >= 16 && force_bn <= 256), "gemm: token tile %d must be a multiple of 16 in [16, 256]", force_bn);
  TGE_REQUIRE(status != nullptr, "gemm_tcgen05: needs a status word");
  if (M == 0) return 0;
  int splits = 0;
  RowSums sums;
  sums.ss = x_ss; sums.slices = x_ss_slices; sums.width = x_ss_width; sums.eps = x_ss_eps;
  int rc = launch_product(x, ldx, w, ldw, bias, out, ldo, M, N, K, epilogue, scratch, scratch_floats, force_bn,
                          force_splits, false, status, stream, &splits, sums);
  if (rc != 1) return rc;
  if (splits > 0) {
    const long long count = epilogue == GEMM_SWIGLU ? (long long)M * N / 2 : (long long)M * N;
    long long blocks = (count + 255) / 256;
    if (blocks > sm_count() * 8) blocks = sm_count() * 8;
    tge_launch(splitk_epilogue_kernel, (int)blocks, 256, 0, stream, (const float*)scratch, bias, out, ldo, M, N, splits,
               epilogue, x_ss, x_ss_slices, x_ss_width, x_ss_eps);
    return tge_launched("splitk_epilogue", 2);
  }
  return 1;
}

// As tge_gemm_tcgen05_add_norm below, but the norm's factor is left to whoever multiplies the result next:
// stream [M, N] float32 += x . w^T (+ bias); scaled_out [M, N] bf16 = stream * norm_weight;
// ss_out float32 [tge_gemm_tcgen05_defer_slices(N), M] = the rows' sums of squares, in slices.  At most 128 tokens.
TGE_API int tge_gemm_tcgen05_defer_slices(int N) { return (N + SCALE_SLICE - 1) / SCALE_SLICE; }

TGE_API int tge_gemm_tcgen05_add_defer(const void* x, long long ldx, const void* w, long long ldw, const float* bias,
                                       float* stream_out, long long ldo, int M, int N, int K, const float* norm_weight,
                                       void* scaled_out, long long ld_scaled, float* ss_out, float* scratch,
                                       long long scratch_floats, int* status, cudaStream_t stream) {
  TGE_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm+defer: bad sizes M=%d N=%d K=%d", M, N, K);
  TGE_REQUIRE(status != nullptr && norm_weight != nullptr && scaled_out != nullptr && ss_out != nullptr, "gemm+defer: bad arguments");
  if (M == 0) return 0;
  if (M > DEFER_MAX_TOKENS || scratch == nullptr) return TGE_UNSUPPORTED;
  int splits = 0;
  int rc = launch_product(x, ldx, w, ldw, nullptr, stream_out, ldo, M, N, K, GEMM_ADD_F32, scratch, scratch_floats, 0, 0,
                          true, status, stream, &splits);
  if (rc != 1) return rc;
  tge_launch(splitk_add_scale_kernel, dim3((N + SCALE_SLICE - 1) / SCALE_SLICE, M), SCALE_SLICE, 0, stream,
             (const float*)scratch, bias, stream_out, ldo, norm_weight, (__nv_bfloat16*)scaled_out, ld_scaled, ss_out, M, N,
             splits);
  return tge_launched("splitk_add_scale", 2);
}

// stream [M, N] float32 += x . w^T (+ bias), then norm_out [M, N] bf16 = RMSNorm(stream rows) * norm_weight:
// the product leaves partial sums in scratch and one kernel per token row adds them into the stream and
// normalises the new row.  scratch must hold at least max(1, k-splits) * M * N floats.  Returns
// TGE_UNSUPPORTED for more than 256 tokens or shapes TMA cannot address (use the separate kernels then).
TGE_API int tge_gemm_tcgen05_add_norm(const void* x, long long ldx, const void* w, long long ldw, const float* bias,
                                      float* stream_out, long long ldo, int M, int N, int K, const float* norm_weight,
                                      float eps, void* norm_out, long long ld_norm, float* scratch,
                                      long long scratch_floats, int* status, cudaStream_t stream) {
  TGE_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm+norm: bad sizes M=%d N=%d K=%d", M, N, K);
  TGE_REQUIRE(status != nullptr && norm_weight != nullptr && norm_out != nullptr && eps > 0.0f, "gemm+norm: bad arguments");
  if (M == 0) return 0;
  if (M > FUSED_MAX_TOKENS || N > NORM_THREADS * NORM_PER_THREAD || scratch == nullptr) return TGE_UNSUPPORTED;
  int splits = 0;
  int rc = launch_product(x, ldx, w, ldw, nullptr, stream_out, ldo, M, N, K, GEMM_ADD_F32, scratch, scratch_floats, 0, 0,
                          true, status, stream, &splits);
  if (rc != 1) return rc;
  tge_launch(splitk_add_norm_kernel, dim3(M), NORM_THREADS, 0, stream,
             (const float*)scratch, bias, stream_out, ldo, norm_weight, eps, (__nv_bfloat16*)norm_out, ld_norm, M, N,
             splits);
  return tge_launched("splitk_add_norm", 2);
}

// The fused q/k/v product of an attention layer for a small batch: qkv = x . w^T + bias, q rotated into
// `qkv` (bf16 [M, >= heads*head_dim]), k rotated and v copied into their pages.  Same conditions and
// return codes as tge_gemm_tcgen05_add_norm; N must be (heads + 2 * kv_heads) * head_dim.
TGE_API int tge_gemm_tcgen05_qkv_rope(const void* x, long long ldx, const void* w, long long ldw, const float* bias,
                                      void* qkv, long long ld_qkv, int M, int N, int K, const float* cos_table,
                                      const float* sin_table, int table_rows, int rotary, const int* positions,
                                      const int* seq_of_token, const int* block_table, int max_pages, void* k_pages,
                                      void* v_pages, int num_pages, int page_size, int heads, int kv_heads,
                                      int head_dim, float* scratch, long long scratch_floats, int* status,
                                      const float* x_ss, int x_ss_slices, int x_ss_width, float x_ss_eps,
                                      cudaStream_t stream) {
  TGE_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm+rope: bad sizes M=%d N=%d K=%d", M, N, K);
  TGE_REQUIRE(N == (heads + 2 * kv_heads) * head_dim, "gemm+rope: %d weight rows are not (heads + 2 kv heads) * head_dim", N);
  TGE_REQUIRE(rotary >= 0 && rotary <= head_dim && rotary % 2 == 0, "gemm+rope: bad rotary width %d", rotary);
  TGE_REQUIRE(status != nullptr && page_size > 0 && max_pages > 0 && num_pages > 0, "gemm+rope: bad arguments");
  if (M == 0) return 0;
  if (M > FUSED_MAX_TOKENS || (size_t)N * sizeof(float) > 200 * 1024 || scratch == nullptr) return TGE_UNSUPPORTED;
  int splits = 0;
  int rc = launch_product(x, ldx, w, ldw, nullptr, qkv, ld_qkv, M, N, K, GEMM_STORE, scratch, scratch_floats, 0, 0, true,
                          status, stream, &splits);
  if (rc != 1) return rc;
  tge_launch(splitk_qkv_rope_store_kernel, dim3(M, heads + 2 * kv_heads), head_dim >= 128 ? 128 : 64,
             (size_t)head_dim * sizeof(float), stream, (const float*)scratch, bias, (__nv_bfloat16*)qkv, ld_qkv, M, N,
             splits, cos_table, sin_table, table_rows, rotary, positions, seq_of_token, block_table, max_pages,
             (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, num_pages, page_size, heads, kv_heads, head_dim, status,
             x_ss, x_ss_slices, x_ss_width, x_ss_eps);
  return tge_launched("splitk_qkv_rope_store", 2);
}
