// Paged causal GQA attention for the bfloat16 path, compiled per head size
// (-DTGE_HEAD_DIM=...).  One kernel serves prompt portions and decode rows.
//
// A block owns one tile of query rows of one kv head of one portion: the rows
// are (query, head-of-group) pairs, query-major, so every K/V tile fetched
// from the pages is used by all the query heads that share it (the structure
// of the reference's group kernel, src/cpu/scalar/attention_scalar.cpp:117-199).
// K/V stream through shared memory in tiles of 64 positions (page-aligned; one
// page-table lookup per 16-byte chunk copy, hoisted out of the inner product),
// scores and the running maximum/sum are float32 (online softmax, the same
// update the reference uses when it merges chunk states,
// src/models/qwen2.cpp:1469-1522), P is rounded to bfloat16 only as the
// operand of the P.V product.  With more than one split along the keys a block
// writes its unnormalised state (m, l, acc) and a second kernel merges the
// splits in split order.
//
// Masking is by absolute position: key t is visible to the query at position p
// when t <= p and, with a window w > 0, t > p - w.
#include <cuda.h>

#include <stdlib.h>

#include <map>
#include <tuple>

#include "common.cuh"

#ifndef TGE_HEAD_DIM
#error "compile with -DTGE_HEAD_DIM=<multiple of 16>"
#endif

namespace {

constexpr int HD = TGE_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 up to 256");
constexpr int BKV = 64;              // key positions per shared-memory tile
constexpr int ROW_ELEMS = HD + 8;    // padded row: an odd count of 16-byte chunks keeps ldmatrix conflict-free
constexpr int CHUNKS = HD / 8;       // 16-byte chunks per row

struct AttnParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k_pages;
  const __nv_bfloat16* v_pages;
  const int* block_table;
  const int* q_start;
  const int* start_pos;
  __nv_bfloat16* out;
  float* partial_o;
  float* partial_ml;
  int* status;
  int q_stride, out_stride;
  int max_pages, num_pages, page_size, page_shift;
  int num_seqs, total_tokens;
  int early_tiles;           // decode: key tiles of settled positions asked for before the dependency wait (0: none)
  int heads, kv_heads, group, bq;
  int window, split_tokens, num_splits;
  float scale_log2;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Copies positions [k0, k0 + BKV) of one kv head into a shared tile; positions
// outside [lo, hi) are zero-filled so that masked columns never meet NaNs.
template <int NWARPS>
__device__ __forceinline__ void load_tile(const AttnParams& p, const __nv_bfloat16* pages, const int* table, int kvh,
                                          __nv_bfloat16* tile, int k0, int lo, int hi, bool& bad_page) {
  for (int c = threadIdx.x; c < BKV * CHUNKS; c += NWARPS * 32) {
    const int j = c / CHUNKS, part = c - j * CHUNKS;
    const int kpos = k0 + j;
    const uint32_t dst = smem_u32(tile + j * ROW_ELEMS + part * 8);
    const void* src = pages;
    int bytes = 0;
    if (kpos >= lo && kpos < hi) {
      const int page_index = kpos >> p.page_shift;
      const int page = page_index < p.max_pages ? table[page_index] : -1;
      if (page >= 0 && page < p.num_pages) {
        src = pages + ((((size_t)page * p.kv_heads + kvh) << p.page_shift) + (kpos & (p.page_size - 1))) * HD + part * 8;
        bytes = 16;
      } else {
        bad_page = true;
      }
    }
    cp_async16(dst, src, bytes);
  }
}

template <int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32) attention_mma_kernel(const AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [2][BKV][ROW_ELEMS]
  __nv_bfloat16* sV = sK + 2 * BKV * ROW_ELEMS;                             // [2][BKV][ROW_ELEMS]
  __shared__ int tile_info[2];
  pdl_trigger();
  pdl_wait();

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int kvh = blockIdx.y, split = blockIdx.z;

  // which portion and which tile of its queries this block owns
  if (tid == 0) {
    int remaining = blockIdx.x, seq = -1, tile = 0;
    for (int s = 0; s < p.num_seqs; ++s) {
      const int q_len = p.q_start[s + 1] - p.q_start[s];
      const int tiles = (q_len + p.bq - 1) / p.bq;
      if (remaining < tiles) { seq = s; tile = remaining; break; }
      remaining -= tiles;
    }
    tile_info[0] = seq;
    tile_info[1] = tile;
  }
  __syncthreads();
  const int seq = tile_info[0];
  if (seq < 0) return;
  const int q_first = tile_info[1] * p.bq;                 // first query of the tile, within the portion
  const int q_begin = p.q_start[seq];
  const int q_len = p.q_start[seq + 1] - q_begin;
  const int q_count = min(p.bq, q_len - q_first);
  const int pos0 = p.start_pos[seq] + q_first;             // position of the tile's first query
  const int* table = p.block_table + (size_t)seq * p.max_pages;

  // key range of the block: union over its rows, cut to this split
  int lo = p.window > 0 ? max(pos0 - p.window + 1, 0) : 0;
  int hi = pos0 + q_count;                                 // exclusive
  if (p.num_splits > 1) {
    lo = max(lo, split * p.split_tokens);
    hi = min(hi, (split + 1) * p.split_tokens);
  }
  if (lo >= hi) return;

  // this thread's two rows
  int row_token[2], row_pos[2], row_head[2];
  bool row_valid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = warp * 16 + g8 + 8 * i;
    const int qi = r / p.group, gg = r - qi * p.group;
    row_valid[i] = qi < q_count;
    row_token[i] = q_begin + q_first + (row_valid[i] ? qi : 0);
    row_pos[i] = pos0 + qi;
    row_head[i] = kvh * p.group + gg;
  }

  // Q fragments (A operand), straight from global memory
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int kc = 0; kc < HD / 16; ++kc) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const __nv_bfloat16* src = p.q + (size_t)row_token[i] * p.q_stride + (size_t)row_head[i] * HD + kc * 16 + 2 * t4;
      qf[kc][i] = row_valid[i] ? *reinterpret_cast<const uint32_t*>(src) : 0u;
      qf[kc][i + 2] = row_valid[i] ? *reinterpret_cast<const uint32_t*>(src + 8) : 0u;
    }
  }

  float o_acc[HD / 8][4];
#pragma unroll
  for (int d = 0; d < HD / 8; ++d)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_acc[d][e] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

  bool bad_page = false;
  const int k_first = lo / BKV * BKV;
  const int num_tiles = (hi - k_first + BKV - 1) / BKV;
  load_tile<NWARPS>(p, p.k_pages, table, kvh, sK, k_first, lo, hi, bad_page);
  load_tile<NWARPS>(p, p.v_pages, table, kvh, sV, k_first, lo, hi, bad_page);
  cp_async_commit();

  for (int it = 0; it < num_tiles; ++it) {
    const int stage = it & 1;
    const int k0 = k_first + it * BKV;
    if (it + 1 < num_tiles) {
      load_tile<NWARPS>(p, p.k_pages, table, kvh, sK + (stage ^ 1) * BKV * ROW_ELEMS, k0 + BKV, lo, hi, bad_page);
      load_tile<NWARPS>(p, p.v_pages, table, kvh, sV + (stage ^ 1) * BKV * ROW_ELEMS, k0 + BKV, lo, hi, bad_page);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* tK = sK + stage * BKV * ROW_ELEMS;
    const __nv_bfloat16* tV = sV + stage * BKV * ROW_ELEMS;

    // S = Q K^T for 16 rows x 64 keys
    float s_acc[BKV / 8][4];
#pragma unroll
    for (int n = 0; n < BKV / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s_acc[n][e] = 0.0f;
#pragma unroll
    for (int kc = 0; kc < HD / 16; ++kc) {
#pragma unroll
      for (int nt = 0; nt < BKV / 8; nt += 2) {
        const int mi = lane >> 3;
        const int n = (nt + (mi >> 1)) * 8 + (lane & 7);
        const int kofs = kc * 16 + (mi & 1) * 8;
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4(smem_u32(tK + n * ROW_ELEMS + kofs), r0, r1, r2, r3);
        mma_bf16(s_acc[nt], qf[kc], r0, r1);
        mma_bf16(s_acc[nt + 1], qf[kc], r2, r3);
      }
    }

    // mask, running maximum, exponentials (float32, base-2 with the scale folded in)
    float m_new[2], corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int first_key = p.window > 0 ? row_pos[i] - p.window + 1 : 0;
      float mx = -INFINITY;
#pragma unroll
      for (int n = 0; n < BKV / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kpos = k0 + n * 8 + 2 * t4 + e;
          const bool visible = row_valid[i] && kpos <= row_pos[i] && kpos >= first_key && kpos >= lo && kpos < hi;
          const float s = visible ? s_acc[n][2 * i + e] * p.scale_log2 : -INFINITY;
          s_acc[n][2 * i + e] = s;
          mx = fmaxf(mx, s);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      m_new[i] = fmaxf(m_run[i], mx);
      const float m_use = m_new[i] == -INFINITY ? 0.0f : m_new[i];
      corr[i] = exp2f(m_run[i] - m_use);
      float sum = 0.0f;
#pragma unroll
      for (int n = 0; n < BKV / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float pv = exp2f(s_acc[n][2 * i + e] - m_use);
          s_acc[n][2 * i + e] = pv;
          sum += pv;
        }
      }
      l_run[i] = l_run[i] * corr[i] + sum;
      m_run[i] = m_new[i];
    }
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) {
      o_acc[d][0] *= corr[0]; o_acc[d][1] *= corr[0];
      o_acc[d][2] *= corr[1]; o_acc[d][3] *= corr[1];
    }

    // O += P V
#pragma unroll
    for (int kk = 0; kk < BKV / 16; ++kk) {
      uint32_t pf[4];
      pf[0] = pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]);
      pf[1] = pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]);
      pf[2] = pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]);
      pf[3] = pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]);
#pragma unroll
      for (int dt = 0; dt < HD / 8; dt += 2) {
        const int mi = lane >> 3;
        const int key = kk * 16 + (mi & 1) * 8 + (lane & 7);
        const int d = (dt + (mi >> 1)) * 8;
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4_trans(smem_u32(tV + key * ROW_ELEMS + d), r0, r1, r2, r3);
        mma_bf16(o_acc[dt], pf, r0, r1);
        mma_bf16(o_acc[dt + 1], pf, r2, r3);
      }
    }
    __syncthreads();
  }
  if (bad_page && p.status) atomicOr(p.status, TGE_STATUS_BAD_PAGE);

  // finish: total the sums over the four lanes that share a row
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!row_valid[i]) continue;
    if (p.num_splits == 1) {
      const float inv = l_run[i] > 0.0f ? 1.0f / l_run[i] : 0.0f;
      __nv_bfloat16* dst = p.out + (size_t)row_token[i] * p.out_stride + (size_t)row_head[i] * HD;
#pragma unroll
      for (int d = 0; d < HD / 8; ++d) {
        *reinterpret_cast<uint32_t*>(dst + d * 8 + 2 * t4) =
            pack_bf16(o_acc[d][2 * i] * inv, o_acc[d][2 * i + 1] * inv);
      }
    } else {
      const size_t slot = ((size_t)split * p.total_tokens + row_token[i]) * p.heads + row_head[i];
      float* dst = p.partial_o + slot * HD;
#pragma unroll
      for (int d = 0; d < HD / 8; ++d) {
        *reinterpret_cast<float2*>(dst + d * 8 + 2 * t4) = make_float2(o_acc[d][2 * i], o_acc[d][2 * i + 1]);
      }
      if (t4 == 0) {
        p.partial_ml[slot * 2] = m_run[i];
        p.partial_ml[slot * 2 + 1] = l_run[i];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Decode: every portion is one token.  A block owns one (request, kv head, split)
// and its 16 rows are the query heads of the group (padded).  The four warps
// share each 64-position tile: warp w takes positions [16w, 16w+16) with its own
// running maximum and sum, tiles arrive through a three-stage cp.async ring, and
// the four states are merged through shared memory at the end, in warp order.
// ---------------------------------------------------------------------------
constexpr int DEC_WARPS = 4;
constexpr int DEC_STAGES = 3;
constexpr int STAGE_ELEMS = 2 * BKV * ROW_ELEMS;   // K tile then V tile

__global__ void __launch_bounds__(DEC_WARPS * 32) attention_decode_kernel(const AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* stages = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int token = p.q_start[seq];
  const int pos = p.start_pos[seq];

  int lo = p.window > 0 ? max(pos - p.window + 1, 0) : 0;
  int hi = pos + 1;
  if (p.num_splits > 1) {
    lo = max(lo, split * p.split_tokens);
    hi = min(hi, (split + 1) * p.split_tokens);
  }
  if (lo >= hi) return;

  // The page ids of this block's key range, fetched once: the copy loops then index shared memory.
  // (The staged row is addressed like the global one, so ids before first_page are never read.)
  int* local_table = reinterpret_cast<int*>(smem_raw + (size_t)DEC_STAGES * STAGE_ELEMS * sizeof(__nv_bfloat16));
  const int first_page = lo >> p.page_shift, last_page = (hi - 1) >> p.page_shift;
  for (int i = first_page + tid; i <= last_page; i += DEC_WARPS * 32)
    local_table[i - first_page] = i < p.max_pages ? p.block_table[(size_t)seq * p.max_pages + i] : -1;
  __syncthreads();
  const int* table = local_table - first_page;

  // Q fragments: rows are the heads of the group
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int kc = 0; kc < HD / 16; ++kc) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = g8 + 8 * i;
      const bool valid = r < p.group;
      const __nv_bfloat16* src = p.q + (size_t)token * p.q_stride + (size_t)(kvh * p.group + (valid ? r : 0)) * HD + kc * 16 + 2 * t4;
      qf[kc][i] = valid ? *reinterpret_cast<const uint32_t*>(src) : 0u;
      qf[kc][i + 2] = valid ? *reinterpret_cast<const uint32_t*>(src + 8) : 0u;
    }
  }
  float o_acc[HD / 8][4];
#pragma unroll
  for (int d = 0; d < HD / 8; ++d)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_acc[d][e] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

  bool bad_page = false;
  const int k_first = lo / BKV * BKV;
  const int num_tiles = (hi - k_first + BKV - 1) / BKV;
#pragma unroll
  for (int s = 0; s < DEC_STAGES - 1; ++s) {
    if (s < num_tiles) {
      load_tile<DEC_WARPS>(p, p.k_pages, table, kvh, stages + s * STAGE_ELEMS, k_first + s * BKV, lo, hi, bad_page);
      load_tile<DEC_WARPS>(p, p.v_pages, table, kvh, stages + s * STAGE_ELEMS + BKV * ROW_ELEMS, k_first + s * BKV, lo, hi, bad_page);
    }
    cp_async_commit();
  }
  for (int it = 0; it < num_tiles; ++it) {
    cp_async_wait<DEC_STAGES - 2>();
    __syncthreads();
    {
      const int next = it + DEC_STAGES - 1;
      if (next < num_tiles) {
        __nv_bfloat16* dst = stages + (next % DEC_STAGES) * STAGE_ELEMS;
        load_tile<DEC_WARPS>(p, p.k_pages, table, kvh, dst, k_first + next * BKV, lo, hi, bad_page);
        load_tile<DEC_WARPS>(p, p.v_pages, table, kvh, dst + BKV * ROW_ELEMS, k_first + next * BKV, lo, hi, bad_page);
      }
      cp_async_commit();
    }
    const __nv_bfloat16* tK = stages + (it % DEC_STAGES) * STAGE_ELEMS;
    const __nv_bfloat16* tV = tK + BKV * ROW_ELEMS;
    const int k0 = k_first + it * BKV + warp * 16;     // this warp's 16 positions
    if (k0 >= hi || k0 + 16 <= lo) continue;            // nothing visible in this slice (warp-uniform)

    float s_acc[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s_acc[n][e] = 0.0f;
#pragma unroll
    for (int kc = 0; kc < HD / 16; ++kc) {
      const int mi = lane >> 3;
      const int n = warp * 16 + (mi >> 1) * 8 + (lane & 7);
      const int kofs = kc * 16 + (mi & 1) * 8;
      uint32_t r0, r1, r2, r3;
      ldmatrix_x4(smem_u32(tK + n * ROW_ELEMS + kofs), r0, r1, r2, r3);
      mma_bf16(s_acc[0], qf[kc], r0, r1);
      mma_bf16(s_acc[1], qf[kc], r2, r3);
    }
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const bool row_valid = g8 + 8 * i < p.group;
      float mx = -INFINITY;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kpos = k0 + n * 8 + 2 * t4 + e;
          const bool visible = row_valid && kpos >= lo && kpos < hi;
          const float sv = visible ? s_acc[n][2 * i + e] * p.scale_log2 : -INFINITY;
          s_acc[n][2 * i + e] = sv;
          mx = fmaxf(mx, sv);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[i], mx);
      const float m_use = m_new == -INFINITY ? 0.0f : m_new;
      corr[i] = exp2f(m_run[i] - m_use);
      float sum = 0.0f;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float pv = exp2f(s_acc[n][2 * i + e] - m_use);
          s_acc[n][2 * i + e] = pv;
          sum += pv;
        }
      }
      l_run[i] = l_run[i] * corr[i] + sum;
      m_run[i] = m_new;
    }
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) {
      o_acc[d][0] *= corr[0]; o_acc[d][1] *= corr[0];
      o_acc[d][2] *= corr[1]; o_acc[d][3] *= corr[1];
    }
    uint32_t pf[4];
    pf[0] = pack_bf16(s_acc[0][0], s_acc[0][1]);
    pf[1] = pack_bf16(s_acc[0][2], s_acc[0][3]);
    pf[2] = pack_bf16(s_acc[1][0], s_acc[1][1]);
    pf[3] = pack_bf16(s_acc[1][2], s_acc[1][3]);
#pragma unroll
    for (int dt = 0; dt < HD / 8; dt += 2) {
      const int mi = lane >> 3;
      const int key = warp * 16 + (mi & 1) * 8 + (lane & 7);
      const int d = (dt + (mi >> 1)) * 8;
      uint32_t r0, r1, r2, r3;
      ldmatrix_x4_trans(smem_u32(tV + key * ROW_ELEMS + d), r0, r1, r2, r3);
      mma_bf16(o_acc[dt], pf, r0, r1);
      mma_bf16(o_acc[dt + 1], pf, r2, r3);
    }
  }
  cp_async_wait<0>();
  __syncthreads();                                      // every warp is done with the stages: reuse them
  if (bad_page && p.status) atomicOr(p.status, TGE_STATUS_BAD_PAGE);

  float* merge_o = reinterpret_cast<float*>(smem_raw);                  // [warps][16][HD]
  float* merge_ml = merge_o + DEC_WARPS * 16 * HD;                      // [warps][16][2]
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    const int r = g8 + 8 * i;
    float* dst = merge_o + ((size_t)warp * 16 + r) * HD;
#pragma unroll
    for (int d = 0; d < HD / 8; ++d)
      *reinterpret_cast<float2*>(dst + d * 8 + 2 * t4) = make_float2(o_acc[d][2 * i], o_acc[d][2 * i + 1]);
    if (t4 == 0) {
      merge_ml[(warp * 16 + r) * 2] = m_run[i];
      merge_ml[(warp * 16 + r) * 2 + 1] = l_run[i];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < p.group * HD; idx += DEC_WARPS * 32) {
    const int r = idx / HD, d = idx - r * HD;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, merge_ml[(w * 16 + r) * 2]);
    const float m_use = m == -INFINITY ? 0.0f : m;
    float l = 0.0f, acc = 0.0f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float scale = exp2f(merge_ml[(w * 16 + r) * 2] - m_use);
      l += scale * merge_ml[(w * 16 + r) * 2 + 1];
      acc += scale * merge_o[((size_t)w * 16 + r) * HD + d];
    }
    const int head = kvh * p.group + r;
    if (p.num_splits == 1) {
      p.out[(size_t)token * p.out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
    } else {
      const size_t slot = ((size_t)split * p.total_tokens + token) * p.heads + head;
      p.partial_o[slot * HD + d] = acc;
      if (d == 0) {
        p.partial_ml[slot * 2] = m;
        p.partial_ml[slot * 2 + 1] = l;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Decode for head sizes that are multiples of 64: the same block and warp layout as above, but the
// tiles come by TMA.  The page pool of a layer is one 2-D tensor [pages * kv_heads * page_size,
// head_dim]; one box is one page of one kv head by 64 columns (128 bytes, 128-byte swizzle), so a
// tile of 64 positions is 64 / page_size boxes per 64-column block for K and as many for V, issued by
// one thread and counted by an mbarrier per stage.  ldmatrix addresses apply the same swizzle.
// Stages are cleared once at the start: boxes of pages a request does not own are never fetched,
// and what masked columns multiply must be finite.
// ---------------------------------------------------------------------------
#if TGE_HEAD_DIM % 64 == 0
constexpr int TMA_BLOCKS = HD / 64;                       // 64-column blocks per row
constexpr int TMA_TILE_BYTES = BKV * HD * 2;              // one K (or V) tile
constexpr int TMA_STAGE_BYTES = 2 * TMA_TILE_BYTES;
constexpr int DEC_TMA_THREADS = (DEC_WARPS + 1) * 32;    // computing warps and one loading warp

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
// Bounded wait: gives up after about two seconds, records it, and lets the caller go on.
__device__ __forceinline__ void mbar_wait_bounded(uint32_t bar, uint32_t parity, int* status) {
  if (mbar_try_wait(bar, parity)) return;
  unsigned long long start;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(start));
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return;
    if ((spin & 1023u) == 0) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
      if (now - start > 2000000000ull) {
        if (status) atomicOr(status, TGE_STATUS_WAIT_TIMEOUT);
        return;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}

// byte offset of the 16-byte chunk holding columns [col, col + 8) of row `row` inside a swizzled tile
__device__ __forceinline__ uint32_t swizzled(int row, int col) {
  const int block = col >> 6, chunk = (col & 63) >> 3;
  return (uint32_t)(block * (BKV * 128) + row * 128 + ((chunk ^ (row & 7)) << 4));
}

// GROUPS: groups of four computing warps.  One group takes every tile; two groups take alternate tiles (the ring then
// has four stages, each always used by the same group), which doubles what one block pulls out of memory: for
// launches of no more blocks than SMs, where a block has its SM to itself.
template <int GROUPS>
__global__ void __launch_bounds__((4 * GROUPS + 1) * 32) attention_decode_tma_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  constexpr int WARPS = 4 * GROUPS, STAGES = GROUPS == 1 ? DEC_STAGES : 4, THREADS = (WARPS + 1) * 32;
  static_assert(STAGES % GROUPS == 0, "a stage must always serve the same group");
  extern __shared__ unsigned char smem_dyn[];
  pdl_trigger();
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;                       // swizzle atoms are 1024 bytes
  unsigned char* generic = smem_dyn + (base - raw);
  const uint32_t bars = base + STAGES * TMA_STAGE_BYTES;          // full[stages], then empty[stages]
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  int* local_table = reinterpret_cast<int*>(generic + STAGES * TMA_STAGE_BYTES + 64);

  const int tid = threadIdx.x, lane = tid & 31, warp = uniform_warp_index();
  const int g8 = lane >> 2, t4 = lane & 3;
  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int token = p.q_start[seq];
  const int pos = p.start_pos[seq];
  int lo = p.window > 0 ? max(pos - p.window + 1, 0) : 0;
  int hi = pos + 1;
  if (p.num_splits > 1) {
    lo = max(lo, split * p.split_tokens);
    hi = min(hi, (split + 1) * p.split_tokens);
  }
  if (lo >= hi) return;

  const int k_first = lo / BKV * BKV;
  const int num_tiles = (hi - k_first + BKV - 1) / BKV;
  const int first_page = k_first >> p.page_shift;
  const int last_page = (k_first + num_tiles * BKV - 1) >> p.page_shift;
  for (int i = first_page + tid; i <= last_page; i += THREADS) {
    int page = i < p.max_pages ? p.block_table[(size_t)seq * p.max_pages + i] : -1;
    if (page >= p.num_pages) page = -2;                                // reported below, never fetched
    local_table[i - first_page] = page;
  }
  {
    uint4* fill = reinterpret_cast<uint4*>(generic);
    for (int i = tid; i < STAGES * TMA_STAGE_BYTES / 16; i += THREADS) fill[i] = make_uint4(0, 0, 0, 0);
  }
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");       // the cleared stages, before TMA writes them
  __syncthreads();
  // All of the above read only what the step was given (lengths, the block table), which no kernel of the step
  // writes: it ran while the kernel before this one finished.  The queries and the newest keys and values are
  // that kernel's work; the keys and values of earlier positions are earlier steps' work, so the loading warp
  // asks for a ring of those tiles first and only then waits for the kernel before this one.

  const int pages_per_tile = BKV >> p.page_shift;
  auto issue = [&](int tile) {                                          // the loading warp's first lane only
    const int stage = tile % STAGES;
    const uint32_t k_dst = base + stage * TMA_STAGE_BYTES, v_dst = k_dst + TMA_TILE_BYTES;
    const uint32_t bar = full_bar(stage);
    int boxes = 0;
    for (int j = 0; j < pages_per_tile; ++j) {
      const int page = local_table[((k_first + tile * BKV) >> p.page_shift) + j - first_page];
      if (page >= 0 && (k_first + tile * BKV + (j << p.page_shift)) < hi) ++boxes;
    }
    mbar_expect_tx(bar, (uint32_t)boxes * 2u * TMA_BLOCKS * (uint32_t)(p.page_size * 128));
    for (int j = 0; j < pages_per_tile; ++j) {
      const int page = local_table[((k_first + tile * BKV) >> p.page_shift) + j - first_page];
      if (page < 0 || (k_first + tile * BKV + (j << p.page_shift)) >= hi) continue;
      const int row = (page * p.kv_heads + kvh) << p.page_shift;
#pragma unroll
      for (int b = 0; b < TMA_BLOCKS; ++b) {
        const uint32_t offset = (uint32_t)(b * (BKV * 128) + (j << p.page_shift) * 128);
        tma_load_2d(k_dst + offset, &map_k, bar, b * 64, row);
        tma_load_2d(v_dst + offset, &map_v, bar, b * 64, row);
      }
    }
  };
  if (warp == WARPS) {
    // The loading warp runs ahead of the others by up to a ring of tiles; nobody waits for anybody else
    // block-wide.  A stage is refilled once all computing warps have released it.
    if (elect_one()) {
      // tiles that end before this step's own position hold nothing this step writes
      const int settled = pos >= k_first ? (pos - k_first) / BKV : 0;
      int tile = 0;
      for (; tile < num_tiles && tile < p.early_tiles && tile < settled; ++tile) issue(tile);
      pdl_wait();
      for (; tile < num_tiles; ++tile) {
        if (tile >= STAGES)
          mbar_wait_bounded(empty_bar(tile % STAGES), (uint32_t)(tile / STAGES - 1) & 1u, p.status);
        issue(tile);
      }
    }
  }
  pdl_wait();

  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int kc = 0; kc < HD / 16; ++kc) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = g8 + 8 * i;
      const bool valid = r < p.group;
      const __nv_bfloat16* src = p.q + (size_t)token * p.q_stride + (size_t)(kvh * p.group + (valid ? r : 0)) * HD + kc * 16 + 2 * t4;
      qf[kc][i] = valid ? *reinterpret_cast<const uint32_t*>(src) : 0u;
      qf[kc][i + 2] = valid ? *reinterpret_cast<const uint32_t*>(src + 8) : 0u;
    }
  }
  float o_acc[HD / 8][4];
#pragma unroll
  for (int d = 0; d < HD / 8; ++d)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_acc[d][e] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  bool bad_page = false;

  const int group = warp >> 2, w4 = warp & 3;            // this warp's group and its quarter of a tile's keys
  for (int it = group; it < (warp < WARPS ? num_tiles : 0); it += GROUPS) {
    const int stage = it % STAGES;
    const int k0 = k_first + it * BKV + w4 * 16;
    // every warp sees every copy land, also of tiles it has no visible position in: the parity of a wait
    // only tells phases apart while nobody is a whole phase behind
    mbar_wait_bounded(full_bar(stage), (uint32_t)(it / STAGES) & 1u, p.status);
    if (k0 >= hi || k0 + 16 <= lo) {
      if (lane == 0) mbar_arrive(empty_bar(stage));
      continue;
    }
    const uint32_t tK = base + stage * TMA_STAGE_BYTES, tV = tK + TMA_TILE_BYTES;
    if (local_table[(max(k0, lo) >> p.page_shift) - first_page] < 0) bad_page = true;   // a visible position without a page

    float s_acc[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s_acc[n][e] = 0.0f;
#pragma unroll
    for (int kc = 0; kc < HD / 16; ++kc) {
      const int mi = lane >> 3;
      const int n = w4 * 16 + (mi >> 1) * 8 + (lane & 7);
      uint32_t r0, r1, r2, r3;
      ldmatrix_x4(tK + swizzled(n, kc * 16 + (mi & 1) * 8), r0, r1, r2, r3);
      mma_bf16(s_acc[0], qf[kc], r0, r1);
      mma_bf16(s_acc[1], qf[kc], r2, r3);
    }
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const bool row_valid = g8 + 8 * i < p.group;
      float mx = -INFINITY;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kpos = k0 + n * 8 + 2 * t4 + e;
          const bool visible = row_valid && kpos >= lo && kpos < hi;
          const float sv = visible ? s_acc[n][2 * i + e] * p.scale_log2 : -INFINITY;
          s_acc[n][2 * i + e] = sv;
          mx = fmaxf(mx, sv);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[i], mx);
      const float m_use = m_new == -INFINITY ? 0.0f : m_new;
      corr[i] = exp2f(m_run[i] - m_use);
      float sum = 0.0f;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float pv = exp2f(s_acc[n][2 * i + e] - m_use);
          s_acc[n][2 * i + e] = pv;
          sum += pv;
        }
      }
      l_run[i] = l_run[i] * corr[i] + sum;
      m_run[i] = m_new;
    }
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {   // the maximum moved: rescale
#pragma unroll
      for (int d = 0; d < HD / 8; ++d) {
        o_acc[d][0] *= corr[0]; o_acc[d][1] *= corr[0];
        o_acc[d][2] *= corr[1]; o_acc[d][3] *= corr[1];
      }
    }
    uint32_t pf[4];
    pf[0] = pack_bf16(s_acc[0][0], s_acc[0][1]);
    pf[1] = pack_bf16(s_acc[0][2], s_acc[0][3]);
    pf[2] = pack_bf16(s_acc[1][0], s_acc[1][1]);
    pf[3] = pack_bf16(s_acc[1][2], s_acc[1][3]);
#pragma unroll
    for (int dt = 0; dt < HD / 8; dt += 2) {
      const int mi = lane >> 3;
      const int key = w4 * 16 + (mi & 1) * 8 + (lane & 7);
      uint32_t r0, r1, r2, r3;
      ldmatrix_x4_trans(tV + swizzled(key, (dt + (mi >> 1)) * 8), r0, r1, r2, r3);
      mma_bf16(o_acc[dt], pf, r0, r1);
      mma_bf16(o_acc[dt + 1], pf, r2, r3);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(stage));        // this warp has read all it needs of the stage
  }
  __syncthreads();                                       // all tiles consumed, no copy in flight: reuse the stages
  if (bad_page && p.status) atomicOr(p.status, TGE_STATUS_BAD_PAGE);

  float* merge_o = reinterpret_cast<float*>(generic);                   // [warps][16][HD]
  float* merge_ml = merge_o + WARPS * 16 * HD;                      // [warps][16][2]
#pragma unroll
  for (int i = 0; i < (warp < WARPS ? 2 : 0); ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    const int r = g8 + 8 * i;
    float* dst = merge_o + ((size_t)warp * 16 + r) * HD;
#pragma unroll
    for (int d = 0; d < HD / 8; ++d)
      *reinterpret_cast<float2*>(dst + d * 8 + 2 * t4) = make_float2(o_acc[d][2 * i], o_acc[d][2 * i + 1]);
    if (t4 == 0) {
      merge_ml[(warp * 16 + r) * 2] = m_run[i];
      merge_ml[(warp * 16 + r) * 2 + 1] = l_run[i];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < p.group * HD; idx += THREADS) {
    const int r = idx / HD, d = idx - r * HD;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) m = fmaxf(m, merge_ml[(w * 16 + r) * 2]);
    const float m_use = m == -INFINITY ? 0.0f : m;
    float l = 0.0f, acc = 0.0f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float scale = exp2f(merge_ml[(w * 16 + r) * 2] - m_use);
      l += scale * merge_ml[(w * 16 + r) * 2 + 1];
      acc += scale * merge_o[((size_t)w * 16 + r) * HD + d];
    }
    const int head = kvh * p.group + r;
    if (p.num_splits == 1) {
      p.out[(size_t)token * p.out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
    } else {
      const size_t slot = ((size_t)split * p.total_tokens + token) * p.heads + head;
      p.partial_o[slot * HD + d] = acc;
      if (d == 0) {
        p.partial_ml[slot * 2] = m;
        p.partial_ml[slot * 2 + 1] = l;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Prompt portions for head sizes that are multiples of 64: eight warps own 128 rows ((query, head-of-group)
// pairs of one kv head), every warp takes 16 rows against the whole 64-position tile, tiles arrive by TMA as
// in the decode kernel.  Tiles that lie wholly before every row's position need no mask; the accumulator is
// rescaled only when a running maximum moved.
// ---------------------------------------------------------------------------
constexpr int PRE_WARPS = 8;                  // warps that compute; one more warp issues the TMA loads
constexpr int PRE_STAGES = 4;
constexpr int PRE_THREADS = (PRE_WARPS + 1) * 32;

__global__ void __launch_bounds__(PRE_THREADS) attention_prefill_tma_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ int tile_info[2];
  pdl_trigger();
  pdl_wait();
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* generic = smem_dyn + (base - raw);
  const uint32_t bars = base + PRE_STAGES * TMA_STAGE_BYTES;            // full[stages], then empty[stages]
  int* local_table = reinterpret_cast<int*>(generic + PRE_STAGES * TMA_STAGE_BYTES + 128);

  const int tid = threadIdx.x, lane = tid & 31, warp = uniform_warp_index();
  const int g8 = lane >> 2, t4 = lane & 3;
  const int kvh = blockIdx.y, split = blockIdx.z;
  if (tid == 0) {
    // Blocks take tiles from the back: under a causal mask the later tiles of a portion are the longer ones,
    // and starting them first keeps the tail of the launch short.
    int total = 0;
    for (int s = 0; s < p.num_seqs; ++s) total += (p.q_start[s + 1] - p.q_start[s] + p.bq - 1) / p.bq;
    int remaining = total - 1 - (int)blockIdx.x, seq = -1, tile = 0;
    for (int s = 0; s < p.num_seqs && remaining >= 0; ++s) {
      const int q_len = p.q_start[s + 1] - p.q_start[s];
      const int tiles = (q_len + p.bq - 1) / p.bq;
      if (remaining < tiles) { seq = s; tile = remaining; break; }
      remaining -= tiles;
    }
    tile_info[0] = seq;
    tile_info[1] = tile;
  }
  __syncthreads();
  const int seq = tile_info[0];
  if (seq < 0) return;
  const int q_first = tile_info[1] * p.bq;
  const int q_begin = p.q_start[seq];
  const int q_len = p.q_start[seq + 1] - q_begin;
  const int q_count = min(p.bq, q_len - q_first);
  const int pos0 = p.start_pos[seq] + q_first;

  int lo = p.window > 0 ? max(pos0 - p.window + 1, 0) : 0;
  int hi = pos0 + q_count;
  if (p.num_splits > 1) {
    lo = max(lo, split * p.split_tokens);
    hi = min(hi, (split + 1) * p.split_tokens);
  }
  if (lo >= hi) return;

  const int k_first = lo / BKV * BKV;
  const int num_tiles = (hi - k_first + BKV - 1) / BKV;
  const int first_page = k_first >> p.page_shift;
  const int last_page = (k_first + num_tiles * BKV - 1) >> p.page_shift;
  for (int i = first_page + tid; i <= last_page; i += PRE_THREADS) {
    int page = i < p.max_pages ? p.block_table[(size_t)seq * p.max_pages + i] : -1;
    if (page >= p.num_pages) page = -2;
    local_table[i - first_page] = page;
  }
  {
    uint4* fill = reinterpret_cast<uint4*>(generic);
    for (int i = tid; i < PRE_STAGES * TMA_STAGE_BYTES / 16; i += PRE_THREADS) fill[i] = make_uint4(0, 0, 0, 0);
  }
  if (tid == 0) {
    for (int s = 0; s < PRE_STAGES; ++s) {
      mbar_init(bars + 8 * s, 1);
      mbar_init(bars + 8 * (PRE_STAGES + s), PRE_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  __syncthreads();

  const int pages_per_tile = BKV >> p.page_shift;
  auto issue = [&](int tile) {
    const int stage = tile % PRE_STAGES;
    const uint32_t k_dst = base + stage * TMA_STAGE_BYTES, v_dst = k_dst + TMA_TILE_BYTES;
    const uint32_t bar = bars + 8 * stage;
    int boxes = 0;
    for (int j = 0; j < pages_per_tile; ++j) {
      const int page = local_table[((k_first + tile * BKV) >> p.page_shift) + j - first_page];
      if (page >= 0 && (k_first + tile * BKV + (j << p.page_shift)) < hi) ++boxes;
    }
    mbar_expect_tx(bar, (uint32_t)boxes * 2u * TMA_BLOCKS * (uint32_t)(p.page_size * 128));
    for (int j = 0; j < pages_per_tile; ++j) {
      const int page = local_table[((k_first + tile * BKV) >> p.page_shift) + j - first_page];
      if (page < 0 || (k_first + tile * BKV + (j << p.page_shift)) >= hi) continue;
      const int row = (page * p.kv_heads + kvh) << p.page_shift;
#pragma unroll
      for (int b = 0; b < TMA_BLOCKS; ++b) {
        const uint32_t offset = (uint32_t)(b * (BKV * 128) + (j << p.page_shift) * 128);
        tma_load_2d(k_dst + offset, &map_k, bar, b * 64, row);
        tma_load_2d(v_dst + offset, &map_v, bar, b * 64, row);
      }
    }
  };
  if (warp == PRE_WARPS) {
    // the loading warp: a stage is refilled as soon as all eight computing warps have released it
    if (elect_one()) {
      for (int tile = 0; tile < num_tiles; ++tile) {
        if (tile >= PRE_STAGES)
          mbar_wait_bounded(bars + 8 * (PRE_STAGES + tile % PRE_STAGES), (uint32_t)(tile / PRE_STAGES - 1) & 1u, p.status);
        issue(tile);
      }
    }
    return;
  }

  int row_token[2], row_pos[2], row_head[2];
  bool row_valid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = warp * 16 + g8 + 8 * i;
    const int qi = r / p.group, gg = r - qi * p.group;
    row_valid[i] = qi < q_count;
    row_token[i] = q_begin + q_first + (row_valid[i] ? qi : 0);
    row_pos[i] = pos0 + qi;
    row_head[i] = kvh * p.group + gg;
  }
  // the warp's rows span these positions (for skipping masks and whole tiles)
  const int warp_q_lo = (warp * 16) / p.group, warp_q_hi = min((warp * 16 + 15) / p.group, q_count - 1);
  const bool warp_active = warp_q_lo < q_count;
  const int warp_pos_lo = pos0 + warp_q_lo, warp_pos_hi = pos0 + warp_q_hi;

  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int kc = 0; kc < HD / 16; ++kc) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const __nv_bfloat16* src = p.q + (size_t)row_token[i] * p.q_stride + (size_t)row_head[i] * HD + kc * 16 + 2 * t4;
      qf[kc][i] = row_valid[i] ? *reinterpret_cast<const uint32_t*>(src) : 0u;
      qf[kc][i + 2] = row_valid[i] ? *reinterpret_cast<const uint32_t*>(src + 8) : 0u;
    }
  }
  float o_acc[HD / 8][4];
#pragma unroll
  for (int d = 0; d < HD / 8; ++d)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_acc[d][e] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  bool bad_page = false;

  for (int it = 0; it < num_tiles; ++it) {
    const int stage = it % PRE_STAGES;
    mbar_wait_bounded(bars + 8 * stage, (uint32_t)(it / PRE_STAGES) & 1u, p.status);
    const uint32_t tK = base + stage * TMA_STAGE_BYTES, tV = tK + TMA_TILE_BYTES;
    const int k0 = k_first + it * BKV;
    // nothing in this tile is visible to this warp's rows (before their windows or after their positions):
    // release the stage at once
    const bool skip = !warp_active || k0 > warp_pos_hi || (p.window > 0 && k0 + BKV <= warp_pos_lo - p.window + 1);
    if (skip) {
      if (lane == 0) mbar_arrive(bars + 8 * (PRE_STAGES + stage));
      continue;
    }
    if (local_table[(max(k0, lo) >> p.page_shift) - first_page] < 0) bad_page = true;

    float s_acc[BKV / 8][4];
#pragma unroll
    for (int n = 0; n < BKV / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s_acc[n][e] = 0.0f;
#pragma unroll
    for (int kc = 0; kc < HD / 16; ++kc) {
#pragma unroll
      for (int nt = 0; nt < BKV / 8; nt += 2) {
        const int mi = lane >> 3;
        const int n = (nt + (mi >> 1)) * 8 + (lane & 7);
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4(tK + swizzled(n, kc * 16 + (mi & 1) * 8), r0, r1, r2, r3);
        mma_bf16(s_acc[nt], qf[kc], r0, r1);
        mma_bf16(s_acc[nt + 1], qf[kc], r2, r3);
      }
    }
    // a tile wholly inside [lo, hi), before every row's position and inside every row's window needs no mask
    const bool clean = k0 >= lo && k0 + BKV <= hi && k0 + BKV - 1 <= warp_pos_lo &&
                       (p.window == 0 || k0 >= warp_pos_hi - p.window + 1) && warp_q_hi < q_count &&
                       (warp * 16 + 15) / p.group < q_count;
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int first_key = p.window > 0 ? row_pos[i] - p.window + 1 : 0;
      float mx = -INFINITY;
#pragma unroll
      for (int n = 0; n < BKV / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float sv = s_acc[n][2 * i + e] * p.scale_log2;
          if (!clean) {
            const int kpos = k0 + n * 8 + 2 * t4 + e;
            const bool visible = row_valid[i] && kpos <= row_pos[i] && kpos >= first_key && kpos >= lo && kpos < hi;
            sv = visible ? sv : -INFINITY;
          }
          s_acc[n][2 * i + e] = sv;
          mx = fmaxf(mx, sv);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[i], mx);
      const float m_use = m_new == -INFINITY ? 0.0f : m_new;
      corr[i] = exp2f(m_run[i] - m_use);
      float sum = 0.0f;
#pragma unroll
      for (int n = 0; n < BKV / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float pv = exp2f(s_acc[n][2 * i + e] - m_use);
          s_acc[n][2 * i + e] = pv;
          sum += pv;
        }
      }
      l_run[i] = l_run[i] * corr[i] + sum;
      m_run[i] = m_new;
    }
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
      for (int d = 0; d < HD / 8; ++d) {
        o_acc[d][0] *= corr[0]; o_acc[d][1] *= corr[0];
        o_acc[d][2] *= corr[1]; o_acc[d][3] *= corr[1];
      }
    }
#pragma unroll
    for (int kk = 0; kk < BKV / 16; ++kk) {
      uint32_t pf[4];
      pf[0] = pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]);
      pf[1] = pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]);
      pf[2] = pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]);
      pf[3] = pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]);
#pragma unroll
      for (int dt = 0; dt < HD / 8; dt += 2) {
        const int mi = lane >> 3;
        const int key = kk * 16 + (mi & 1) * 8 + (lane & 7);
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4_trans(tV + swizzled(key, (dt + (mi >> 1)) * 8), r0, r1, r2, r3);
        mma_bf16(o_acc[dt], pf, r0, r1);
        mma_bf16(o_acc[dt + 1], pf, r2, r3);
      }
    }
    __syncwarp();                                        // the whole warp has read the stage
    if (lane == 0) mbar_arrive(bars + 8 * (PRE_STAGES + stage));
  }
  if (bad_page && p.status) atomicOr(p.status, TGE_STATUS_BAD_PAGE);

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!row_valid[i]) continue;
    if (p.num_splits == 1) {
      const float inv = l_run[i] > 0.0f ? 1.0f / l_run[i] : 0.0f;
      __nv_bfloat16* dst = p.out + (size_t)row_token[i] * p.out_stride + (size_t)row_head[i] * HD;
#pragma unroll
      for (int d = 0; d < HD / 8; ++d)
        *reinterpret_cast<uint32_t*>(dst + d * 8 + 2 * t4) = pack_bf16(o_acc[d][2 * i] * inv, o_acc[d][2 * i + 1] * inv);
    } else {
      const size_t slot = ((size_t)split * p.total_tokens + row_token[i]) * p.heads + row_head[i];
      float* dst = p.partial_o + slot * HD;
#pragma unroll
      for (int d = 0; d < HD / 8; ++d)
        *reinterpret_cast<float2*>(dst + d * 8 + 2 * t4) = make_float2(o_acc[d][2 * i], o_acc[d][2 * i + 1]);
      if (t4 == 0) {
        p.partial_ml[slot * 2] = m_run[i];
        p.partial_ml[slot * 2 + 1] = l_run[i];
      }
    }
  }
}

#include "attention_tc.cuh"
#include "attention_tc2.cuh"

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The tensor map of a page pool, made once per (address, geometry) and kept.
const CUtensorMap* pool_map(const void* pages, int num_pages, int kv_heads, int page_size) {
  static EncodeTiledFn encode = nullptr;
  static bool tried = false;
  static std::map<std::tuple<const void*, int, int, int>, CUtensorMap> maps;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      encode = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  if (!encode) {
    tge_set_error("attention_decode: the driver does not export cuTensorMapEncodeTiled");
    return nullptr;
  }
  const auto key = std::make_tuple(pages, num_pages, kv_heads, page_size);
  auto found = maps.find(key);
  if (found != maps.end()) return &found->second;
  CUtensorMap map;
  cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)num_pages * kv_heads * page_size};
  cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)page_size};
  cuuint32_t elem[2] = {1, 1};
  CUresult rc = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, elem,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    tge_set_error("attention_decode: cuTensorMapEncodeTiled failed with code %d", (int)rc);
    return nullptr;
  }
  return &maps.emplace(key, map).first->second;
}
#endif  // TGE_HEAD_DIM % 64 == 0

// Merges the split states of one (token, head): out = sum_s 2^(m_s - M) acc_s / sum_s 2^(m_s - M) l_s,
// over the splits that hold keys visible to the row, in split order.
template <int HELD>                                                  // splits whose state is held in registers
__global__ void attention_merge_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                                       const int* __restrict__ positions, __nv_bfloat16* __restrict__ out,
                                       int out_stride, int total_tokens, int heads, int window, int split_tokens,
                                       int num_splits, int first_token) {
  pdl_trigger();
  const int t = blockIdx.x + first_token, h = blockIdx.y;
  const int pos = positions[t];                                     // given to the step: not the previous kernel's work
  pdl_wait();
  const size_t stride = (size_t)total_tokens * heads;               // slots per split
  const size_t slot0 = (size_t)t * heads + h;
  if (num_splits <= HELD) {
    // Every load is asked for before the first result is needed, the row's position among them: one round
    // trip instead of four.  Splits without a key visible to the row are read too (the scratch holds all
    // splits; what lies there is old) and dropped by selection, never by a weight of zero.
    float2 ml[HELD];
#pragma unroll
    for (int i = 0; i < HELD; ++i)
      ml[i] = i < num_splits ? *reinterpret_cast<const float2*>(partial_ml + ((size_t)i * stride + slot0) * 2)
                             : make_float2(-INFINITY, 0.0f);
    const int first_key = window > 0 ? max(pos - window + 1, 0) : 0;
    const int s_lo = first_key / split_tokens;
    const int s_hi = min(pos / split_tokens, num_splits - 1);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
      float o[HELD];
#pragma unroll
      for (int i = 0; i < HELD; ++i) o[i] = i < num_splits ? partial_o[((size_t)i * stride + slot0) * HD + d] : 0.0f;
#pragma unroll
      for (int i = 0; i < HELD; ++i) {
        const bool live = i >= s_lo && i <= s_hi;
        ml[i] = live ? ml[i] : make_float2(-INFINITY, 0.0f);
        o[i] = live ? o[i] : 0.0f;
      }
      float m = -INFINITY;
#pragma unroll
      for (int i = 0; i < HELD; ++i) m = fmaxf(m, ml[i].x);
      const float m_use = m == -INFINITY ? 0.0f : m;
      float l = 0.0f, acc = 0.0f;
#pragma unroll
      for (int i = 0; i < HELD; ++i) {          // in split order; a split beyond s_hi has m = -inf: weight 0
        const float scale = exp2f(ml[i].x - m_use);
        l += scale * ml[i].y;
        acc += scale * o[i];
      }
      out[(size_t)t * out_stride + (size_t)h * HD + d] = __float2bfloat16_rn(acc * (l > 0.0f ? 1.0f / l : 0.0f));
    }
    return;
  }
  const int first_key = window > 0 ? max(pos - window + 1, 0) : 0;
  const int s_lo = first_key / split_tokens;
  const int s_hi = min(pos / split_tokens, num_splits - 1);
  float m = -INFINITY;
  for (int s = s_lo; s <= s_hi; ++s) m = fmaxf(m, partial_ml[((size_t)s * stride + slot0) * 2]);
  const float m_use = m == -INFINITY ? 0.0f : m;
  float l = 0.0f;
  for (int s = s_lo; s <= s_hi; ++s) {
    const size_t slot = (size_t)s * stride + slot0;
    l += exp2f(partial_ml[slot * 2] - m_use) * partial_ml[slot * 2 + 1];
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float acc = 0.0f;
    for (int s = s_lo; s <= s_hi; ++s) {
      const size_t slot = (size_t)s * stride + slot0;
      acc += exp2f(partial_ml[slot * 2] - m_use) * partial_o[slot * HD + d];
    }
    out[(size_t)t * out_stride + (size_t)h * HD + d] = __float2bfloat16_rn(acc * inv);
  }
}

// Sixteen states in registers serve most steps; a single long request cut into up to 48 splits takes the wider
// instance, and beyond that the kernel walks the splits in a loop.
void launch_merge(dim3 grid, cudaStream_t stream, const float* partial_o, const float* partial_ml, const int* positions,
                  __nv_bfloat16* out, int out_stride, int total_tokens, int heads, int window, int split_tokens,
                  int num_splits, int first_token) {
  const int threads = HD >= 128 ? 128 : (HD >= 64 ? 64 : 32);
  if (num_splits <= 16)
    tge_launch(attention_merge_kernel<16>, grid, threads, 0, stream, partial_o, partial_ml, positions, out, out_stride,
               total_tokens, heads, window, split_tokens, num_splits, first_token);
  else
    tge_launch(attention_merge_kernel<48>, grid, threads, 0, stream, partial_o, partial_ml, positions, out, out_stride,
               total_tokens, heads, window, split_tokens, num_splits, first_token);
}

template <int NWARPS>
int launch(const AttnParams& p, int tiles, cudaStream_t stream) {
  const size_t smem = (size_t)4 * BKV * ROW_ELEMS * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attention_mma_kernel<NWARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) {
      tge_set_error("attention_mma: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
      return -2;
    }
    configured = true;
  }
  dim3 grid(tiles, p.kv_heads, p.num_splits);
  tge_launch(attention_mma_kernel<NWARPS>, grid, NWARPS * 32, smem, stream, p);
  return tge_check_launch("attention_mma");
}

}  // namespace

TGE_API int tge_attention_mma_head_dim() { return HD; }

// Rows of scratch a call needs: float32 [splits, tokens, heads, HD] for acc and [splits, tokens, heads, 2] for (m, l).
TGE_API long long tge_attention_mma_scratch_floats(int tokens, int heads, int num_splits) {
  return num_splits > 1 ? (long long)num_splits * tokens * heads * (HD + 2) : 0;
}

// q: [tokens, heads*HD] with row stride q_stride (elements); pages: [num_pages, kv_heads, page_size, HD].
// q_start [num_seqs+1], start_pos [num_seqs], positions [tokens] are int32 on the device.
// max_q_len / max_ctx_len are host-side bounds used only for launch geometry.
// split_tokens: 0 = one split; else a multiple of 64 (keys per split).  scratch: see above.
// `first_token`: the sequences given here start at this token of the step (earlier tokens belong to sequences
// that another launch serves); q, out, positions and the scratch layout stay those of the whole step.
static int attention_dispatch(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                              const int* block_table, int max_pages, int num_pages, int page_size,
                              const int* q_start, const int* start_pos, const int* positions, int num_seqs,
                              int tokens, int max_q_len, int max_ctx_len, void* out, int out_stride, int heads,
                              int kv_heads, float scale, int window, int split_tokens, float* scratch, int* status,
                              int first_token, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && num_seqs >= 0, "attention_mma: negative sizes");
  TGE_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
              "attention_mma: heads %d must be a positive multiple of kv heads %d", heads, kv_heads);
  const int group = heads / kv_heads;
  TGE_REQUIRE(group <= 64, "attention_mma: %d query heads per kv head exceed the 64 rows of a tile", group);
  TGE_REQUIRE(page_size > 0 && BKV % page_size == 0, "attention_mma: page size %d must divide %d", page_size, BKV);
  TGE_REQUIRE(q_stride % 2 == 0 && out_stride % 2 == 0, "attention_mma: odd row strides");
  TGE_REQUIRE(((uintptr_t)q % 4 == 0) && ((uintptr_t)out % 4 == 0) && ((uintptr_t)k_pages % 16 == 0) &&
                  ((uintptr_t)v_pages % 16 == 0), "attention_mma: misaligned tensors");
  TGE_REQUIRE(window >= 0 && split_tokens >= 0 && split_tokens % BKV == 0,
              "attention_mma: keys per split %d must be a multiple of %d", split_tokens, BKV);
  if (tokens == 0 || num_seqs == 0) return 0;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
  p.block_table = block_table; p.q_start = q_start; p.start_pos = start_pos;
  p.out = (__nv_bfloat16*)out; p.status = status;
  p.q_stride = q_stride; p.out_stride = out_stride;
  p.max_pages = max_pages; p.num_pages = num_pages; p.page_size = page_size;
  p.page_shift = 0;
  while ((1 << p.page_shift) < page_size) ++p.page_shift;
  p.num_seqs = num_seqs; p.total_tokens = tokens;
  static const bool early = getenv("TGE_NO_EARLY_KV") == nullptr || getenv("TGE_NO_EARLY_KV")[0] == '\0';
  p.early_tiles = early ? DEC_STAGES : 0;
  p.heads = heads; p.kv_heads = kv_heads; p.group = group;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  int num_splits = 1;
  if (split_tokens > 0 && max_ctx_len > split_tokens) num_splits = (max_ctx_len + split_tokens - 1) / split_tokens;
  p.split_tokens = split_tokens > 0 ? split_tokens : max_ctx_len;
  p.num_splits = num_splits;
  TGE_REQUIRE(num_splits == 1 || scratch != nullptr, "attention_mma: %d splits need scratch memory", num_splits);
  p.partial_o = scratch;
  p.partial_ml = scratch ? scratch + (size_t)num_splits * tokens * heads * HD : nullptr;

#if TGE_HEAD_DIM % 64 == 0
  if (max_q_len <= 1 && tokens == num_seqs && group <= 16 && page_size >= 8) {
    const CUtensorMap* map_k = pool_map(k_pages, num_pages, kv_heads, page_size);
    const CUtensorMap* map_v = pool_map(v_pages, num_pages, kv_heads, page_size);
    if (!map_k || !map_v) return -3;
    const int range = (num_splits > 1 ? p.split_tokens : max_ctx_len) + 2 * BKV;
    // No more blocks than SMs, each with many keys: a block has its SM to itself and runs two groups of warps on
    // alternate tiles (batch 32 at context 2,048, not cut: 3.82 -> 3.66 ms per step).  With few tiles per block the
    // second group only adds to what has to be set up and merged (batch 4, nine splits of 256 keys: 2.95 -> 3.10).
    static const bool two_ok = getenv("TGE_DECODE_ONE_GROUP") == nullptr || getenv("TGE_DECODE_ONE_GROUP")[0] == '\0';
    auto smem_of = [&](int ring) {
      return 1024 + (size_t)ring * TMA_STAGE_BYTES + 64 + ((size_t)(range >> p.page_shift) + 2) * sizeof(int);
    };
    const bool two_groups = two_ok && (long long)num_seqs * kv_heads * num_splits <= tge_sm_count() &&
                            (num_splits > 1 ? p.split_tokens : max_ctx_len) >= 1536 && smem_of(4) <= 227 * 1024;
    const int stages = two_groups ? 4 : DEC_STAGES;
    const size_t smem = smem_of(stages);
    TGE_REQUIRE(smem <= 227 * 1024, "attention_decode: %d keys per block need %zu bytes of shared memory; use smaller splits", range, smem);
    static size_t configured[2] = {0, 0};
    if (smem > configured[two_groups]) {
      cudaError_t err = two_groups
          ? cudaFuncSetAttribute(attention_decode_tma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
          : cudaFuncSetAttribute(attention_decode_tma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) {
        tge_set_error("attention_decode: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
        return -2;
      }
      configured[two_groups] = smem;
    }
    p.bq = 1;
    p.early_tiles = p.early_tiles ? stages : 0;
    dim3 grid(num_seqs, kv_heads, num_splits);
    if (two_groups) tge_launch(attention_decode_tma_kernel<2>, grid, 9 * 32, smem, stream, *map_k, *map_v, p);
    else tge_launch(attention_decode_tma_kernel<1>, grid, DEC_TMA_THREADS, smem, stream, *map_k, *map_v, p);
    int rc = tge_check_launch("attention_decode_tma");
    if (rc != 0) return rc;
    if (num_splits > 1) {
      dim3 mgrid(tokens - first_token, heads);
      launch_merge(mgrid, stream, p.partial_o, p.partial_ml, positions, p.out, out_stride, tokens, heads, window, p.split_tokens, num_splits, first_token);
      return tge_launched("attention_merge", 2);
    }
    return 1;
  }
#endif
  if (max_q_len <= 1 && tokens == num_seqs && group <= 16) {
    // stages, then one page id per page of the longest key range a block can own
    const int range = num_splits > 1 ? p.split_tokens : max_ctx_len;
    const size_t smem = (size_t)DEC_STAGES * STAGE_ELEMS * sizeof(__nv_bfloat16) + ((size_t)(range >> p.page_shift) + 2) * sizeof(int);
    TGE_REQUIRE(smem <= 227 * 1024, "attention_decode: %d keys per block need %zu bytes of shared memory; use smaller splits", range, smem);
    static size_t configured = 0;
    if (smem > configured) {
      cudaError_t err = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) {
        tge_set_error("attention_decode: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
        return -2;
      }
      configured = smem;
    }
    p.bq = 1;
    dim3 grid(num_seqs, kv_heads, num_splits);
    tge_launch(attention_decode_kernel, grid, DEC_WARPS * 32, smem, stream, p);
    int rc = tge_check_launch("attention_decode");
    if (rc != 0) return rc;
    if (num_splits > 1) {
      dim3 mgrid(tokens - first_token, heads);
      launch_merge(mgrid, stream, p.partial_o, p.partial_ml, positions, p.out, out_stride, tokens, heads, window, p.split_tokens, num_splits, first_token);
      return tge_launched("attention_merge", 2);
    }
    return 1;
  }
#if TGE_HEAD_DIM % 64 == 0
  if (max_q_len > 1 && group <= 64 && page_size >= 8) {
    const CUtensorMap* map_k = pool_map(k_pages, num_pages, kv_heads, page_size);
    const CUtensorMap* map_v = pool_map(v_pages, num_pages, kv_heads, page_size);
    if (!map_k || !map_v) return -3;
    p.bq = (PRE_WARPS * 16) / group;
    const int range = (num_splits > 1 ? p.split_tokens : max_ctx_len) + 2 * BKV;
    static const bool use_tc = getenv("TGE_NO_TC_ATTENTION") == nullptr || getenv("TGE_NO_TC_ATTENTION")[0] == '\0';
    if (use_tc && tc::smem_bytes(range >> p.page_shift) <= 227 * 1024 && q_stride % 8 == 0 && (uintptr_t)q % 16 == 0 &&
        out_stride % 8 == 0 && (uintptr_t)out % 16 == 0) {
      // the tcgen05 kernels: 128 rows per query tile as well
      static const bool one_tile = getenv("TGE_ATTENTION_ONE_TILE") != nullptr && getenv("TGE_ATTENTION_ONE_TILE")[0] != '\0';
      if (tc2::FITS && !one_tile && tc2::smem_bytes(range >> p.page_shift) <= 227 * 1024) {
        // two query tiles per block, one block per SM
        const size_t smem2 = tc2::smem_bytes(range >> p.page_shift);
        static size_t configured_tc2 = 0;
        if (smem2 > configured_tc2) {
          cudaError_t err = cudaFuncSetAttribute(tc2::attention_prefill_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
          if (err != cudaSuccess) {
            tge_set_error("attention_prefill_tc2: cannot reserve %zu bytes of shared memory: %s", smem2, cudaGetErrorString(err));
            return -2;
          }
          configured_tc2 = smem2;
        }
        const int pairs = ((tokens - first_token + p.bq - 1) / p.bq + 1) / 2 + num_seqs;
        dim3 grid2(pairs * kv_heads, 1, num_splits);
        tge_launch(tc2::attention_prefill_tc2_kernel, grid2, tc2::THREADS, smem2, stream, *map_k, *map_v, p);
        int rc2 = tge_check_launch("attention_prefill_tc2");
        if (rc2 != 0) return rc2;
        if (num_splits > 1) {
          dim3 mgrid(tokens - first_token, heads);
          launch_merge(mgrid, stream, p.partial_o, p.partial_ml, positions, p.out, out_stride, tokens, heads, window, p.split_tokens, num_splits, first_token);
          return tge_launched("attention_merge", 2);
        }
        return 1;
      }
      const size_t smem = tc::smem_bytes(range >> p.page_shift);
      static size_t configured_tc = 0;
      if (smem > configured_tc) {
        cudaError_t err = cudaFuncSetAttribute(tc::attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) {
          tge_set_error("attention_prefill_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
          return -2;
        }
        configured_tc = smem;
      }
      const int tiles = (tokens - first_token + p.bq - 1) / p.bq + num_seqs;
      dim3 grid(tiles * kv_heads, 1, num_splits);
      tge_launch(tc::attention_prefill_tc_kernel, grid, tc::THREADS, smem, stream, *map_k, *map_v, p);
      int rc = tge_check_launch("attention_prefill_tc");
      if (rc != 0) return rc;
      if (num_splits > 1) {
        dim3 mgrid(tokens - first_token, heads);
        launch_merge(mgrid, stream, p.partial_o, p.partial_ml, positions, p.out, out_stride, tokens, heads, window, p.split_tokens, num_splits, first_token);
        return tge_launched("attention_merge", 2);
      }
      return 1;
    }
    const size_t smem = 1024 + (size_t)PRE_STAGES * TMA_STAGE_BYTES + 128 + ((size_t)(range >> p.page_shift) + 2) * sizeof(int);
    if (smem <= 227 * 1024) {
      static size_t configured = 0;
      if (smem > configured) {
        cudaError_t err = cudaFuncSetAttribute(attention_prefill_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) {
          tge_set_error("attention_prefill: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
          return -2;
        }
        configured = smem;
      }
      const int tiles = (tokens - first_token + p.bq - 1) / p.bq + num_seqs;
      dim3 grid(tiles, kv_heads, num_splits);
      tge_launch(attention_prefill_tma_kernel, grid, PRE_THREADS, smem, stream, *map_k, *map_v, p);
      int rc = tge_check_launch("attention_prefill_tma");
      if (rc != 0) return rc;
      if (num_splits > 1) {
        dim3 mgrid(tokens - first_token, heads);
        launch_merge(mgrid, stream, p.partial_o, p.partial_ml, positions, p.out, out_stride, tokens, heads, window, p.split_tokens, num_splits, first_token);
        return tge_launched("attention_merge", 2);
      }
      return 1;
    }
  }
#endif
  // rows per block: one warp (16 rows) per block when every portion is a single token and the group fits
  int nwarps = 4;
  if (max_q_len <= 1) nwarps = group <= 16 ? 1 : (group <= 32 ? 2 : 4);
  const int rows = nwarps * 16;
  p.bq = rows / group;
  const int tiles = (tokens - first_token + p.bq - 1) / p.bq + num_seqs;  // upper bound over any cut into portions
  int rc;
  if (nwarps == 1) rc = launch<1>(p, tiles, stream);
  else if (nwarps == 2) rc = launch<2>(p, tiles, stream);
  else rc = launch<4>(p, tiles, stream);
  if (rc != 0) return rc;
  if (num_splits > 1) {
    dim3 grid(tokens - first_token, heads);
    launch_merge(grid, stream, p.partial_o, p.partial_ml, positions, p.out, out_stride, tokens, heads, window, p.split_tokens, num_splits, first_token);
    return tge_launched("attention_merge", 2);
  }
  return 1;
}

// `decode_prefix`: the caller knows that the first so many sequences of a step that also holds longer portions
// bring one token each (0: unknown or none).  They then go to the split-key decode kernel, which reads each
// sequence's keys once for all query heads of a kv head, instead of filling one 128-row query tile of the
// prefill kernel each; the other sequences follow in a second launch.  A row's value does not depend on the
// route beyond rounding.
TGE_API int tge_attention_mma(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                              const int* block_table, int max_pages, int num_pages, int page_size,
                              const int* q_start, const int* start_pos, const int* positions, int num_seqs,
                              int tokens, int max_q_len, int max_ctx_len, void* out, int out_stride, int heads,
                              int kv_heads, float scale, int window, int split_tokens, float* scratch, int* status,
                              int decode_prefix, int prefix_split_tokens, cudaStream_t stream) {
  TGE_REQUIRE(decode_prefix >= 0 && decode_prefix <= num_seqs, "attention_mma: %d leading single tokens of %d sequences",
              decode_prefix, num_seqs);
  TGE_REQUIRE(prefix_split_tokens >= 0 && prefix_split_tokens % BKV == 0,
              "attention_mma: keys per split %d of the leading single tokens must be a multiple of %d", prefix_split_tokens, BKV);
  if (decode_prefix == 0 || max_q_len <= 1 || decode_prefix == num_seqs || kv_heads <= 0 || heads / kv_heads > 16)
    return attention_dispatch(q, q_stride, k_pages, v_pages, block_table, max_pages, num_pages, page_size, q_start, start_pos,
                              positions, num_seqs, tokens, max_q_len, max_ctx_len, out, out_stride, heads, kv_heads, scale,
                              window, split_tokens, scratch, status, 0, stream);
  const int first = attention_dispatch(q, q_stride, k_pages, v_pages, block_table, max_pages, num_pages, page_size, q_start,
                                       start_pos, positions, decode_prefix, decode_prefix, 1, max_ctx_len, out, out_stride,
                                       heads, kv_heads, scale, window, prefix_split_tokens, scratch, status, 0, stream);
  if (first < 0) return first;
  const int rest = attention_dispatch(q, q_stride, k_pages, v_pages, block_table + (size_t)decode_prefix * max_pages, max_pages,
                                      num_pages, page_size, q_start + decode_prefix, start_pos + decode_prefix, positions,
                                      num_seqs - decode_prefix, tokens, max_q_len, max_ctx_len, out, out_stride, heads,
                                      kv_heads, scale, window, split_tokens, scratch, status, decode_prefix, stream);
  return rest < 0 ? rest : first + rest;
}
