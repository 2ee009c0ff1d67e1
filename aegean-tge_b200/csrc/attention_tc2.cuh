// Prompt-portion attention on the 5th-generation tensor cores, two query tiles per block.
// Included by attention_mma.cu after attention_tc.cuh, whose helpers (namespace tc) it uses.
//
// attention_tc.cuh gives each block one tile of 128 rows and fits two blocks on an SM; every block then
// fetches its own K and V from L2, and a block's chain per tile (K lands -> scores -> softmax -> P V ->
// the stage is free -> next K) is barely hidden by its one neighbour.  Here one block owns the SM:
//   * two tiles of 128 rows ((query, head-of-group) pairs of one kv head, consecutive queries) share
//     every K/V tile, so K and V cross L2 -> shared memory once per 256 rows;
//   * all 512 tensor-memory columns: two score buffers per query tile (4 x 64) and one output accumulator
//     per query tile (2 x head size, head size <= 128);
//   * eight softmax warps (four per query tile, one row per thread), one warp issuing the score
//     products, one issuing the P V products (one thread, then still chosen by `lane == 0`, issued a tcgen05.mma about every 85 cycles, and
//     a product of 128 x 64 x 16 keeps the tensor core busy for 32; two issuers gave 58 -> 52 us at 2,048
//     tokens, a third one nothing), one warp issuing copies; three stages of K and V; P in buffers of its own.
// While the tensor core adds one tile's P V, the other tile's softmax runs.
// Masking, splits along the keys, the rescaling threshold and the output layout are those of attention_tc.cuh.
#pragma once

namespace tc2 {

using tc::commit;
using tc::desc_k_major;
using tc::desc_mn_major;
using tc::fence_after;
using tc::fence_before;
using tc::load32;
using tc::mma;
using tc::store32;
using tc::wait_loads;

constexpr int ROWS = 128;
constexpr int QTILES = 2;
constexpr int SOFTMAX_WARPS = 4 * QTILES;
constexpr int SCORE_WARP = SOFTMAX_WARPS, MMA_WARP = SOFTMAX_WARPS + 1, COPY_WARP = SOFTMAX_WARPS + 2;
constexpr int THREADS = (SOFTMAX_WARPS + 3) * 32;
constexpr int STAGES = 3;
constexpr int Q_BYTES = ROWS * HD * 2;             // per query tile
constexpr int P_BYTES = ROWS * BKV * 2;            // per query tile
constexpr int TMEM_COLS = 512;
constexpr bool FITS = 2 * QTILES * BKV + QTILES * HD <= TMEM_COLS;
constexpr int BARRIER_BYTES = 256;

constexpr size_t smem_bytes(int table_entries) {
  return 1024 + (size_t)QTILES * (Q_BYTES + P_BYTES) + (size_t)STAGES * TMA_STAGE_BYTES + BARRIER_BYTES +
         ((size_t)table_entries + 2) * sizeof(int);
}

__global__ void __launch_bounds__(THREADS, 1) attention_prefill_tc2_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ int pair_info[2];
  __shared__ uint32_t tmem_slot;
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* generic = smem_dyn + (base - raw);
  // layout: Q tiles | P tiles | stages (K then V) | barriers | page ids
  const uint32_t q_smem = base;
  const uint32_t p_smem = base + QTILES * Q_BYTES;
  const uint32_t stages = p_smem + QTILES * P_BYTES;
  const uint32_t bars = stages + STAGES * TMA_STAGE_BYTES;
  const uint32_t k_bar = bars, v_bar = k_bar + 8 * STAGES, empty_bar = v_bar + 8 * STAGES;
  const uint32_t s_bar = empty_bar + 8 * STAGES;          // [query tile][score buffer]
  const uint32_t p_bar = s_bar + 8 * 2 * QTILES;          // [query tile]
  const uint32_t o_bar = p_bar + 8 * QTILES;              // [query tile]
  const uint32_t free_bar = o_bar + 8 * QTILES;           // [query tile][score buffer]: the softmax has read the scores
  int* local_table = reinterpret_cast<int*>(generic + (stages - base) + STAGES * TMA_STAGE_BYTES + BARRIER_BYTES);

  const int tid = threadIdx.x, lane = tid & 31, warp = uniform_warp_index();
  const int kvh = (int)blockIdx.x % p.kv_heads, pair_rank = (int)blockIdx.x / p.kv_heads, split = blockIdx.z;
  if (tid == 0) {
    // a block takes two consecutive tiles of queries of one request; long ones first
    int total = 0;
    for (int s = 0; s < p.num_seqs; ++s) total += ((p.q_start[s + 1] - p.q_start[s] + p.bq - 1) / p.bq + 1) / 2;
    int remaining = total - 1 - pair_rank, seq = -1, pair = 0;
    for (int s = 0; s < p.num_seqs && remaining >= 0; ++s) {
      const int pairs = ((p.q_start[s + 1] - p.q_start[s] + p.bq - 1) / p.bq + 1) / 2;
      if (remaining < pairs) { seq = s; pair = remaining; break; }
      remaining -= pairs;
    }
    pair_info[0] = seq;
    pair_info[1] = pair;
  }
  __syncthreads();
  const int seq = pair_info[0];
  if (seq < 0) return;
  const int q_first = pair_info[1] * QTILES * p.bq;
  const int q_begin = p.q_start[seq];
  const int q_len = p.q_start[seq + 1] - q_begin;
  const int q_total = min(QTILES * p.bq, q_len - q_first);          // queries of both tiles together
  const int pos0 = p.start_pos[seq] + q_first;
  int lo = p.window > 0 ? max(pos0 - p.window + 1, 0) : 0;
  int hi = pos0 + q_total;
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
    if (page >= p.num_pages) page = -2;
    local_table[i - first_page] = page;
  }
  {  // stages start cleared: boxes of pages the request does not own are never fetched
    uint4* fill = reinterpret_cast<uint4*>(generic + (stages - base));
    for (int i = tid; i < STAGES * TMA_STAGE_BYTES / 16; i += THREADS) fill[i] = make_uint4(0, 0, 0, 0);
  }
  // this thread's row (softmax warps): which query tile, which query, which head
  const int qt = warp >> 2;                                          // query tile of a softmax warp
  const int r = (warp & 3) * 32 + lane;                              // row in the tile = tensor-memory lane
  const int qi = r / p.group, gg = r - qi * p.group;
  const int q_in_pair = qt * p.bq + qi;
  const bool row_valid = warp < SOFTMAX_WARPS && qi < p.bq && q_in_pair < q_total;
  const int row_token = q_begin + q_first + (row_valid ? q_in_pair : 0);
  const int row_pos = pos0 + q_in_pair;
  const int row_head = kvh * p.group + gg;
  // Everything above read what the step was given (lengths, positions, the block table) and cleared this block's own
  // shared memory, while the kernel before this one was still running; the queries and the newest keys are its work.
  pdl_wait();
  if (warp < SOFTMAX_WARPS) {
    // Q row into the K-major swizzled tile of its query tile: 64-column blocks of [128 rows][128 bytes]
    const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t)row_token * p.q_stride + (size_t)row_head * HD);
    unsigned char* q_tile = generic + qt * Q_BYTES;
#pragma unroll
    for (int c = 0; c < HD / 8; ++c) {
      const uint4 v = row_valid ? src[c] : make_uint4(0, 0, 0, 0);
      const int block = c >> 3, chunk = c & 7;
      *reinterpret_cast<uint4*>(q_tile + block * (ROWS * 128) + r * 128 + ((chunk ^ (r & 7)) << 4)) = v;
    }
  }
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(k_bar + 8 * s, 1);
      mbar_init(v_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int i = 0; i < 2 * QTILES; ++i) {
      mbar_init(s_bar + 8 * i, 1);
      mbar_init(free_bar + 8 * i, 4);
    }
    for (int i = 0; i < QTILES; ++i) {
      mbar_init(p_bar + 8 * i, 4);
      mbar_init(o_bar + 8 * i, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");     // Q tiles and cleared stages, before the async proxy touches them
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = tmem_slot;
  pdl_trigger();                                                      // tensor memory is held: the next kernel may be scheduled
  auto s_tmem = [&](int tile, int buffer) { return tmem_base + (uint32_t)((tile * 2 + buffer) * BKV); };
  auto o_tmem = [&](int tile) { return tmem_base + (uint32_t)(2 * QTILES * BKV + tile * HD); };

  if (warp == COPY_WARP) {
    // ------------------------------- copies: one box per lane, K's boxes first -------------------------------
    const int pages_per_tile = BKV >> p.page_shift;
    const int boxes = pages_per_tile * TMA_BLOCKS * 2;
    for (int tile = 0; tile < num_tiles; ++tile) {
      const int stage = tile % STAGES;
      if (tile >= STAGES) mbar_wait_bounded(empty_bar + 8 * stage, (uint32_t)(tile / STAGES - 1) & 1u, p.status);
      const uint32_t k_dst = stages + stage * TMA_STAGE_BYTES, v_dst = k_dst + TMA_TILE_BYTES;
      const int tile_first = k_first + tile * BKV;
      int wanted = 0;
      for (int j = lane; j < pages_per_tile; j += 32) {
        const int page = local_table[(tile_first >> p.page_shift) + j - first_page];
        if (page >= 0 && tile_first + (j << p.page_shift) < hi) ++wanted;
      }
      wanted = __reduce_add_sync(0xffffffffu, wanted);
      if (lane == 0) {
        mbar_expect_tx(k_bar + 8 * stage, (uint32_t)wanted * TMA_BLOCKS * (uint32_t)(p.page_size * 128));
        mbar_expect_tx(v_bar + 8 * stage, (uint32_t)wanted * TMA_BLOCKS * (uint32_t)(p.page_size * 128));
      }
      __syncwarp();
      for (int box = lane; box < boxes; box += 32) {
        const int which = box >= boxes / 2, rest = box - which * (boxes / 2);
        const int b = rest % TMA_BLOCKS, j = rest / TMA_BLOCKS;
        const int page = local_table[(tile_first >> p.page_shift) + j - first_page];
        if (page < 0 || tile_first + (j << p.page_shift) >= hi) continue;
        const int row = (page * p.kv_heads + kvh) << p.page_shift;
        const uint32_t offset = (uint32_t)(b * (BKV * 128) + (j << p.page_shift) * 128);
        tma_load_2d((which ? v_dst : k_dst) + offset, which ? &map_v : &map_k, (which ? v_bar : k_bar) + 8 * stage, b * 64, row);
      }
    }
  } else if (warp == SCORE_WARP) {
    // ------------------------------- score products -------------------------------
    // S = Q K^T of key tile j for both query tiles, into their score buffers (j & 1).  A buffer is free
    // once the softmax warps have read tile j - 2 out of it (a barrier of its own: a waiter that could fall
    // two phases behind cannot tell them apart by parity).
    if (elect_one()) {
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BKV >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
      for (int tile = 0; tile < num_tiles; ++tile) {
        const int stage = tile % STAGES;
        mbar_wait_bounded(k_bar + 8 * stage, (uint32_t)(tile / STAGES) & 1u, p.status);
        const uint64_t k_desc = desc_k_major(stages + stage * TMA_STAGE_BYTES);
#pragma unroll
        for (int t = 0; t < QTILES; ++t) {
          if (tile >= 2) mbar_wait_bounded(free_bar + 8 * (t * 2 + (tile & 1)), (uint32_t)((tile >> 1) - 1) & 1u, p.status);
          fence_after();
          const uint64_t q_desc = desc_k_major(q_smem + t * Q_BYTES);
          const uint32_t d_tmem = s_tmem(t, tile & 1);
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint32_t block = ks >> 2, step = ks & 3;
            mma(d_tmem, q_desc + ((block * (ROWS * 128) + step * 32) >> 4), k_desc + ((block * (BKV * 128) + step * 32) >> 4),
                idesc_s, ks > 0 ? 1u : 0u);
          }
          commit(s_bar + 8 * (t * 2 + (tile & 1)));
        }
      }
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------- P V products -------------------------------
    if (elect_one()) {
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
      for (int it = 0; it < num_tiles; ++it) {
        const int stage = it % STAGES;
        const uint64_t v_desc = desc_mn_major(stages + stage * TMA_STAGE_BYTES + TMA_TILE_BYTES, BKV * 128);
#pragma unroll
        for (int t = 0; t < QTILES; ++t) {
          mbar_wait_bounded(p_bar + 8 * t, (uint32_t)it & 1u, p.status);
          if (t == 0) mbar_wait_bounded(v_bar + 8 * stage, (uint32_t)(it / STAGES) & 1u, p.status);
          fence_after();
          const uint64_t p_desc = desc_k_major(p_smem + t * P_BYTES);
#pragma unroll
          for (int ks = 0; ks < BKV / 16; ++ks)
            mma(o_tmem(t), p_desc + ((ks * 32) >> 4), v_desc + ((ks * (16 * 128)) >> 4), idesc_o, (it > 0 || ks > 0) ? 1u : 0u);
          commit(o_bar + 8 * t);
        }
        // The stage is free once both products have read V; the scores that read its K were complete
        // before the softmax that these products waited for could start.
        commit(empty_bar + 8 * stage);
      }
    }
  } else {
    // ------------------------------- softmax, one row per thread -------------------------------
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const int first_key = p.window > 0 ? row_pos - p.window + 1 : 0;
    const uint32_t my_s_bar = s_bar + 8 * (qt * 2), my_p_bar = p_bar + 8 * qt, my_o_bar = o_bar + 8 * qt;
    const uint32_t my_o = o_tmem(qt);
    const uint32_t p_row = p_smem + qt * P_BYTES + r * 128;
    float m_run = -INFINITY, l_run = 0.0f;            // m_run: the row's reference, in raw score units
    const float step_raw = tc::RESCALE_STEP / p.scale_log2;
    bool bad_page = false;
    for (int it = 0; it < num_tiles; ++it) {
      const int k0 = k_first + it * BKV;
      mbar_wait_bounded(my_s_bar + 8 * (it & 1), (uint32_t)(it >> 1) & 1u, p.status);
      fence_after();
      if (local_table[(max(k0, lo) >> p.page_shift) - first_page] < 0) bad_page = true;
      uint32_t s_bits[BKV];
      const uint32_t s_now = s_tmem(qt, it & 1);
      load32(s_now + lane_base, s_bits);
      load32(s_now + lane_base + 32, s_bits + 32);
      wait_loads();
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(free_bar + 8 * (qt * 2 + (it & 1)));      // the buffer may take the scores of tile it + 2
      // a tile that every row of the warp sees whole needs no mask
      // (rows beyond the tile's queries hold zeros and are never stored: they need none either)
      const bool whole = !row_valid || (k0 + BKV - 1 <= row_pos && k0 >= first_key && k0 >= lo && k0 + BKV <= hi);
      float mx = -INFINITY;
      if (__all_sync(0xffffffffu, whole)) {
#pragma unroll
        for (int j = 0; j < BKV; j += 2) mx = tc::max3(mx, __uint_as_float(s_bits[j]), __uint_as_float(s_bits[j + 1]));
      } else {
#pragma unroll
        for (int j = 0; j < BKV; ++j) {
          const int kpos = k0 + j;
          const bool visible = row_valid && kpos <= row_pos && kpos >= first_key && kpos >= lo && kpos < hi;
          const float sv = visible ? __uint_as_float(s_bits[j]) : -INFINITY;
          s_bits[j] = __float_as_uint(sv);
          mx = fmaxf(mx, sv);
        }
      }
      const bool moved = mx > m_run + step_raw || m_run == -INFINITY;
      const float m_new = moved ? mx : m_run;
      const float m_use = m_new == -INFINITY ? 0.0f : m_new;
      const float corr = exp2f((m_run - m_use) * p.scale_log2);            // exp2(-inf) = 0 while nothing was visible yet
      const float shift = -m_use * p.scale_log2;
      const uint64_t scale2 = tc::pair(p.scale_log2, p.scale_log2), shift2 = tc::pair(shift, shift);
      uint64_t sum2 = tc::pair(0.0f, 0.0f);
      if (it > 0) {
        // P has one buffer per query tile, and the accumulator may be rescaled below: the previous tile's
        // product must have read the one and written the other
        mbar_wait_bounded(my_o_bar, (uint32_t)(it - 1) & 1u, p.status);
        fence_after();
      }
#pragma unroll
      for (int c = 0; c < BKV / 8; ++c) {
        float pv[8];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          float a, b;
          tc::unpair(tc::fma2(tc::pair(__uint_as_float(s_bits[c * 8 + e]), __uint_as_float(s_bits[c * 8 + e + 1])), scale2, shift2), a, b);
          pv[e] = tc::ex2(a);               // a masked score is -inf: 2^-inf = 0
          pv[e + 1] = tc::ex2(b);
          sum2 = tc::add2(sum2, tc::pair(pv[e], pv[e + 1]));
        }
        const uint32_t dst = p_row + ((c ^ (r & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(dst), "r"(pack_bf16(pv[0], pv[1])),
                     "r"(pack_bf16(pv[2], pv[3])), "r"(pack_bf16(pv[4], pv[5])), "r"(pack_bf16(pv[6], pv[7])) : "memory");
      }
      float sum_even, sum_odd;
      tc::unpair(sum2, sum_even, sum_odd);
      l_run = l_run * corr + (sum_even + sum_odd);
      const bool rescale = it > 0 && moved && m_run != -INFINITY;
      m_run = m_new;
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // P, before the tensor core reads it
      if (it > 0 && __any_sync(0xffffffffu, rescale)) {
        const float factor = rescale ? corr : 1.0f;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o_bits[32];
          load32(my_o + lane_base + c * 32, o_bits);
          wait_loads();
#pragma unroll
          for (int e = 0; e < 32; ++e) o_bits[e] = __float_as_uint(__uint_as_float(o_bits[e]) * factor);
          store32(my_o + lane_base + c * 32, o_bits);
        }
      }
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(my_p_bar);
    }
    if (bad_page && p.status) atomicOr(p.status, TGE_STATUS_BAD_PAGE);
    mbar_wait_bounded(my_o_bar, (uint32_t)(num_tiles - 1) & 1u, p.status);
    fence_after();
    const float inv = (p.num_splits == 1) ? (l_run > 0.0f ? 1.0f / l_run : 0.0f) : 1.0f;
    const size_t slot = ((size_t)split * p.total_tokens + row_token) * p.heads + row_head;
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) {
      uint32_t o_bits[32];
      load32(my_o + lane_base + c * 32, o_bits);           // every lane takes part in the load; only valid rows store
      wait_loads();
      if (!row_valid) continue;
      if (p.num_splits == 1) {
        uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)row_token * p.out_stride + (size_t)row_head * HD + c * 32);
#pragma unroll
        for (int e = 0; e < 4; ++e)
          dst[e] = make_uint4(pack_bf16(__uint_as_float(o_bits[e * 8]) * inv, __uint_as_float(o_bits[e * 8 + 1]) * inv),
                              pack_bf16(__uint_as_float(o_bits[e * 8 + 2]) * inv, __uint_as_float(o_bits[e * 8 + 3]) * inv),
                              pack_bf16(__uint_as_float(o_bits[e * 8 + 4]) * inv, __uint_as_float(o_bits[e * 8 + 5]) * inv),
                              pack_bf16(__uint_as_float(o_bits[e * 8 + 6]) * inv, __uint_as_float(o_bits[e * 8 + 7]) * inv));
      } else {
        float4* dst = reinterpret_cast<float4*>(p.partial_o + slot * HD + c * 32);
#pragma unroll
        for (int e = 0; e < 8; ++e)
          dst[e] = make_float4(__uint_as_float(o_bits[e * 4]), __uint_as_float(o_bits[e * 4 + 1]),
                               __uint_as_float(o_bits[e * 4 + 2]), __uint_as_float(o_bits[e * 4 + 3]));
      }
    }
    if (row_valid && p.num_splits > 1) {
      p.partial_ml[slot * 2] = m_run == -INFINITY ? -INFINITY : m_run * p.scale_log2;   // merged in scaled base-2 units
      p.partial_ml[slot * 2 + 1] = l_run;
    }
  }
  fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
  }
}

}  // namespace tc2
