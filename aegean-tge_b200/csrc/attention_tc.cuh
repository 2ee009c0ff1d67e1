// Prompt-portion attention on the 5th-generation tensor cores, for head sizes that are multiples of 64.
// Included by attention_mma.cu (which provides AttnParams, the TMA and mbarrier helpers and the
// page-pool tensor maps).
//
// A block owns 128 rows ((query, head-of-group) pairs of one kv head) = the 128 lanes of tensor memory.
// Per tile of 64 key positions:
//   1. K and V arrive by TMA (one box per page and 64 columns, 128-byte swizzle), two stages;
//   2. one thread issues S = Q K^T as tcgen05.mma (Q and K both K-major in shared memory) into
//      tensor-memory columns [0, 64);
//   3. the 128 softmax threads each read their own row with tcgen05.ld - the running maximum and sum
//      are thread-local, no shuffles - mask by position, exponentiate in float32 and write P (bfloat16)
//      into shared memory in the K-major swizzled layout, over the K tile that step 2 has finished with;
//   4. the issuing thread adds P V (V is MN-major in shared memory: head dimension contiguous) into the
//      output accumulator in columns [64, 64 + head_dim);
//   5. a row whose running maximum rose by more than 2^8 rescales its accumulator in tensor memory
//      (tcgen05.ld, multiply, tcgen05.st) before the next product is added; smaller rises keep the old
//      reference (probabilities then reach up to 256, which bfloat16 and the float32 sums hold without
//      loss); rows read their output once, at the end.
// Six warps: four do the softmax (one row per thread), one issues the products, one issues the TMA
// copies, its lanes one box each - a single thread that does both spends most of a tile's time issuing
// copies.  Two blocks fit on an SM, so one block's softmax overlaps the other's products.
// Masking, splits along the keys and the output layout are those of the other attention kernels.
#pragma once

namespace tc {

constexpr int ROWS = 128;
constexpr int THREADS = 192;                       // four softmax warps, one warp that issues products, one that issues copies
constexpr float RESCALE_STEP = 8.0f;               // in powers of two: how far a row's maximum may rise before its reference moves
constexpr int STAGES = 2;
constexpr int Q_BYTES = ROWS * HD * 2;
constexpr int P_BYTES = ROWS * BKV * 2;            // 16 KiB
constexpr bool P_OVER_K = TMA_TILE_BYTES >= P_BYTES;   // P reuses the K tile of its stage when that is large enough
constexpr int TMEM_COLS = (2 * BKV + HD) <= 128 ? 128 : ((2 * BKV + HD) <= 256 ? 256 : 512);   // two score buffers and the output, a power of two

__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void load32(uint32_t taddr, uint32_t r[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void wait_loads() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ void store32(uint32_t taddr, const uint32_t r[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31]) : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

// Two float32 lanes at a time (sm_100 has paired FMA and ADD), one MUFU exponential, three-input maximum:
// the softmax warps are bound by the number of instructions they issue per score.
__device__ __forceinline__ uint64_t pair(float lo, float hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void unpair(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float ex2(float x) {       // 2^x; arguments are <= 0 here, tiny results flush to zero
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// K-major operand: rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// MN-major operand (the contiguous direction is N): 64-element blocks of N `block_stride` bytes apart,
// groups of 8 k-rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t block_stride) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(block_stride >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

__global__ void __launch_bounds__(THREADS, 2) attention_prefill_tc_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ int tile_info[2];
  __shared__ uint32_t tmem_slot;
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* generic = smem_dyn + (base - raw);
  // layout: Q tile | [P tile] | stages (K then V) | barriers | page ids
  const uint32_t q_smem = base;
  const uint32_t p_own = base + Q_BYTES;                                   // used only when P does not fit over K
  const uint32_t stages = base + Q_BYTES + (P_OVER_K ? 0 : P_BYTES);
  const uint32_t bars = stages + STAGES * TMA_STAGE_BYTES;
  // full_bar: K of a stage has landed; v_bar: V has; s_bar: one per score buffer
  const uint32_t full_bar = bars, empty_bar = bars + 8 * STAGES, s_bar = bars + 16 * STAGES, p_bar = s_bar + 16, o_bar = s_bar + 24,
                 v_bar = s_bar + 32;
  int* local_table = reinterpret_cast<int*>(generic + (stages - base) + STAGES * TMA_STAGE_BYTES + 128);   // after the barriers

  const int tid = threadIdx.x, lane = tid & 31, warp = uniform_warp_index();
  // Blocks are handed out in the order of blockIdx.x: the kv head changes fastest, so that the long tiles of
  // every kv head start first and the short ones fill the gaps (with the kv head as blockIdx.y, a whole kv
  // head's long tiles started only after the first ones' short tiles).
  const int kvh = (int)blockIdx.x % p.kv_heads, tile_rank = (int)blockIdx.x / p.kv_heads, split = blockIdx.z;
  if (tid == 0) {
    int total = 0;
    for (int s = 0; s < p.num_seqs; ++s) total += (p.q_start[s + 1] - p.q_start[s] + p.bq - 1) / p.bq;
    int remaining = total - 1 - tile_rank, seq = -1, tile = 0;                // long tiles first
    for (int s = 0; s < p.num_seqs && remaining >= 0; ++s) {
      const int tiles = (p.q_start[s + 1] - p.q_start[s] + p.bq - 1) / p.bq;
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
  for (int i = first_page + tid; i <= last_page; i += THREADS) {
    int page = i < p.max_pages ? p.block_table[(size_t)seq * p.max_pages + i] : -1;
    if (page >= p.num_pages) page = -2;
    local_table[i - first_page] = page;
  }
  {  // stages start cleared: boxes of pages the request does not own are never fetched
    uint4* fill = reinterpret_cast<uint4*>(generic + (stages - base));
    for (int i = tid; i < STAGES * TMA_STAGE_BYTES / 16; i += THREADS) fill[i] = make_uint4(0, 0, 0, 0);
  }
  // this thread's row (softmax warps): which query, which head
  const int r = tid;
  const int qi = r / p.group, gg = r - qi * p.group;
  const bool row_valid = tid < ROWS && qi < q_count;
  const int row_token = q_begin + q_first + (row_valid ? qi : 0);
  const int row_pos = pos0 + qi;
  const int row_head = kvh * p.group + gg;
  // Everything above read what the step was given (lengths, positions, the block table) and cleared this block's own
  // shared memory, while the kernel before this one was still running; the queries and the newest keys are its work.
  pdl_wait();
  if (tid < ROWS) {
    // Q row into the K-major swizzled tile: 64-column blocks of [128 rows][128 bytes]
    const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t)row_token * p.q_stride + (size_t)row_head * HD);
#pragma unroll
    for (int c = 0; c < HD / 8; ++c) {
      const uint4 v = row_valid ? src[c] : make_uint4(0, 0, 0, 0);
      const int block = c >> 3, chunk = c & 7;
      *reinterpret_cast<uint4*>(generic + block * (ROWS * 128) + r * 128 + ((chunk ^ (r & 7)) << 4)) = v;
    }
  }
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(v_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    mbar_init(s_bar, 1);
    mbar_init(s_bar + 8, 1);
    mbar_init(p_bar, 4);
    mbar_init(o_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");     // Q tile and cleared stages, before the async proxy reads or writes them
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = tmem_slot;
  pdl_trigger();                                                      // tensor memory is held: the next kernel may be scheduled
  const uint32_t s_tmem = tmem_base, o_tmem = tmem_base + 2 * BKV;

  if (warp == 5) {
    // ------------------------------- copies: one box per lane -------------------------------
    // A tile is (pages per tile) x (64-column blocks) x (K, V) boxes.  Each lane takes boxes of its own;
    // the first lane announces the bytes of those that will really be fetched.
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
        mbar_expect_tx(full_bar + 8 * stage, (uint32_t)wanted * TMA_BLOCKS * (uint32_t)(p.page_size * 128));
        mbar_expect_tx(v_bar + 8 * stage, (uint32_t)wanted * TMA_BLOCKS * (uint32_t)(p.page_size * 128));
      }
      __syncwarp();
      // K's boxes first: the scores of the tile can start while V is still on its way
      for (int box = lane; box < boxes; box += 32) {
        const int which = box >= boxes / 2, rest = box - which * (boxes / 2);
        const int b = rest % TMA_BLOCKS, j = rest / TMA_BLOCKS;
        const uint32_t bar = (which ? v_bar : full_bar) + 8 * stage;
        const int page = local_table[(tile_first >> p.page_shift) + j - first_page];
        if (page < 0 || tile_first + (j << p.page_shift) >= hi) continue;
        const int row = (page * p.kv_heads + kvh) << p.page_shift;
        const uint32_t offset = (uint32_t)(b * (BKV * 128) + (j << p.page_shift) * 128);
        tma_load_2d((which ? v_dst : k_dst) + offset, which ? &map_v : &map_k, bar, b * 64, row);
      }
    }
  } else if (warp == 4) {
    // ------------------------------- products -------------------------------
    if (elect_one()) {
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BKV >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
      const uint64_t q_desc = desc_k_major(q_smem);
      // S = Q K^T of one tile into score buffer (tile & 1); descriptors move by (byte offset >> 4)
      auto issue_scores = [&](int tile) {
        const int stage = tile % STAGES;
        mbar_wait_bounded(full_bar + 8 * stage, (uint32_t)(tile / STAGES) & 1u, p.status);
        fence_after();
        const uint64_t k_desc = desc_k_major(stages + stage * TMA_STAGE_BYTES);
        const uint32_t d_tmem = s_tmem + (uint32_t)((tile & 1) * BKV);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t block = ks >> 2, step = ks & 3;
          mma(d_tmem, q_desc + ((block * (ROWS * 128) + step * 32) >> 4), k_desc + ((block * (BKV * 128) + step * 32) >> 4),
              idesc_s, ks > 0 ? 1u : 0u);
        }
        commit(s_bar + 8 * (tile & 1));
      };
      issue_scores(0);
      for (int it = 0; it < num_tiles; ++it) {
        const int stage = it % STAGES;
        // the next tile's scores are computed while the softmax warps work on this tile's
        if (it + 1 < num_tiles) issue_scores(it + 1);
        mbar_wait_bounded(p_bar, (uint32_t)it & 1u, p.status);
        mbar_wait_bounded(v_bar + 8 * stage, (uint32_t)(it / STAGES) & 1u, p.status);
        fence_after();
        const uint32_t k_tile = stages + stage * TMA_STAGE_BYTES, v_tile = k_tile + TMA_TILE_BYTES;
        const uint64_t p_desc = desc_k_major(P_OVER_K ? k_tile : p_own), v_desc = desc_mn_major(v_tile, BKV * 128);
#pragma unroll
        for (int ks = 0; ks < BKV / 16; ++ks)
          mma(o_tmem, p_desc + ((ks * 32) >> 4), v_desc + ((ks * (16 * 128)) >> 4), idesc_o, (it > 0 || ks > 0) ? 1u : 0u);
        commit(o_bar);
        commit(empty_bar + 8 * stage);      // the stage is free once this product has read P and V
      }
    }
  } else {
    // ------------------------------- softmax, one row per thread -------------------------------
    // The output accumulates in tensor memory across tiles.  A row's running maximum is in raw score
    // units; when it rises, the row's accumulator is rescaled in tensor memory before the next product
    // is added (a whole warp does it together, rows whose maximum stood still use a factor of one).
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const int first_key = p.window > 0 ? row_pos - p.window + 1 : 0;
    float m_run = -INFINITY, l_run = 0.0f;            // m_run: the row's reference, in raw score units
    const float step_raw = RESCALE_STEP / p.scale_log2;
    bool bad_page = false;
    for (int it = 0; it < num_tiles; ++it) {
      const int stage = it % STAGES;
      const int k0 = k_first + it * BKV;
      mbar_wait_bounded(s_bar + 8 * (it & 1), (uint32_t)(it >> 1) & 1u, p.status);
      fence_after();
      if (local_table[(max(k0, lo) >> p.page_shift) - first_page] < 0) bad_page = true;
      uint32_t s_bits[BKV];
      const uint32_t s_now = s_tmem + (uint32_t)((it & 1) * BKV);
      load32(s_now + lane_base, s_bits);
      load32(s_now + lane_base + 32, s_bits + 32);
      wait_loads();
      // a tile that every row of the warp sees whole needs no mask
      // (rows beyond the tile's queries hold zeros and are never stored: they need none either)
      const bool whole = !row_valid || (k0 + BKV - 1 <= row_pos && k0 >= first_key && k0 >= lo && k0 + BKV <= hi);
      float mx = -INFINITY;
      if (__all_sync(0xffffffffu, whole)) {
#pragma unroll
        for (int j = 0; j < BKV; j += 2) mx = max3(mx, __uint_as_float(s_bits[j]), __uint_as_float(s_bits[j + 1]));
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
      // The reference that exponents are taken against moves only when the maximum rose by more than
      // RESCALE_STEP powers of two (or nothing was visible so far): the accumulator in tensor memory is
      // then seldom rescaled after the first tiles.
      const bool moved = mx > m_run + step_raw || m_run == -INFINITY;
      const float m_new = moved ? mx : m_run;
      const float m_use = m_new == -INFINITY ? 0.0f : m_new;
      const float corr = exp2f((m_run - m_use) * p.scale_log2);            // exp2(-inf) = 0 while nothing was visible yet
      const float shift = -m_use * p.scale_log2;
      const uint64_t scale2 = pair(p.scale_log2, p.scale_log2), shift2 = pair(shift, shift);
      uint64_t sum2 = pair(0.0f, 0.0f);
      const uint32_t p_row = (P_OVER_K ? stages + stage * TMA_STAGE_BYTES : p_own) + r * 128;
      if (!P_OVER_K && it > 0) {
        // P has one buffer of its own here: the previous tile's product must have read it
        mbar_wait_bounded(o_bar, (uint32_t)(it - 1) & 1u, p.status);
        fence_after();
      }
#pragma unroll
      for (int c = 0; c < BKV / 8; ++c) {
        float pv[8];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          float a, b;
          unpair(fma2(pair(__uint_as_float(s_bits[c * 8 + e]), __uint_as_float(s_bits[c * 8 + e + 1])), scale2, shift2), a, b);
          pv[e] = ex2(a);               // a masked score is -inf: 2^-inf = 0
          pv[e + 1] = ex2(b);
          sum2 = add2(sum2, pair(pv[e], pv[e + 1]));
        }
        const uint32_t dst = p_row + ((c ^ (r & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(dst), "r"(pack_bf16(pv[0], pv[1])),
                     "r"(pack_bf16(pv[2], pv[3])), "r"(pack_bf16(pv[4], pv[5])), "r"(pack_bf16(pv[6], pv[7])) : "memory");
      }
      float sum_even, sum_odd;
      unpair(sum2, sum_even, sum_odd);
      l_run = l_run * corr + (sum_even + sum_odd);
      const bool rescale = it > 0 && moved && m_run != -INFINITY;
      m_run = m_new;
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // P, before the tensor core reads it
      if (it > 0) {
        // the previous product must have landed before this tile's is added (and before any rescaling)
        mbar_wait_bounded(o_bar, (uint32_t)(it - 1) & 1u, p.status);
        fence_after();
        if (__any_sync(0xffffffffu, rescale)) {
          const float factor = rescale ? corr : 1.0f;
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o_bits[32];
            load32(o_tmem + lane_base + c * 32, o_bits);
            wait_loads();
#pragma unroll
            for (int e = 0; e < 32; ++e) o_bits[e] = __float_as_uint(__uint_as_float(o_bits[e]) * factor);
            store32(o_tmem + lane_base + c * 32, o_bits);
          }
        }
      }
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_bar);
    }
    if (bad_page && p.status) atomicOr(p.status, TGE_STATUS_BAD_PAGE);
    mbar_wait_bounded(o_bar, (uint32_t)(num_tiles - 1) & 1u, p.status);
    fence_after();
    const float inv = (p.num_splits == 1) ? (l_run > 0.0f ? 1.0f / l_run : 0.0f) : 1.0f;
    const size_t slot = ((size_t)split * p.total_tokens + row_token) * p.heads + row_head;
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) {
      uint32_t o_bits[32];
      load32(o_tmem + lane_base + c * 32, o_bits);           // every lane takes part in the load; only valid rows store
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
  if (warp == 4) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
  }
}

constexpr size_t smem_bytes(int table_entries) {
  return 1024 + Q_BYTES + (P_OVER_K ? 0 : P_BYTES) + (size_t)STAGES * TMA_STAGE_BYTES + 128 + ((size_t)table_entries + 2) * sizeof(int);
}

}  // namespace tc
