// Embedding, RMSNorm, residual add, rotary rotation fused with the cache store.
//
// Formulas follow the reference's scalar kernels:
//   rms norm     src/cpu/scalar/norm_rope_scalar.cpp:8-21
//   rotate-half  src/cpu/scalar/norm_rope_scalar.cpp:23-41
//   cache write  src/models/qwen2.cpp:2308-2329 (rotated K and plain V, after the bias)
//   embedding    src/models/qwen2.cpp:1143-1152
#include "common.cuh"

// ---------------------------------------------------------------------------
// embedding: x[t, :] = table[ids[t], :] as float32
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int hidden, int vocab, int* status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* dst = out + (size_t)t * hidden;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, TGE_STATUS_BAD_TOKEN);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.0f;
    return;
  }
  const T* src = table + (size_t)id * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_float<T>(src[i]);
}

TGE_API int tge_embedding(const void* table, int is_bf16, const int* ids, float* out, int tokens,
                          int hidden, int vocab, int* status, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0, "embedding: bad sizes tokens=%d hidden=%d vocab=%d",
              tokens, hidden, vocab);
  if (tokens == 0) return 0;
  if (is_bf16)
    tge_launch(embedding_kernel<__nv_bfloat16>, tokens, 256, 0, stream, (const __nv_bfloat16*)table, ids, out, hidden, vocab, status);
  else
    tge_launch(embedding_kernel<float>, tokens, 256, 0, stream, (const float*)table, ids, out, hidden, vocab, status);
  return tge_launched("embedding", 1);
}

// ---------------------------------------------------------------------------
// RMSNorm over the float32 stream; output in the run dtype.
//   s = sum x_i^2 ; scale = 1 / sqrt(s / dim + eps) ; out_i = x_i * scale * w_i
// One block per output row; optional row gather (rows[r] = source row).
// ---------------------------------------------------------------------------
template <typename TOut>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                               const int* __restrict__ rows, TOut* __restrict__ out, int hidden,
                               int src_rows, float eps, int* status) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  int src = rows ? rows[r] : r;
  if (src < 0 || src >= src_rows) {
    if (threadIdx.x == 0) atomicOr(status, TGE_STATUS_BAD_ROW);
    src = 0;
  }
  const float* in = x + (size_t)src * hidden;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = in[i];
    sum = fmaf(v, v, sum);
  }
  sum = block_sum(sum, scratch);
  const float scale = 1.0f / sqrtf(sum / (float)hidden + eps);
  TOut* dst = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = from_float<TOut>(in[i] * scale * weight[i]);
}

// The same with 16-byte loads and the row held in registers between the two passes:
// hidden a multiple of 4 and at most 16 values per thread.
constexpr int NORM_VEC_ITERS = 4;

__device__ __forceinline__ void store4(float* dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 packed;
  packed.x = *reinterpret_cast<const uint32_t*>(&lo);
  packed.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = packed;
}

template <typename TOut>
__global__ void __launch_bounds__(512) rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                                          const int* __restrict__ rows, TOut* __restrict__ out,
                                                          int hidden, int src_rows, float eps, int* status) {
  __shared__ float scratch[32];
  pdl_trigger();
  const int quads = hidden >> 2;
  float4 gain[NORM_VEC_ITERS], value[NORM_VEC_ITERS];
#pragma unroll
  for (int k = 0; k < NORM_VEC_ITERS; ++k) {      // constants of the model: before the wait
    const int i = threadIdx.x + k * blockDim.x;
    gain[k] = i < quads ? reinterpret_cast<const float4*>(weight)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  const int r = blockIdx.x;
  int src = rows ? rows[r] : r;
  if (src < 0 || src >= src_rows) {
    if (threadIdx.x == 0) atomicOr(status, TGE_STATUS_BAD_ROW);
    src = 0;
  }
  const float4* in = reinterpret_cast<const float4*>(x + (size_t)src * hidden);
  float sum = 0.0f;
#pragma unroll
  for (int k = 0; k < NORM_VEC_ITERS; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    value[k] = i < quads ? in[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    sum = fmaf(value[k].x, value[k].x, sum);
    sum = fmaf(value[k].y, value[k].y, sum);
    sum = fmaf(value[k].z, value[k].z, sum);
    sum = fmaf(value[k].w, value[k].w, sum);
  }
  sum = block_sum(sum, scratch);
  const float scale = 1.0f / sqrtf(sum / (float)hidden + eps);
  TOut* dst = out + (size_t)r * hidden;
#pragma unroll
  for (int k = 0; k < NORM_VEC_ITERS; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < quads)
      store4(dst + 4 * (size_t)i, value[k].x * scale * gain[k].x, value[k].y * scale * gain[k].y,
             value[k].z * scale * gain[k].z, value[k].w * scale * gain[k].w);
  }
}

TGE_API int tge_rmsnorm(const float* x, const float* weight, const int* rows, void* out, int out_is_bf16,
                        int out_rows, int src_rows, int hidden, float eps, int* status, cudaStream_t stream) {
  TGE_REQUIRE(out_rows >= 0 && hidden > 0 && src_rows >= 0, "rmsnorm: bad sizes rows=%d hidden=%d", out_rows, hidden);
  TGE_REQUIRE(eps > 0.0f, "rmsnorm: eps must be positive");
  if (out_rows == 0) return 0;
  int threads = hidden >= 2048 ? 512 : 256;
  const bool aligned = ((uintptr_t)x | (uintptr_t)weight | (uintptr_t)out) % 16 == 0;
  if (hidden % 4 == 0 && hidden / 4 <= NORM_VEC_ITERS * threads && aligned) {
    // more and smaller blocks per SM keep more loads in flight while others sit in their reduction
    if (hidden / 4 <= NORM_VEC_ITERS * 256) threads = 256;
    if (out_is_bf16)
      tge_launch(rmsnorm_vec_kernel<__nv_bfloat16>, out_rows, threads, 0, stream, x, weight, rows, (__nv_bfloat16*)out, hidden, src_rows, eps, status);
    else
      tge_launch(rmsnorm_vec_kernel<float>, out_rows, threads, 0, stream, x, weight, rows, (float*)out, hidden, src_rows, eps, status);
    return tge_launched("rmsnorm", 1);
  }
  if (out_is_bf16)
    tge_launch(rmsnorm_kernel<__nv_bfloat16>, out_rows, threads, 0, stream, x, weight, rows, (__nv_bfloat16*)out, hidden, src_rows, eps, status);
  else
    tge_launch(rmsnorm_kernel<float>, out_rows, threads, 0, stream, x, weight, rows, (float*)out, hidden, src_rows, eps, status);
  return tge_launched("rmsnorm", 1);
}

// ---------------------------------------------------------------------------
// x += y  (float32 stream, y in the run dtype)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void add_to_stream_kernel(float* __restrict__ x, const T* __restrict__ y, size_t count) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < count; i += stride) x[i] += to_float<T>(y[i]);
}

TGE_API int tge_add_to_stream(float* x, const void* y, int y_is_bf16, long long count, cudaStream_t stream) {
  TGE_REQUIRE(count >= 0, "add_to_stream: negative count");
  if (count == 0) return 0;
  long long blocks = (count + 255) / 256;
  if (blocks > tge_sm_count() * 16) blocks = tge_sm_count() * 16;
  if (y_is_bf16)
    add_to_stream_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(x, (const __nv_bfloat16*)y, (size_t)count);
  else
    add_to_stream_kernel<float><<<(int)blocks, 256, 0, stream>>>(x, (const float*)y, (size_t)count);
  return tge_launched("add_to_stream", 1);
}

// ---------------------------------------------------------------------------
// Rotary rotation of q and k (rotate-half pairing over the first `rotary`
// dimensions of each head) fused with the store of k and v into their pages.
//   lo' = lo*cos - hi*sin ; hi' = lo*sin + hi*cos      (float32)
// q is rotated in place inside the fused qkv rows; k is rotated on its way into
// the cache, v is copied.  A page is [kv_heads, page_size, head_dim].
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_store_kernel(T* __restrict__ qkv, int row_stride, const float* __restrict__ cos_table,
                                     const float* __restrict__ sin_table, int table_rows,
                                     const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                     const int* __restrict__ block_table, int max_pages, T* __restrict__ k_pages,
                                     T* __restrict__ v_pages, int num_pages, int page_size, int heads, int kv_heads,
                                     int head_dim, int rotary, int store_kv, int* status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  T* row = qkv + (size_t)t * row_stride;
  const int half = rotary / 2;
  const bool rotate = half > 0;
  if (rotate && (pos < 0 || pos >= table_rows)) {
    if (threadIdx.x == 0) atomicOr(status, TGE_STATUS_BAD_ROW);
    return;
  }
  const float* cs = cos_table + (size_t)pos * half;
  const float* sn = sin_table + (size_t)pos * half;
  // queries, in place
  if (rotate) {
    for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
      const int h = i / half, d = i - h * half;
      T* v = row + (size_t)h * head_dim;
      const float lo = to_float<T>(v[d]), hi = to_float<T>(v[d + half]);
      const float c = cs[d], s = sn[d];
      v[d] = from_float<T>(lo * c - hi * s);
      v[d + half] = from_float<T>(lo * s + hi * c);
    }
  }
  if (!store_kv) return;
  const int seq = seq_of_token[t];
  const int page = block_table[(size_t)seq * max_pages + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, TGE_STATUS_BAD_PAGE);
    return;
  }
  const int slot = pos % page_size;
  const T* k_row = row + (size_t)heads * head_dim;
  const T* v_row = k_row + (size_t)kv_heads * head_dim;
  for (int i = threadIdx.x; i < kv_heads * head_dim; i += blockDim.x) {
    const int h = i / head_dim, d = i - h * head_dim;
    const size_t dst = (((size_t)page * kv_heads + h) * page_size + slot) * head_dim + d;
    float kv;
    if (d < half) {
      const float lo = to_float<T>(k_row[i]), hi = to_float<T>(k_row[i + half]);
      kv = lo * cs[d] - hi * sn[d];
    } else if (d < rotary) {
      const float lo = to_float<T>(k_row[i - half]), hi = to_float<T>(k_row[i]);
      kv = lo * sn[d - half] + hi * cs[d - half];
    } else {
      kv = to_float<T>(k_row[i]);
    }
    k_pages[dst] = from_float<T>(kv);
    v_pages[dst] = v_row[i];
  }
}

// bfloat16 with everything a multiple of 8 elements: units of 16 bytes.  A unit is either a rotation
// (8 low and the 8 matching high elements of a q or k head) or a plain copy (v, and the tail of a k head
// beyond the rotary width).  Same formulas as above.
__device__ __forceinline__ void unpack8(const uint4& raw, float f[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(h[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
}
__device__ __forceinline__ uint4 pack8(const float f[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return raw;
}

__global__ void rope_kv_store_vec_kernel(__nv_bfloat16* __restrict__ qkv, int row_stride, const float* __restrict__ cos_table,
                                         const float* __restrict__ sin_table, int table_rows,
                                         const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                         const int* __restrict__ block_table, int max_pages,
                                         __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                                         int num_pages, int page_size, int heads, int kv_heads, int head_dim, int rotary,
                                         int store_kv, int* status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  __nv_bfloat16* row = qkv + (size_t)t * row_stride;
  const int half = rotary / 2;
  const int rot_units = half / 8, tail_units = (head_dim - rotary) / 8, dim_units = head_dim / 8;
  const int q_units = heads * rot_units;
  const int k_rot_units = store_kv ? kv_heads * rot_units : 0;
  const int k_tail_units = store_kv ? kv_heads * tail_units : 0;
  const int v_units = store_kv ? kv_heads * dim_units : 0;
  const int rotations = q_units + k_rot_units;
  const int total = rotations + k_tail_units + v_units;
  for (int u = threadIdx.x; u < total; u += blockDim.x) {
    // where the unit comes from depends on nothing that has to be looked up: ask for the data first,
    // then walk the chain position -> page
    int h, d;
    const __nv_bfloat16* src;
    __nv_bfloat16* page_base;      // k or v pages for units that go to the cache
    const bool rotation = u < rotations, is_q = u < q_units;
    if (rotation) {
      const int v = is_q ? u : u - q_units;
      h = v / rot_units; d = (v - h * rot_units) * 8;
      src = row + (size_t)(is_q ? h : heads + h) * head_dim + d;
      page_base = k_pages;
    } else if (u < rotations + k_tail_units) {
      const int v = u - rotations;
      h = v / tail_units; d = rotary + (v - h * tail_units) * 8;
      src = row + (size_t)(heads + h) * head_dim + d;
      page_base = k_pages;
    } else {
      const int v = u - rotations - k_tail_units;
      h = v / dim_units; d = (v - h * dim_units) * 8;
      src = row + (size_t)(heads + kv_heads + h) * head_dim + d;
      page_base = v_pages;
    }
    const uint4 first = *reinterpret_cast<const uint4*>(src);
    uint4 second = first;
    if (rotation) second = *reinterpret_cast<const uint4*>(src + half);
    const int pos = positions[t];
    if (rotation && (pos < 0 || pos >= table_rows)) {
      atomicOr(status, TGE_STATUS_BAD_ROW);
      continue;
    }
    __nv_bfloat16* dst = row + (size_t)h * head_dim + d;
    if (!is_q) {
      const int page = block_table[(size_t)seq_of_token[t] * max_pages + pos / page_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(status, TGE_STATUS_BAD_PAGE);
        continue;
      }
      dst = page_base + (((size_t)page * kv_heads + h) * page_size + pos % page_size) * head_dim + d;
    }
    if (!rotation) {
      *reinterpret_cast<uint4*>(dst) = first;
      continue;
    }
    const float* cs = cos_table + (size_t)pos * half + d;
    const float* sn = sin_table + (size_t)pos * half + d;
    float lo[8], hi[8], c[8], s[8], out_lo[8], out_hi[8];
    *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cs);
    *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cs + 4);
    *reinterpret_cast<float4*>(s) = *reinterpret_cast<const float4*>(sn);
    *reinterpret_cast<float4*>(s + 4) = *reinterpret_cast<const float4*>(sn + 4);
    unpack8(first, lo);
    unpack8(second, hi);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      out_lo[i] = lo[i] * c[i] - hi[i] * s[i];
      out_hi[i] = lo[i] * s[i] + hi[i] * c[i];
    }
    *reinterpret_cast<uint4*>(dst) = pack8(out_lo);
    *reinterpret_cast<uint4*>(dst + half) = pack8(out_hi);
  }
}

TGE_API int tge_rope_kv_store(void* qkv, int is_bf16, int row_stride, const float* cos_table, const float* sin_table,
                              int table_rows, const int* positions, const int* seq_of_token, const int* block_table,
                              int max_pages, void* k_pages, void* v_pages, int num_pages, int page_size, int tokens,
                              int heads, int kv_heads, int head_dim, int rotary, int store_kv, int* status,
                              cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && heads > 0 && kv_heads >= 0 && head_dim > 0, "rope_kv_store: bad sizes");
  TGE_REQUIRE(rotary >= 0 && rotary <= head_dim && rotary % 2 == 0,
              "rope_kv_store: rotary width %d must be even and at most head_dim %d", rotary, head_dim);
  TGE_REQUIRE(!store_kv || (page_size > 0 && max_pages > 0 && num_pages > 0), "rope_kv_store: bad page geometry");
  TGE_REQUIRE(row_stride >= (heads + (store_kv ? 2 * kv_heads : 0)) * head_dim, "rope_kv_store: row stride %d too small", row_stride);
  if (tokens == 0) return 0;
  const bool by_sixteen_bytes = is_bf16 && rotary % 16 == 0 && head_dim % 8 == 0 && row_stride % 8 == 0 &&
                                ((uintptr_t)qkv | (uintptr_t)cos_table | (uintptr_t)sin_table) % 16 == 0 &&
                                (!store_kv || ((uintptr_t)k_pages | (uintptr_t)v_pages) % 16 == 0);
  if (by_sixteen_bytes) {
    const int units = heads * (rotary / 16) + (store_kv ? kv_heads * (rotary / 16 + (head_dim - rotary) / 8 + head_dim / 8) : 0);
    int threads = (units + 31) / 32 * 32;
    if (threads > 512) threads = 512;
    if (threads < 32) threads = 32;
    tge_launch(rope_kv_store_vec_kernel, tokens, threads, 0, stream,
        (__nv_bfloat16*)qkv, row_stride, cos_table, sin_table, table_rows, positions, seq_of_token, block_table,
        max_pages, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, num_pages, page_size, heads, kv_heads, head_dim,
        rotary, store_kv, status);
    return tge_launched("rope_kv_store", 1);
  }
  if (is_bf16)
    tge_launch(rope_kv_store_kernel<__nv_bfloat16>, tokens, 256, 0, stream,
        (__nv_bfloat16*)qkv, row_stride, cos_table, sin_table, table_rows, positions, seq_of_token, block_table,
        max_pages, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, num_pages, page_size, heads, kv_heads, head_dim,
        rotary, store_kv, status);
  else
    tge_launch(rope_kv_store_kernel<float>, tokens, 256, 0, stream,
        (float*)qkv, row_stride, cos_table, sin_table, table_rows, positions, seq_of_token, block_table, max_pages,
        (float*)k_pages, (float*)v_pages, num_pages, page_size, heads, kv_heads, head_dim, rotary, store_kv, status);
  return tge_launched("rope_kv_store", 1);
}

// out[m, n] = rows[m, n] / sqrt(sum over slices of sums[slice][m] / width + eps), bfloat16: completes rows that
// travelled without their RMSNorm factor, for a taker that cannot apply it itself.
namespace {
__global__ void scale_rows_kernel(const __nv_bfloat16* __restrict__ rows, long long ld_rows, const float* __restrict__ sums,
                                  int slices, int width, float eps, __nv_bfloat16* __restrict__ out, long long ld_out,
                                  int m_rows, int n_cols) {
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x;
  float sum = 0.0f;
  for (int slice = 0; slice < slices; ++slice) sum += sums[(size_t)slice * m_rows + m];
  const float factor = 1.0f / sqrtf(sum / (float)width + eps);
  for (int n = threadIdx.x; n < n_cols; n += blockDim.x)
    out[(size_t)m * ld_out + n] = __float2bfloat16_rn(__bfloat162float(rows[(size_t)m * ld_rows + n]) * factor);
}
}  // namespace

TGE_API int tge_scale_rows(const void* rows, long long ld_rows, const float* sums, int slices, int width, float eps,
                           void* out, long long ld_out, int m_rows, int n_cols, cudaStream_t stream) {
  TGE_REQUIRE(m_rows >= 0 && n_cols > 0 && slices > 0 && width > 0, "scale_rows: bad sizes");
  if (m_rows == 0) return 0;
  tge_launch(scale_rows_kernel, m_rows, 256, 0, stream, (const __nv_bfloat16*)rows, ld_rows, sums, slices, width, eps,
             (__nv_bfloat16*)out, ld_out, m_rows, n_cols);
  return tge_launched("scale_rows", 1);
}
