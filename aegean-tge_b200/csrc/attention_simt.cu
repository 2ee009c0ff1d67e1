// Paged causal attention on the CUDA cores, any head size, float32 arithmetic.
//
// One warp per (token, query head).  Keys are visited in position order with a
// running maximum, so a row's result depends only on its own keys, never on
// the batch it arrives in or on how its request was cut into portions.  It is
// the attention of the whole float32 path and of head sizes the tensor-core
// kernel was not compiled for.
//
// Per query head h at position p (reference: src/cpu/scalar/attention_scalar.cpp:48-115,
// src/models/qwen2.cpp:1243-1304): kv head = h / group; for t in [first, p]:
// s_t = dot(q, K_t) * scale (dot first, scale after); softmax over s; out = sum w_t V_t.
// The causal mask is the loop bound; `window` > 0 additionally drops keys older
// than p - window + 1.
#include "common.cuh"

namespace {

constexpr int MAX_PER_LANE = 8;  // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(128) attention_simt_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
    const int* __restrict__ block_table, int max_pages, int num_pages, int page_size,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, T* __restrict__ out, int out_stride,
    int heads, int kv_heads, int head_dim, float scale, int window, int* status) {
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * 4 + warp;
  if (h >= heads) return;
  const int group = heads / kv_heads;
  const int kvh = h / group;
  const int pos = positions[t];
  const int seq = seq_of_token[t];
  const int* table = block_table + (size_t)seq * max_pages;

  float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * head_dim;
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < head_dim ? to_float<T>(qrow[d]) : 0.0f;
    acc[i] = 0.0f;
  }
  float m = -INFINITY, l = 0.0f;
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  for (int page_index = first / page_size; page_index * page_size <= pos; ++page_index) {
    const int page = page_index < max_pages ? table[page_index] : -1;
    if (page < 0 || page >= num_pages) {
      if (lane == 0) atomicOr(status, TGE_STATUS_BAD_PAGE);
      break;
    }
    const size_t base = ((size_t)page * kv_heads + kvh) * page_size * head_dim;
    const int lo = max(first - page_index * page_size, 0);
    const int hi = min(pos - page_index * page_size, page_size - 1);
    for (int slot = lo; slot <= hi; ++slot) {
      const T* krow = k_pages + base + (size_t)slot * head_dim;
      const T* vrow = v_pages + base + (size_t)slot * head_dim;
      float dot = 0.0f;
#pragma unroll
      for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) dot = fmaf(qv[i], to_float<T>(krow[d]), dot);
      }
      dot = warp_sum(dot);
      const float s = dot * scale;
      const float m_new = fmaxf(m, s);
      const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first key
      const float p = expf(s - m_new);
      l = l * corr + p;
#pragma unroll
      for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) acc[i] = fmaf(p, to_float<T>(vrow[d]), acc[i] * corr);
      }
      m = m_new;
    }
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  T* orow = out + (size_t)t * out_stride + (size_t)h * head_dim;
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    if (d < head_dim) orow[d] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace

TGE_API int tge_attention_simt(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                               const int* block_table, int max_pages, int num_pages, int page_size,
                               const int* positions, const int* seq_of_token, void* out, int out_stride, int tokens,
                               int heads, int kv_heads, int head_dim, float scale, int window, int is_bf16,
                               int* status, cudaStream_t stream) {
  TGE_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
              "attention: heads %d must be a positive multiple of kv heads %d", heads, kv_heads);
  TGE_REQUIRE(head_dim > 0 && head_dim <= 32 * MAX_PER_LANE, "attention: head_dim %d outside (0, %d]", head_dim,
              32 * MAX_PER_LANE);
  TGE_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0, "attention: bad page geometry");
  TGE_REQUIRE(window >= 0, "attention: negative window");
  if (tokens == 0) return 0;
  dim3 grid(tokens, (heads + 3) / 4);
  if (is_bf16)
    attention_simt_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table,
        max_pages, num_pages, page_size, positions, seq_of_token, (__nv_bfloat16*)out, out_stride, heads, kv_heads,
        head_dim, scale, window, status);
  else
    attention_simt_kernel<float><<<grid, 128, 0, stream>>>(
        (const float*)q, q_stride, (const float*)k_pages, (const float*)v_pages, block_table, max_pages, num_pages,
        page_size, positions, seq_of_token, (float*)out, out_stride, heads, kv_heads, head_dim, scale, window, status);
  return tge_launched("attention_simt", 1);
}
