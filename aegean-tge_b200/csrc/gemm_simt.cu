// Matrix product on the CUDA cores with float32 accumulation: out = x . w^T (+ epilogue).
//
// This is the whole float32 path's product (plain FFMA, no reduced-precision
// matrix mode) and the fallback of the bfloat16 path for shapes the tensor-core
// kernel refuses.  Every output element is accumulated over k in ascending
// order by one thread, so its value depends on neither the tile it falls in
// nor on what else is in the batch.  The formula is the reference's
// row-times-vector product (src/tensor/reference.cpp:29-45) followed by the
// separate bias loop (src/models/qwen2.cpp:2062-2068), SiLU gate
// (src/cpu/scalar/norm_rope_scalar.cpp:43-51) or residual add
// (src/models/qwen2.cpp:2101-2103).
#include "common.cuh"

enum GemmEpilogue : int {
  GEMM_STORE = 0,      // out[m, n] = acc + bias[n], run dtype
  GEMM_STORE_F32 = 1,  // out[m, n] = acc + bias[n], float32
  GEMM_ADD_F32 = 2,    // residual[m, n] += acc + bias[n], float32 in place
  GEMM_SWIGLU = 3,     // w rows interleaved (gate_i, up_i): out[m, i] = silu(g) * u, run dtype
};

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T>
__device__ __forceinline__ void load4(const T* base, size_t row_stride, int row, int rows, int k, int K, bool vec,
                                      float out[4]);

template <>
__device__ __forceinline__ void load4<float>(const float* base, size_t row_stride, int row, int rows, int k, int K,
                                             bool vec, float out[4]) {
  if (row < rows && vec && k + 3 < K) {
    const float4 v = *reinterpret_cast<const float4*>(base + (size_t)row * row_stride + k);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    return;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = (row < rows && k + i < K) ? base[(size_t)row * row_stride + k + i] : 0.0f;
}

template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* base, size_t row_stride, int row, int rows,
                                                     int k, int K, bool vec, float out[4]) {
  if (row < rows && vec && k + 3 < K) {
    const uint2 raw = *reinterpret_cast<const uint2*>(base + (size_t)row * row_stride + k);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    out[0] = __low2float(a); out[1] = __high2float(a); out[2] = __low2float(b); out[3] = __high2float(b);
    return;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    out[i] = (row < rows && k + i < K) ? __bfloat162float(base[(size_t)row * row_stride + k + i]) : 0.0f;
}

template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const T* __restrict__ x, size_t ldx, const T* __restrict__ w,
                                                        size_t ldw, const float* __restrict__ bias, void* out,
                                                        size_t ldo, int M, int N, int K, int epilogue, int vec) {
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int load_row = tid >> 2, load_k = (tid & 3) * 4;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    float xv[4], wv[4];
    load4<T>(x, ldx, m0 + load_row, M, k0 + load_k, K, vec != 0, xv);
    load4<T>(w, ldw, n0 + load_row, N, k0 + load_k, K, vec != 0, wv);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      xs[load_k + i][load_row] = xv[i];
      ws[load_k + i][load_row] = wv[i];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
    if (epilogue == GEMM_SWIGLU) {
#pragma unroll
      for (int j = 0; j < TN; j += 2) {
        const int n = n0 + tx * TN + j;
        if (n + 1 >= N) continue;
        float g = acc[i][j], u = acc[i][j + 1];
        if (bias) { g += bias[n]; u += bias[n + 1]; }
        const float a = g / (1.0f + expf(-g)) * u;
        reinterpret_cast<T*>(out)[(size_t)m * ldo + (n >> 1)] = from_float<T>(a);
      }
      continue;
    }
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      if (epilogue == GEMM_STORE) {
        reinterpret_cast<T*>(out)[(size_t)m * ldo + n] = from_float<T>(v);
      } else if (epilogue == GEMM_STORE_F32) {
        reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = v;
      } else {
        reinterpret_cast<float*>(out)[(size_t)m * ldo + n] += v;
      }
    }
  }
}

}  // namespace

// x [M, K] (row stride ldx), w [N, K] (row stride ldw), both in the run dtype;
// bias float32 [N] or null; out as the epilogue says (row stride ldo, in elements).
TGE_API int tge_gemm_simt(const void* x, long long ldx, const void* w, long long ldw, const float* bias, void* out,
                          long long ldo, int M, int N, int K, int is_bf16, int epilogue, cudaStream_t stream) {
  TGE_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
  TGE_REQUIRE(epilogue >= GEMM_STORE && epilogue <= GEMM_SWIGLU, "gemm: unknown epilogue %d", epilogue);
  TGE_REQUIRE(epilogue != GEMM_SWIGLU || N % 2 == 0, "gemm: the gated epilogue needs an even number of weight rows, got %d", N);
  TGE_REQUIRE(ldx >= K && ldw >= K, "gemm: row strides %lld/%lld shorter than K=%d", ldx, ldw, K);
  if (M == 0) return 0;
  const size_t elem = is_bf16 ? 2 : 4;
  const size_t align = is_bf16 ? 8 : 16;
  const int vec = (K % 4 == 0) && ((ldx * elem) % align == 0) && ((ldw * elem) % align == 0) &&
                  ((uintptr_t)x % align == 0) && ((uintptr_t)w % align == 0);
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (is_bf16)
    gemm_simt_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (size_t)ldx,
                                                              (const __nv_bfloat16*)w, (size_t)ldw, bias, out,
                                                              (size_t)ldo, M, N, K, epilogue, vec);
  else
    gemm_simt_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, (size_t)ldx, (const float*)w, (size_t)ldw,
                                                      bias, out, (size_t)ldo, M, N, K, epilogue, vec);
  return tge_launched("gemm_simt", 1);
}
