// True 32-bit matrix product on CUDA cores: out[M, N] = x[M, K] . w[N, K]^T.
//
// No tensor cores and no reduced-precision mode: every product and sum is an
// fp32 fused multiply-add.  Each output element is accumulated by one thread
// over k = 0 .. K-1 in rising order, so a row's result does not depend on how
// many other rows are in the call (the projections of the reference are plain
// `F.linear` calls: src/torchinferno/models/llama3/pipeline.py:206-208,245,248-250,400).
// Optionally w and/or x may be bf16 in memory; they are widened on load.
#include "common.cuh"

namespace tib {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TX, typename TW>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const TX* __restrict__ x, const TW* __restrict__ w, float* __restrict__ out, int M,
                int N, int K, int64_t ldx, int64_t ldw, int64_t ldo) {
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each 4 x 4 outputs
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 x 16 elements per tile, 256 threads: 4 elements each.
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int e = tid + it * 256;
      const int r = e >> 4, c = e & 15;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      xs[c][r] = (gm < M && gk < K) ? to_f32(x[(size_t)gm * ldx + gk]) : 0.f;
      ws[c][r] = (gn < N && gk < K) ? to_f32(w[(size_t)gn * ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) out[(size_t)gm * ldo + gn] = acc[i][j];
    }
  }
}

}  // namespace tib

using namespace tib;

// x: [M, K] (row stride ldx), w: [N, K] (row stride ldw), out: [M, N] fp32 (row stride ldo).
TIB_API int tib_gemm_f32(const void* x, const void* w, float* out, int M, int N, int K, int64_t ldx,
                         int64_t ldw, int64_t ldo, int x_dtype, int w_dtype, cudaStream_t stream) {
  if (M == 0 || N == 0) return TIB_OK;
  if (!x || !w || !out || M < 0 || N < 0 || K < 1) return TIB_E_ARG;
  dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
  if (grid.y > 65535) return TIB_E_SIZE;
  if (x_dtype == TIB_F32 && w_dtype == TIB_F32)
    gemm_f32_kernel<float, float><<<grid, 256, 0, stream>>>((const float*)x, (const float*)w, out, M, N, K, ldx, ldw, ldo);
  else if (x_dtype == TIB_F32 && w_dtype == TIB_BF16)
    gemm_f32_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>((const float*)x, (const __nv_bfloat16*)w, out, M, N, K, ldx, ldw, ldo);
  else if (x_dtype == TIB_BF16 && w_dtype == TIB_F32)
    gemm_f32_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (const float*)w, out, M, N, K, ldx, ldw, ldo);
  else if (x_dtype == TIB_BF16 && w_dtype == TIB_BF16)
    gemm_f32_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, out, M, N, K, ldx, ldw, ldo);
  else
    return TIB_E_DTYPE;
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}
