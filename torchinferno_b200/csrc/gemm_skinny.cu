// Projections of a decode step: out[M, N] = x[M, K] . w[N, K]^T for few rows (M <= 64), bf16.
//
// With so few rows the product is a stream of the weights: every byte of w is read once and the
// arithmetic is free.  The reference sends these to cuBLAS (`F.linear`, optionally with
// pre-transposed weights for M <= 64: src/torchinferno/models/llama3/tensor_parallel.py:11176-11239).
// Here a block owns 16 output features (16 rows of w) and its eight warps each stream one eighth of
// K for those rows with 16-byte loads that go straight into tensor-core fragments: the weights are
// the 16-row operand of mma.m16n8k16 and the tokens its 8 columns.  Within a 32-wide k block the
// order of k inside the instruction is permuted (thread t supplies k = 8t .. 8t+7), which a dot
// product does not mind, so no shuffle or shared-memory staging is needed.  The eight partial sums
// meet in shared memory.
#include "common.cuh"

namespace tib {

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kSkinnyWarps = 8;

// NT: n-tiles of 8 tokens (M <= 8 * NT); U: k blocks in flight per thread.
template <int NT, int U, typename TOut>
__global__ void __launch_bounds__(kSkinnyWarps * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, TOut* __restrict__ out,
                   int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo) {
  __shared__ float red[kSkinnyWarps][16][NT * 8 + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, tig = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int blocks = K >> 5;
  const int b_begin = (int)((int64_t)blocks * warp / kSkinnyWarps), b_end = (int)((int64_t)blocks * (warp + 1) / kSkinnyWarps);

  const bool row_lo = n0 + g < N, row_hi = n0 + g + 8 < N;
  const __nv_bfloat16* w_lo = w + (size_t)(row_lo ? n0 + g : 0) * ldw + tig * 8;
  const __nv_bfloat16* w_hi = w + (size_t)(row_hi ? n0 + g + 8 : 0) * ldw + tig * 8;
  const __nv_bfloat16* x_row[NT];
  bool x_ok[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    x_ok[t] = t * 8 + g < M;
    x_row[t] = x + (size_t)(x_ok[t] ? t * 8 + g : 0) * ldx + tig * 8;
  }

  float acc[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[t][j] = 0.f;

  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (int b = b_begin; b < b_end; b += U) {
    uint4 wl[U], wh[U], xv[U][NT];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool in = b + u < b_end;
      const int k = (b + u) << 5;
      wl[u] = (in && row_lo) ? ld_stream16(w_lo + k) : zero;
      wh[u] = (in && row_hi) ? ld_stream16(w_hi + k) : zero;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool in = b + u < b_end;
      const int k = (b + u) << 5;
#pragma unroll
      for (int t = 0; t < NT; ++t)
        xv[u][t] = (in && x_ok[t]) ? __ldg(reinterpret_cast<const uint4*>(x_row[t] + k)) : zero;
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        mma16816(acc[t], wl[u].x, wh[u].x, wl[u].y, wh[u].y, xv[u][t].x, xv[u][t].y);
        mma16816(acc[t], wl[u].z, wh[u].z, wl[u].w, wh[u].w, xv[u][t].z, xv[u][t].w);
      }
  }

  // acc[t][0..1]: feature g, tokens 8t + 2 tig + {0, 1}; acc[t][2..3]: feature g + 8
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    red[warp][g][t * 8 + tig * 2] = acc[t][0];
    red[warp][g][t * 8 + tig * 2 + 1] = acc[t][1];
    red[warp][g + 8][t * 8 + tig * 2] = acc[t][2];
    red[warp][g + 8][t * 8 + tig * 2 + 1] = acc[t][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < M * 16; idx += kSkinnyWarps * 32) {
    const int tok = idx >> 4, f = idx & 15;
    if (n0 + f >= N) continue;
    float sum = 0.f;
#pragma unroll
    for (int wi = 0; wi < kSkinnyWarps; ++wi) sum += red[wi][f][tok];
    out[(size_t)tok * ldo + n0 + f] = from_f32<TOut>(sum);
  }
}

template <int NT, int U>
static int launch_skinny(const void* x, const void* w, void* out, int M, int N, int K, int64_t ldx, int64_t ldw,
                         int64_t ldo, int out_dtype, cudaStream_t stream) {
  const int grid = ceil_div(N, 16);
  if (out_dtype == TIB_BF16)
    gemm_skinny_kernel<NT, U, __nv_bfloat16><<<grid, kSkinnyWarps * 32, 0, stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, N, K, ldx, ldw, ldo);
  else if (out_dtype == TIB_F32)
    gemm_skinny_kernel<NT, U, float><<<grid, kSkinnyWarps * 32, 0, stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (float*)out, M, N, K, ldx, ldw, ldo);
  else
    return TIB_E_DTYPE;
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

}  // namespace tib

using namespace tib;

// Whether tib_gemm_skinny takes this shape: at most 64 rows, K a multiple of 32.
TIB_API int tib_gemm_skinny_supports(int M, int N, int K) {
  return M >= 1 && M <= 64 && N >= 1 && K >= 32 && K % 32 == 0;
}

// x: [M, K] bf16 (row stride ldx), w: [N, K] bf16 (row stride ldw), out: [M, N] bf16 or fp32.
// Rows of x and w must start on 16-byte boundaries.
TIB_API int tib_gemm_skinny(const void* x, const void* w, void* out, int M, int N, int K, int64_t ldx, int64_t ldw,
                            int64_t ldo, int out_dtype, cudaStream_t stream) {
  if (M == 0 || N == 0) return TIB_OK;
  if (!x || !w || !out) return TIB_E_ARG;
  if (!tib_gemm_skinny_supports(M, N, K)) return TIB_E_SIZE;
  if ((((uintptr_t)x | (uintptr_t)w) & 15) || ldx % 8 || ldw % 8) return TIB_E_ALIGN;
  if (M <= 8) return launch_skinny<1, 4>(x, w, out, M, N, K, ldx, ldw, ldo, out_dtype, stream);
  if (M <= 16) return launch_skinny<2, 4>(x, w, out, M, N, K, ldx, ldw, ldo, out_dtype, stream);
  if (M <= 32) return launch_skinny<4, 2>(x, w, out, M, N, K, ldx, ldw, ldo, out_dtype, stream);
  return launch_skinny<8, 1>(x, w, out, M, N, K, ldx, ldw, ldo, out_dtype, stream);
}
