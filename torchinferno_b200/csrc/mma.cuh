// Pieces shared by the mma.sync attention kernels: cp.async, ldmatrix, the bf16 MMA, the streaming-softmax
// step on MMA fragments, and the kernel that merges the partial results of a split context.
#pragma once

#include "common.cuh"
#include <math_constants.h>

namespace tib {

// ----------------------------------------------------------------- PTX bits
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are zero-filled, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One step of the streaming softmax for a warp's 16 rows over NT n-tiles of 8 keys: scores s are
// already scaled and masked (-inf).  Updates m, l (per-thread partial sums), rescales o and
// returns the probabilities packed as the A fragments of the P.V product (one per 16 keys).
template <int NT, int ONT>
__device__ __forceinline__ void softmax_step(float (&s)[NT][4], float (&m)[2], float (&l)[2], float (&o)[ONT][4],
                                             uint32_t (&p)[NT / 2][4]) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {  // h = 0: row g, h = 1: row g + 8
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * h], s[nt][2 * h + 1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m[h], mx);
    const float base = m_new == -CUDART_INF_F ? 0.f : m_new;
    const float alpha = exp2f(m[h] - base);
    m[h] = m_new;
    float sum = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      s[nt][2 * h] = exp2f(s[nt][2 * h] - base);
      s[nt][2 * h + 1] = exp2f(s[nt][2 * h + 1] - base);
      sum += s[nt][2 * h] + s[nt][2 * h + 1];
    }
    l[h] = l[h] * alpha + sum;
    if (__any_sync(0xffffffffu, alpha != 1.f)) {  // once the running max has settled nothing is rescaled
#pragma unroll
      for (int n = 0; n < ONT; ++n) {
        o[n][2 * h] *= alpha;
        o[n][2 * h + 1] *= alpha;
      }
    }
  }
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    p[kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    p[kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    p[kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    p[kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
  }
}

// grid: (heads, n_entries), D threads.  The weights of the parts are computed first (one load per part,
// all in flight together), then every thread sums its output element with several loads in flight.
template <int D>
__global__ void __launch_bounds__(D)
decode_merge_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                    __nv_bfloat16* __restrict__ out, const int* __restrict__ q_start, int heads, int num_splits,
                    int head_dim) {
  // (D threads; head_dim <= D is the width of a head in memory)
  pdl_wait();   // (returns at once when the launch was an ordinary one)
  pdl_trigger();
  extern __shared__ float merge_w[];     // [num_splits] weights, then 1 / sum
  const int entry = blockIdx.y, head = blockIdx.x;
  const int row0 = q_start[entry];
  if (q_start[entry + 1] - row0 != 1) return;
  const size_t base_slot = ((size_t)entry * heads + head) * num_splits;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float mm = -CUDART_INF_F;
    for (int s = lane; s < num_splits; s += 32) mm = fmaxf(mm, partial_ml[(base_slot + s) * 2]);
    mm = warp_max(mm);
    float sum = 0.f;
    for (int s = lane; s < num_splits; s += 32) {
      const float ms = partial_ml[(base_slot + s) * 2];
      const float w = ms == -CUDART_INF_F ? 0.f : exp2f(ms - mm);   // an empty part wrote no output
      merge_w[s] = w;
      sum += w == 0.f ? 0.f : w * partial_ml[(base_slot + s) * 2 + 1];
    }
    sum = warp_sum(sum);
    if (lane == 0) merge_w[num_splits] = 1.f / sum;
  }
  __syncthreads();
  if ((int)threadIdx.x >= head_dim) return;
  const float* po = partial_o + base_slot * head_dim + threadIdx.x;
  float acc = 0.f;
#pragma unroll 8
  for (int s = 0; s < num_splits; ++s) {
    const float w = merge_w[s];
    acc += w == 0.f ? 0.f : w * po[(size_t)s * head_dim];
  }
  out[((size_t)row0 * heads + head) * head_dim + threadIdx.x] = __float2bfloat16_rn(acc * merge_w[num_splits]);
}

}  // namespace tib
