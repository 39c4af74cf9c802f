// Next-token choice on the device: greedy argmax and temperature sampling.
//
// Greedy: the lowest index among the maxima, as torch.argmax
// (src/torchinferno/runtime/sampling.py:7-9); a NaN counts as the largest value
// (src/torchinferno/kernels/triton_ops.py:72-119 propagates NaN likewise).
// Temperature: the Gumbel-max form argmax(logits / T - log(-log u)), which draws
// from softmax(logits / T) (src/torchinferno/models/llama3/tensor_parallel.py:9946-9996).
// The uniform u comes from Philox4x32-10 keyed by the request's seed with the
// counter (vocab index / 4, position of the token being drawn), so the token
// drawn for a request at a position does not depend on what else is in the batch.
#include "common.cuh"
#include <math_constants.h>

namespace tib {

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

__device__ __forceinline__ uint32_t philox_u32(uint64_t seed, uint32_t position, uint32_t index) {
  uint32_t c[4] = {index >> 2, position, 0u, 0u};
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c[index & 3];
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  // NaN beats everything; among equals the lower index wins.
  const bool vn = v != v, bn = bv != bv;
  if (vn != bn) return vn;
  if (vn) return i < bi;
  return v > bv || (v == bv && i < bi);
}

__global__ void __launch_bounds__(1024)
sample_kernel(const float* __restrict__ logits, int64_t row_stride, const float* __restrict__ temperature,
              const int64_t* __restrict__ seeds, const int* __restrict__ positions,
              int* __restrict__ out, int vocab, int* __restrict__ records, const int* __restrict__ record_slots,
              int max_slots, int* __restrict__ history) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sv[32];
  __shared__ int si[32];
  const int row = blockIdx.x;
  const float* lg = logits + (size_t)row * row_stride;
  float temp = temperature ? temperature[row] : 0.f;
  uint64_t seed = seeds ? (uint64_t)seeds[row] : 0ull;
  uint32_t pos = positions ? (uint32_t)positions[row] : 0u;
  int* record = nullptr;
  if (records) {
    // parameters from the request's own record: its length after this step is the position of the token drawn now
    const int slot = record_slots[row];
    if (slot >= 0 && slot < max_slots) {
      record = records + (size_t)slot * TIB_REC_WORDS;
      temp = __int_as_float(record[TIB_REC_TEMPERATURE]);
      seed = ((uint64_t)(uint32_t)record[TIB_REC_SEED_HI] << 32) | (uint32_t)record[TIB_REC_SEED_LO];
      pos = (uint32_t)record[TIB_REC_LENGTH];
    }
  }
  const bool greedy = !(temp > 0.f);
  float bv = -CUDART_INF_F;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = lg[i];
    if (!greedy) {
      const uint32_t r = philox_u32(seed, pos, (uint32_t)i);
      const float u = ((float)(r >> 8) + 0.5f) * (1.0f / 16777216.0f);  // in (0, 1)
      v = v / temp - logf(-logf(u));
    }
    if (better(v, i, bv, bi)) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    bv = lane < nw ? sv[lane] : -CUDART_INF_F;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) {
      out[row] = bi;
      if (history) history[row] = bi;
      if (record) {
        record[TIB_REC_LAST_TOKEN] = bi;
        record[TIB_REC_DRAWN] += 1;
      }
    }
  }
}

}  // namespace tib

using namespace tib;

// logits: [n_rows, vocab] fp32 (row stride in elements); temperature, seeds, positions: [n_rows]
// or null (null temperature: greedy for every row).  out: [n_rows] token ids.
TIB_API int tib_sample(const float* logits, int64_t row_stride, const float* temperature,
                       const int64_t* seeds, const int* positions, int* out, int n_rows, int vocab,
                       cudaStream_t stream) {
  if (n_rows == 0) return TIB_OK;
  if (!logits || !out || n_rows < 0 || vocab < 1) return TIB_E_ARG;
  int threads = 1024;
  while (threads > 32 && threads / 2 >= vocab) threads /= 2;
  TIB_LAUNCH_DEPENDENT(sample_kernel, n_rows, threads, 0, stream, logits, row_stride, temperature, seeds, positions, out, vocab,
                       (int*)nullptr, (const int*)nullptr, 0, (int*)nullptr);
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

// The same with every row's parameters taken from its request's record (common.cuh: TibRequestRecord):
// records [max_slots][TIB_REC_WORDS], record_slots [n_rows] the slot of each row's request.  The drawn token is
// written to out[row], to the record (next input token; count of drawn tokens) and, when given, to history[row].
// A slot outside the table is drawn greedily and writes no record.
TIB_API int tib_sample_records(const float* logits, int64_t row_stride, int* records, const int* record_slots, int max_slots,
                               int* out, int* history, int n_rows, int vocab, cudaStream_t stream) {
  if (n_rows == 0) return TIB_OK;
  if (!logits || !out || !records || !record_slots || n_rows < 0 || vocab < 1 || max_slots < 1) return TIB_E_ARG;
  int threads = 1024;
  while (threads > 32 && threads / 2 >= vocab) threads /= 2;
  TIB_LAUNCH_DEPENDENT(sample_kernel, n_rows, threads, 0, stream, logits, row_stride, (const float*)nullptr,
                       (const int64_t*)nullptr, (const int*)nullptr, out, vocab, records, record_slots, max_slots, history);
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}
