// Embedding lookup, RMSNorm (plain and fused with the residual add), SwiGLU and casts.
//
// The residual stream is held in 32-bit whatever the activation type: the
// embedding writes it, every fused add+norm updates it in place, and the
// normalised rows leave in the activation type T (float or bf16).
//
// Formulas (file:line in the reference project):
//   RMSNorm      y = x * rsqrt(mean(x^2) + eps) * w, all in fp32
//                src/torchinferno/kernels/triton_ops.py:2044-2048
//   add + norm   h = x + residual (fp32), n = rmsnorm(h)
//                src/torchinferno/kernels/triton_ops.py:2088-2096
//   SwiGLU       gate / (1 + exp(-gate)) * up, gate in fp32
//                src/torchinferno/kernels/triton_ops.py:29-32
#include "common.cuh"

namespace tib {

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const int id = ids[row];
  float* dst = out + (size_t)row * hidden;
  if (id < 0 || id >= vocab) {  // an id outside the table must show, not alias a row
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = __int_as_float(0x7fc00000);
    return;
  }
  const T* src = table + (size_t)id * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = to_f32(src[c]);
}

// bf16 table, width a multiple of 8: eight elements a thread and pass (one 16-byte load, two 16-byte stores), so that
// a row of a few thousand columns is one or two passes of a block and not sixteen (7.6 -> about 2 us for the eight
// rows of a decode step, which is all latency).
__global__ void embedding_bf16x8_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                        float* __restrict__ out, int hidden, int vocab) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const int id = ids[row];
  float* dst = out + (size_t)row * hidden;
  const bool known = id >= 0 && id < vocab;        // an id outside the table must show, not alias a row
  const __nv_bfloat16* src = table + (size_t)(known ? id : 0) * hidden;
  const float nan = __int_as_float(0x7fc00000);
  for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
    float4 lo = make_float4(nan, nan, nan, nan), hi = lo;
    if (known) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + c);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float2 a = bf16x2_floats(p[0]), b = bf16x2_floats(p[1]), e = bf16x2_floats(p[2]), f = bf16x2_floats(p[3]);
      lo = make_float4(a.x, a.y, b.x, b.y);
      hi = make_float4(e.x, e.y, f.x, f.y);
    }
    *reinterpret_cast<float4*>(dst + c) = lo;
    *reinterpret_cast<float4*>(dst + c + 4) = hi;
  }
}

// ------------------------------------------------------------------ RMSNorm
// One block per output row.  delta == nullptr: plain norm of residual[row].
// rows != nullptr: output row i reads source row rows[i] and the residual is
// left untouched (used to norm only the rows whose logits are wanted).
template <typename T>
__global__ void add_rmsnorm_kernel(const T* __restrict__ delta, float* __restrict__ residual,
                                   const int* __restrict__ rows, const float* __restrict__ weight,
                                   T* __restrict__ out, int hidden, float eps) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[33];
  const int orow = blockIdx.x;
  const int srow = rows ? rows[orow] : orow;
  float* res = residual + (size_t)srow * hidden;
  const T* dl = delta ? delta + (size_t)srow * hidden : nullptr;
  const bool write_back = (delta != nullptr) && (rows == nullptr);
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float h = res[c];
    if (dl) h += to_f32(dl[c]);
    if (write_back) res[c] = h;
    ss += h * h;
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)hidden + eps);
  T* dst = out + (size_t)orow * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float h = res[c];
    if (dl && !write_back) h += to_f32(dl[c]);
    dst[c] = from_f32<T>(h * inv * weight[c]);
  }
}

// bf16 rows whose width is a multiple of 8 and at most 8 * 1024: every thread keeps its eight
// elements in registers, so the row is read once (16-byte loads) and written once.
__global__ void __launch_bounds__(1024)
add_rmsnorm_bf16x8_kernel(const __nv_bfloat16* __restrict__ delta, float* __restrict__ residual,
                          const int* __restrict__ rows, const float* __restrict__ weight,
                          __nv_bfloat16* __restrict__ out, int hidden, float eps) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[33];
  const int orow = blockIdx.x;
  const int srow = rows ? rows[orow] : orow;
  const int c = threadIdx.x * 8;
  const bool active = c < hidden;
  const bool write_back = (delta != nullptr) && (rows == nullptr);
  float h[8];
  float ss = 0.f;
  if (active) {
    float* res = residual + (size_t)srow * hidden + c;
    const float4 r0 = *reinterpret_cast<const float4*>(res), r1 = *reinterpret_cast<const float4*>(res + 4);
    h[0] = r0.x; h[1] = r0.y; h[2] = r0.z; h[3] = r0.w; h[4] = r1.x; h[5] = r1.y; h[6] = r1.z; h[7] = r1.w;
    if (delta) {
      const uint4 raw = *reinterpret_cast<const uint4*>(delta + (size_t)srow * hidden + c);
      const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = bf16x2_floats(d2[i]);
        h[2 * i] += f.x;
        h[2 * i + 1] += f.y;
      }
    }
    if (write_back) {
      *reinterpret_cast<float4*>(res) = make_float4(h[0], h[1], h[2], h[3]);
      *reinterpret_cast<float4*>(res + 4) = make_float4(h[4], h[5], h[6], h[7]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += h[i] * h[i];
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)hidden + eps);
  if (active) {
    const float4 w0 = *reinterpret_cast<const float4*>(weight + c), w1 = *reinterpret_cast<const float4*>(weight + c + 4);
    const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    uint4 packed;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(h[2 * i] * inv * w[2 * i], h[2 * i + 1] * inv * w[2 * i + 1]);
    *reinterpret_cast<uint4*>(out + (size_t)orow * hidden + c) = packed;
  }
}

// Plain RMSNorm of rows held in type T (for parts that norm something other
// than the residual stream, e.g. per-head norms).
template <typename T>
__global__ void rmsnorm_t_kernel(const T* __restrict__ x, const float* __restrict__ weight,
                                 T* __restrict__ out, int hidden, float eps) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[33];
  const T* src = x + (size_t)blockIdx.x * hidden;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float h = to_f32(src[c]);
    ss += h * h;
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)hidden + eps);
  T* dst = out + (size_t)blockIdx.x * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x)
    dst[c] = from_f32<T>(to_f32(src[c]) * inv * weight[c]);
}

// ------------------------------------------------------------------- SwiGLU
// gate_up rows hold either all gates, then all ups (interleaved 0), or gate i and up i side by side (interleaved 1:
// the layout in which one tile of a fused gate/up product holds both).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter,
                              int64_t total, int interleaved) {
  pdl_wait();
  pdl_trigger();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / inter;
    const int col = (int)(i - row * inter);
    const T* src = gate_up + row * 2 * (int64_t)inter;
    const float g = to_f32(interleaved ? src[2 * col] : src[col]);
    const float u = to_f32(interleaved ? src[2 * col + 1] : src[inter + col]);
    out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
  }
}

// x * sigmoid(x) with the fast exponential and reciprocal (a few ulp of fp32: far below the bf16 rounding of
// the result); the exact functions cost more instructions than the kernel has time for beside its loads.
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.f + __expf(-x)); }

// bf16, intermediate width a multiple of 8: 16-byte loads and stores.
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                     int inter, int64_t total_vec, int interleaved) {
  pdl_wait();
  pdl_trigger();
  const int per_row = inter >> 3;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / per_row;
    const int col = (int)(i - row * per_row) << 3;
    const __nv_bfloat16* src = gate_up + row * 2 * (int64_t)inter + (interleaved ? 2 * col : col);
    // eight (gate, up) pairs: two vectors of gates and of ups, or two vectors of pairs
    const uint4 a = *reinterpret_cast<const uint4*>(src), b = *reinterpret_cast<const uint4*>(src + (interleaved ? 8 : inter));
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
    uint4 packed;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
    if (interleaved) {
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const float2 p0 = bf16x2_floats(a2[2 * k]), p1 = bf16x2_floats(a2[2 * k + 1]);
        const float2 q0 = bf16x2_floats(b2[2 * k]), q1 = bf16x2_floats(b2[2 * k + 1]);
        o2[k] = __floats2bfloat162_rn(silu_fast(p0.x) * p0.y, silu_fast(p1.x) * p1.y);
        o2[2 + k] = __floats2bfloat162_rn(silu_fast(q0.x) * q0.y, silu_fast(q1.x) * q1.y);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 g = bf16x2_floats(a2[k]), u = bf16x2_floats(b2[k]);
        o2[k] = __floats2bfloat162_rn(silu_fast(g.x) * u.x, silu_fast(g.y) * u.y);
      }
    }
    *reinterpret_cast<uint4*>(out + row * (int64_t)inter + col) = packed;
  }
}

template <typename A, typename B>
__global__ void cast_kernel(const A* __restrict__ in, B* __restrict__ out, int64_t total) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x)
    out[i] = from_f32<B>(to_f32(in[i]));
}

__global__ void scatter_i32_kernel(int* __restrict__ dst, const int* __restrict__ index,
                                   const int* __restrict__ value, int n, int64_t dst_size) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const int64_t at = index[i];
    if (at >= 0 && at < dst_size) dst[at] = value[i];
  }
}

__global__ void decode_inputs_kernel(int* __restrict__ records, const int* __restrict__ slots, int max_slots,
                                     int* __restrict__ token_ids, int* __restrict__ positions, int n) {
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const int slot = slots[i];
    if (slot < 0 || slot >= max_slots) {       // (the embedding then writes NaN: it must show)
      token_ids[i] = -1;
      positions[i] = 0;
      return;
    }
    int* record = records + (size_t)slot * TIB_REC_WORDS;
    const int length = record[TIB_REC_LENGTH];
    token_ids[i] = record[TIB_REC_LAST_TOKEN];
    positions[i] = length;
    record[TIB_REC_LENGTH] = length + 1;
  }
}

static inline int norm_threads(int hidden) {
  int t = ((hidden + 3) / 4 + 31) / 32 * 32;  // about four elements a thread
  if (t < 32) t = 32;
  if (t > 1024) t = 1024;
  return t;
}

}  // namespace tib

using namespace tib;

TIB_API int tib_embedding(const int* ids, const void* table, float* out, int n_tokens, int hidden,
                          int vocab, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return TIB_OK;
  if (!ids || !table || !out || n_tokens < 0 || hidden < 1 || vocab < 1) return TIB_E_ARG;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == TIB_F32)
    TIB_LAUNCH_DEPENDENT(embedding_kernel<float>, n_tokens, threads, 0, stream, ids, (const float*)table, out, hidden, vocab);
  else if (dtype == TIB_BF16 && hidden % 8 == 0 && (((uintptr_t)table | (uintptr_t)out) & 15) == 0)
    TIB_LAUNCH_DEPENDENT(embedding_bf16x8_kernel, n_tokens, hidden >= 4096 ? 512 : hidden >= 1024 ? 128 : 64, 0, stream, ids,
                         (const __nv_bfloat16*)table, out, hidden, vocab);
  else if (dtype == TIB_BF16)
    TIB_LAUNCH_DEPENDENT(embedding_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, ids, (const __nv_bfloat16*)table, out, hidden, vocab);
  else
    return TIB_E_DTYPE;
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

// delta may be null (plain norm of the residual); rows may be null (all rows in order).
TIB_API int tib_add_rmsnorm(const void* delta, float* residual, const int* rows, const float* weight,
                            void* out, int n_out, int hidden, float eps, int dtype,
                            cudaStream_t stream) {
  if (n_out == 0) return TIB_OK;
  if (!residual || !weight || !out || n_out < 0 || hidden < 1) return TIB_E_ARG;
  const int threads = norm_threads(hidden);
  if (dtype == TIB_F32)
    TIB_LAUNCH_DEPENDENT(add_rmsnorm_kernel<float>, n_out, threads, 0, stream, (const float*)delta, residual, rows, weight, (float*)out, hidden, eps);
  else if (dtype == TIB_BF16 && hidden % 8 == 0 && hidden <= 8192 &&
           (((uintptr_t)residual | (uintptr_t)weight | (uintptr_t)out | (uintptr_t)delta) & 15) == 0) {
    const int vec_threads = ((hidden / 8) + 31) / 32 * 32;
    TIB_LAUNCH_DEPENDENT(add_rmsnorm_bf16x8_kernel, n_out, vec_threads, 0, stream, (const __nv_bfloat16*)delta, residual, rows, weight, (__nv_bfloat16*)out, hidden, eps);
  } else if (dtype == TIB_BF16)
    TIB_LAUNCH_DEPENDENT(add_rmsnorm_kernel<__nv_bfloat16>, n_out, threads, 0, stream, (const __nv_bfloat16*)delta, residual, rows, weight, (__nv_bfloat16*)out, hidden, eps);
  else
    return TIB_E_DTYPE;
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

TIB_API int tib_rmsnorm(const void* x, const float* weight, void* out, int n_rows, int hidden,
                        float eps, int dtype, cudaStream_t stream) {
  if (n_rows == 0) return TIB_OK;
  if (!x || !weight || !out || n_rows < 0 || hidden < 1) return TIB_E_ARG;
  const int threads = norm_threads(hidden);
  if (dtype == TIB_F32)
    TIB_LAUNCH_DEPENDENT(rmsnorm_t_kernel<float>, n_rows, threads, 0, stream, (const float*)x, weight, (float*)out, hidden, eps);
  else if (dtype == TIB_BF16)
    TIB_LAUNCH_DEPENDENT(rmsnorm_t_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, (const __nv_bfloat16*)x, weight, (__nv_bfloat16*)out, hidden, eps);
  else
    return TIB_E_DTYPE;
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

TIB_API int tib_swiglu(const void* gate_up, void* out, int n_rows, int inter, int dtype, int interleaved,
                       cudaStream_t stream) {
  const int64_t total = (int64_t)n_rows * inter;
  if (total == 0) return TIB_OK;
  if (!gate_up || !out || n_rows < 0 || inter < 1) return TIB_E_ARG;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == TIB_F32)
    TIB_LAUNCH_DEPENDENT(swiglu_kernel<float>, blocks, threads, 0, stream, (const float*)gate_up, (float*)out, inter, total, interleaved);
  else if (dtype == TIB_BF16 && inter % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
    const int64_t vec = total / 8, want_v = (vec + threads - 1) / threads;
    TIB_LAUNCH_DEPENDENT(swiglu_bf16x8_kernel, (int)(want_v < 148 * 16 ? want_v : 148 * 16), threads, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, vec, interleaved);
  } else if (dtype == TIB_BF16)
    TIB_LAUNCH_DEPENDENT(swiglu_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total, interleaved);
  else
    return TIB_E_DTYPE;
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

// Cast between float and bf16: in_dtype -> out_dtype.
TIB_API int tib_cast(const void* in, void* out, int64_t total, int in_dtype, int out_dtype,
                     cudaStream_t stream) {
  if (total == 0) return TIB_OK;
  if (!in || !out || total < 0) return TIB_E_ARG;
  const int threads = 256;
  const int64_t want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (in_dtype == TIB_BF16 && out_dtype == TIB_F32)
    cast_kernel<__nv_bfloat16, float><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)in, (float*)out, total);
  else if (in_dtype == TIB_F32 && out_dtype == TIB_BF16)
    cast_kernel<float, __nv_bfloat16><<<blocks, threads, 0, stream>>>((const float*)in, (__nv_bfloat16*)out, total);
  else
    return TIB_E_DTYPE;
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

// dst[index[i]] = value[i] for i < n; indices outside [0, dst_size) are skipped.
// Used to apply queued block-table changes in one launch.
TIB_API int tib_scatter_i32(int* dst, const int* index, const int* value, int n, int64_t dst_size,
                            cudaStream_t stream) {
  if (n == 0) return TIB_OK;
  if (!dst || !index || !value || n < 0) return TIB_E_ARG;
  scatter_i32_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(dst, index, value, n, dst_size);
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

// The inputs of a decode step from the requests' own records (common.cuh: TibRequestRecord): request i of the step
// sits in slot slots[i]; its next token and its position are read from its record, and the record moves one
// position on.  A request appears at most once in slots.
TIB_API int tib_decode_inputs(int* records, const int* slots, int max_slots, int* token_ids, int* positions, int n,
                              cudaStream_t stream) {
  if (n == 0) return TIB_OK;
  if (!records || !slots || !token_ids || !positions || n < 0 || max_slots < 1) return TIB_E_ARG;
  TIB_LAUNCH_DEPENDENT(decode_inputs_kernel, ceil_div(n, 128), 128, 0, stream, records, slots, max_slots, token_ids, positions, n);
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

// Programmatic dependent launch of this library's small kernels on (1, the default) or off (0);
// returns the setting before.  Off, every kernel starts only when the one before it has ended.
TIB_API int tib_set_dependent_launch(int on) {
  const int before = tib::dependent_launch_flag();
  tib::dependent_launch_flag() = on ? 1 : 0;
  return before;
}
