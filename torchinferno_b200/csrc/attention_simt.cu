// Paged causal attention on CUDA cores, for any head size, group size, page
// size and window.  It serves the 32-bit path of the engine and every shape the
// tensor-core kernels refuse.
//
// Formula (src/torchinferno/models/llama3/raw_ops.py:44-51): s = (q . k) / sqrt(d)
// (the scale is an argument), a key is allowed iff key_pos <= query_pos (and,
// with a window w > 0, query_pos - key_pos < w), p = softmax(s) in fp32, o = p . v.
// Streaming form with running max / sum / accumulator as in
// src/torchinferno/kernels/triton_ops.py:2555-2574.
//
// Exactness: one warp owns one (query token, query head) row from start to end.
// It walks the keys in blocks of 32 that are aligned to absolute positions
// (block b = keys 32b .. 32b+31), in rising order, so the arithmetic of a row
// depends only on its own position and keys, never on how the batch was cut,
// which other rows share the block, or which pages hold the keys.
#include "common.cuh"
#include <math_constants.h>

namespace tib {

constexpr int kAttnWarps = 4;
constexpr int kAttnRowsPerWarp = 4;
constexpr int kAttnRows = kAttnWarps * kAttnRowsPerWarp;  // rows (token, head) per block
constexpr int kAttnKeys = 32;                              // keys per step = lanes

struct AttnArgs {
  const int* q_start;      // [n_entries + 1] first token row of each entry
  const int* kv_start;     // [n_entries] position of the entry's first query token
  const int* slots;        // [n_entries] row of the block table
  const int* block_table;  // [slots, table_stride]
  int table_stride;
  int heads, kv_heads, head_dim;
  int page_size;
  int64_t page_stride;     // elements between pages of this layer
  int num_pages;
  int window;              // 0: all earlier keys
  float scale;
  int group_chunk;         // query heads of one kv head handled by one block
  int q_tile;              // query tokens per block
  int* error_word;
};

template <typename T, int DPL>
__global__ void __launch_bounds__(kAttnWarps * 32)
paged_attention_simt_kernel(const T* __restrict__ q, const T* __restrict__ pool,
                            T* __restrict__ out, AttnArgs a) {
  extern __shared__ float smem[];
  const int d = a.head_dim;
  float* q_s = smem;                           // [kAttnRows][d]
  float* k_s = q_s + kAttnRows * d;            // [32][d + 1]
  float* v_s = k_s + kAttnKeys * (d + 1);      // [32][d]

  const int entry = blockIdx.y;
  const int group = a.heads / a.kv_heads;
  const int chunks = (group + a.group_chunk - 1) / a.group_chunk;
  const int kvh = blockIdx.z / chunks;
  const int g0 = (blockIdx.z - kvh * chunks) * a.group_chunk;
  const int gc = min(a.group_chunk, group - g0);

  const int row0 = a.q_start[entry];
  const int q_len = a.q_start[entry + 1] - row0;
  const int t0 = blockIdx.x * a.q_tile;
  if (t0 >= q_len) return;
  const int nt = min(a.q_tile, q_len - t0);
  const int nrows = nt * gc;
  const int pos0 = a.kv_start[entry] + t0;     // position of the first query of the tile
  const int last_pos = pos0 + nt - 1;          // highest key any row may read
  const int* table = a.block_table + (size_t)a.slots[entry] * a.table_stride;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q_width = a.heads * d;

  // Stage the queries (fp32).
  for (int e = threadIdx.x; e < nrows * d; e += blockDim.x) {
    const int r = e / d, dd = e - r * d;
    const int t = r / gc, g = r - t * gc;
    q_s[r * d + dd] = to_f32(q[(size_t)(row0 + t0 + t) * q_width + (kvh * group + g0 + g) * d + dd]);
  }

  float m[kAttnRowsPerWarp], l[kAttnRowsPerWarp], acc[kAttnRowsPerWarp][DPL];
#pragma unroll
  for (int i = 0; i < kAttnRowsPerWarp; ++i) {
    m[i] = -CUDART_INF_F;
    l[i] = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) acc[i][j] = 0.f;
  }

  int first_key = 0;
  if (a.window > 0) first_key = max(0, pos0 - a.window + 1);
  const int b_lo = first_key / kAttnKeys, b_hi = last_pos / kAttnKeys;

  for (int b = b_lo; b <= b_hi; ++b) {
    __syncthreads();  // previous block's tiles are no longer read (and q_s is written)
    // Stage keys and values of block b.  Keys past last_pos are not yet written
    // (or belong to nobody): they are filled with zeros and always masked.
    for (int e = threadIdx.x; e < kAttnKeys * d; e += blockDim.x) {
      const int j = e / d, dd = e - j * d;
      const int kp = b * kAttnKeys + j;
      float kval = 0.f, vval = 0.f;
      if (kp <= last_pos && kp >= first_key) {
        const int page = table[kp / a.page_size];
        if (page >= 0 && page < a.num_pages) {
          const T* kpage = pool + (size_t)page * a.page_stride;
          const size_t off = ((size_t)kvh * a.page_size + (kp % a.page_size)) * d + dd;
          kval = to_f32(kpage[off]);
          vval = to_f32(kpage[(size_t)a.kv_heads * a.page_size * d + off]);
        } else if (a.error_word) {
          atomicExch(a.error_word, 0x10000 + entry);
        }
      }
      k_s[j * (d + 1) + dd] = kval;
      v_s[j * d + dd] = vval;
    }
    __syncthreads();

#pragma unroll
    for (int i = 0; i < kAttnRowsPerWarp; ++i) {
      const int r = warp * kAttnRowsPerWarp + i;
      if (r >= nrows) continue;                       // uniform in the warp
      const int qpos = pos0 + r / gc;
      const int lo = a.window > 0 ? max(0, qpos - a.window + 1) : 0;
      if (b * kAttnKeys > qpos || b * kAttnKeys + kAttnKeys - 1 < lo) continue;  // nothing allowed
      const int kp = b * kAttnKeys + lane;
      const bool allowed = kp <= qpos && kp >= lo;
      float s = 0.f;
      const float* qr = q_s + r * d;
      const float* kr = k_s + lane * (d + 1);
      for (int dd = 0; dd < d; ++dd) s = fmaf(qr[dd], kr[dd], s);
      s = allowed ? s * a.scale : -CUDART_INF_F;
      const float m_new = fmaxf(m[i], warp_max(s));   // finite: the block holds an allowed key
      const float alpha = m[i] == -CUDART_INF_F ? 0.f : expf(m[i] - m_new);
      const float p = allowed ? expf(s - m_new) : 0.f;
      l[i] = l[i] * alpha + warp_sum(p);
      m[i] = m_new;
#pragma unroll
      for (int j = 0; j < DPL; ++j) acc[i][j] *= alpha;
      for (int kk = 0; kk < kAttnKeys; ++kk) {
        const float pk = __shfl_sync(0xffffffffu, p, kk);
#pragma unroll
        for (int j = 0; j < DPL; ++j) {
          const int dd = lane + 32 * j;
          if (dd < d) acc[i][j] = fmaf(pk, v_s[kk * d + dd], acc[i][j]);
        }
      }
    }
  }

#pragma unroll
  for (int i = 0; i < kAttnRowsPerWarp; ++i) {
    const int r = warp * kAttnRowsPerWarp + i;
    if (r >= nrows) continue;
    const int t = r / gc, g = r - t * gc;
    T* dst = out + (size_t)(row0 + t0 + t) * q_width + (kvh * group + g0 + g) * d;
    const float inv = 1.f / l[i];
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      const int dd = lane + 32 * j;
      if (dd < d) dst[dd] = from_f32<T>(acc[i][j] * inv);
    }
  }
}

template <typename T, int DPL>
static int launch_attention(const void* q, const void* pool, void* out, const AttnArgs& a,
                            int n_entries, int max_q_len, cudaStream_t stream) {
  const int d = a.head_dim;
  const size_t smem = sizeof(float) * ((size_t)kAttnRows * d + (size_t)kAttnKeys * (d + 1) + (size_t)kAttnKeys * d);
  if (smem > 227 * 1024) return TIB_E_SMEM;
  auto kern = paged_attention_simt_kernel<T, DPL>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int group = a.heads / a.kv_heads;
  const int chunks = (group + a.group_chunk - 1) / a.group_chunk;
  dim3 grid(ceil_div(max_q_len, a.q_tile), n_entries, a.kv_heads * chunks);
  kern<<<grid, kAttnWarps * 32, smem, stream>>>((const T*)q, (const T*)pool, (T*)out, a);
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

}  // namespace tib

using namespace tib;

// q, out: [n_tokens, heads * head_dim]; pool: this layer's pages
// [pages][2][kv_heads][page_size][head_dim]; q_start: [n_entries + 1];
// kv_start, slots: [n_entries]; max_q_len: the longest entry of the batch.
TIB_API int tib_paged_attention_simt(const void* q, const void* pool, void* out, const int* q_start,
                                     const int* kv_start, const int* slots, const int* block_table,
                                     int table_stride, int n_entries, int max_q_len, int heads,
                                     int kv_heads, int head_dim, int page_size, int64_t page_stride,
                                     int num_pages, int window, float scale, int* error_word,
                                     int dtype, cudaStream_t stream) {
  if (n_entries == 0 || max_q_len == 0) return TIB_OK;
  if (!q || !pool || !out || !q_start || !kv_start || !slots || !block_table) return TIB_E_ARG;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads != 0 || head_dim < 1 || page_size < 1) return TIB_E_SIZE;
  if (head_dim > 256) return TIB_E_SIZE;
  if (n_entries > 65535) return TIB_E_SIZE;
  AttnArgs a;
  a.q_start = q_start; a.kv_start = kv_start; a.slots = slots; a.block_table = block_table;
  a.table_stride = table_stride; a.heads = heads; a.kv_heads = kv_heads; a.head_dim = head_dim;
  a.page_size = page_size; a.page_stride = page_stride; a.num_pages = num_pages; a.window = window;
  a.scale = scale; a.error_word = error_word;
  const int group = heads / kv_heads;
  a.group_chunk = group < kAttnRows ? group : kAttnRows;
  a.q_tile = kAttnRows / a.group_chunk;
  const int chunks = (group + a.group_chunk - 1) / a.group_chunk;
  if ((int64_t)kv_heads * chunks > 65535) return TIB_E_SIZE;
  const int dpl = (head_dim + 31) / 32;
#define TIB_ATTN_DISPATCH(T)                                                                     \
  (dpl <= 1 ? launch_attention<T, 1>(q, pool, out, a, n_entries, max_q_len, stream)             \
   : dpl <= 2 ? launch_attention<T, 2>(q, pool, out, a, n_entries, max_q_len, stream)           \
   : dpl <= 4 ? launch_attention<T, 4>(q, pool, out, a, n_entries, max_q_len, stream)           \
              : launch_attention<T, 8>(q, pool, out, a, n_entries, max_q_len, stream))
  if (dtype == TIB_F32) return TIB_ATTN_DISPATCH(float);
  if (dtype == TIB_BF16) return TIB_ATTN_DISPATCH(__nv_bfloat16);
#undef TIB_ATTN_DISPATCH
  return TIB_E_DTYPE;
}
