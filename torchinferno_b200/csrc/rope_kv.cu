// Rotary position encoding of q and k, fused with the write of k and v into
// the paged cache.
//
// Formula (src/torchinferno/models/llama3/pipeline.py:555-568): angle =
// float(position) * inv_freq[i]; rotate-half pairs (i, i + rot/2):
//   lo' = lo * cos - hi * sin,   hi' = hi * cos + lo * sin.
// Angles, cos and sin are 32-bit.  The frequency table is an input, so any
// scaling law is a different table, not a different kernel.  `interleaved`
// pairs (2i, 2i+1) instead; `rot_dim` < head_dim leaves the tail unrotated.
//
// Cache layout of one layer: [pages][2 (k, v)][kv_heads][page_size][head_dim];
// a token at `position` of the request in `slot` goes to page
// block_table[slot][position / page_size] at offset position % page_size
// (slot arithmetic as in src/torchinferno/runtime/paged.py:463-477).
#include "common.cuh"

namespace tib {

template <typename T>
__global__ void rope_append_kernel(const T* __restrict__ qkv, T* __restrict__ q_out,
                                   T* __restrict__ pool, const int* __restrict__ positions,
                                   const int* __restrict__ token_slot,
                                   const int* __restrict__ block_table, int table_stride,
                                   const float* __restrict__ inv_freq, int heads, int kv_heads,
                                   int head_dim, int rot_dim, int interleaved, int page_size,
                                   int64_t page_stride, int num_pages, int write_kv,
                                   int* __restrict__ error_word) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float cs[];  // cos[rot/2], sin[rot/2]
  const int tok = blockIdx.x;
  const int pos = positions[tok];
  const int half = rot_dim >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cn;
    sincosf((float)pos * inv_freq[i], &sn, &cn);
    cs[i] = cn;
    cs[half + i] = sn;
  }
  __syncthreads();

  const int q_width = heads * head_dim, kv_width = kv_heads * head_dim;
  const T* row = qkv + (size_t)tok * (q_width + 2 * kv_width);

  // q: rotate into q_out
  const int pairs_per_head = head_dim >> 1;  // work items per head: rotated pairs + pass-through pairs
  for (int w = threadIdx.x; w < heads * pairs_per_head; w += blockDim.x) {
    const int hh = w / pairs_per_head, i = w - hh * pairs_per_head;
    const T* src = row + hh * head_dim;
    T* dst = q_out + (size_t)tok * q_width + hh * head_dim;
    if (i < half) {
      const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
      const float lo = to_f32(src[a]), hi = to_f32(src[b]);
      const float c = cs[i], s = cs[half + i];
      dst[a] = from_f32<T>(rope_lo(lo, hi, c, s));
      dst[b] = from_f32<T>(rope_hi(lo, hi, c, s));
    } else {
      const int a = rot_dim + 2 * (i - half);
      dst[a] = src[a];
      dst[a + 1] = src[a + 1];
    }
  }
  if (!write_kv) return;

  const int slot = token_slot[tok];
  const int page = block_table[(size_t)slot * table_stride + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (error_word && threadIdx.x == 0) atomicExch(error_word, 1 + tok);
    return;
  }
  const int off = pos % page_size;
  T* kpage = pool + (size_t)page * page_stride;
  T* vpage = kpage + (size_t)kv_heads * page_size * head_dim;
  const T* ksrc = row + q_width;
  const T* vsrc = ksrc + kv_width;
  for (int w = threadIdx.x; w < kv_heads * pairs_per_head; w += blockDim.x) {
    const int hh = w / pairs_per_head, i = w - hh * pairs_per_head;
    const T* src = ksrc + hh * head_dim;
    T* dst = kpage + ((size_t)hh * page_size + off) * head_dim;
    if (i < half) {
      const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
      const float lo = to_f32(src[a]), hi = to_f32(src[b]);
      const float c = cs[i], s = cs[half + i];
      dst[a] = from_f32<T>(rope_lo(lo, hi, c, s));
      dst[b] = from_f32<T>(rope_hi(lo, hi, c, s));
    } else {
      const int a = rot_dim + 2 * (i - half);
      dst[a] = src[a];
      dst[a + 1] = src[a + 1];
    }
  }
  for (int w = threadIdx.x; w < kv_width; w += blockDim.x) {
    const int hh = w / head_dim, dd = w - hh * head_dim;
    vpage[((size_t)hh * page_size + off) * head_dim + dd] = vsrc[w];
  }
}

// bf16, full rotate-half rotation, head size a multiple of 16.  A work item is eight dims of the lower half of a q or
// k head and their partners in the upper half (two 16-byte loads and stores), or sixteen dims of a v head (two
// 16-byte copies).  A thread asks for its first item's data before the block makes its table of cos and sin and
// before it looks its page up, so that the row is on its way from memory while that happens.
// (MAXT: the most threads a block is launched with; the registers a thread may use follow from it)
template <int MAXT>
__global__ void __launch_bounds__(MAXT)
rope_append_bf16x8_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                          __nv_bfloat16* __restrict__ pool, const int* __restrict__ positions,
                          const int* __restrict__ token_slot, const int* __restrict__ block_table,
                          int table_stride, const float* __restrict__ inv_freq, int heads, int kv_heads,
                          int head_dim, int chunk_shift, int page_size, int64_t page_stride, int num_pages, int write_kv,
                          int* __restrict__ error_word) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(16) float cs[];  // cos[d/2], sin[d/2]
  const int tok = blockIdx.x;
  const int half = head_dim >> 1;
  const int q_width = heads * head_dim, kv_width = kv_heads * head_dim;
  const __nv_bfloat16* row = qkv + (size_t)tok * (q_width + 2 * kv_width);
  const int chunks = half >> 3;                 // work items per q, k or v head
  const int rot_items = (heads + (write_kv ? kv_heads : 0)) * chunks;
  const int items = rot_items + (write_kv ? kv_heads * chunks : 0);
  // (chunk_shift: log2 of the work items per head when that is a power of two, else -1)
  auto head_of = [&](int w) { return chunk_shift >= 0 ? w >> chunk_shift : w / chunks; };
  // where the two 16-byte pieces of item w stand in the row: q heads, k heads and v heads follow one another there
  auto source = [&](int w, const __nv_bfloat16*& a, const __nv_bfloat16*& b) {
    const int hh = head_of(w), c = (w - hh * chunks) << 3;
    if (w < rot_items) {
      a = row + hh * head_dim + c;
      b = a + half;
    } else {                                    // v: sixteen dims in a row
      a = row + hh * head_dim + 2 * c;
      b = a + 8;
    }
  };
  int w = threadIdx.x;
  uint4 araw = make_uint4(0, 0, 0, 0), braw = araw;
  if (w < items) {
    const __nv_bfloat16 *a, *b;
    source(w, a, b);
    araw = *reinterpret_cast<const uint4*>(a);
    braw = *reinterpret_cast<const uint4*>(b);
  }
  const int pos = positions[tok];
  __nv_bfloat16* kpage = nullptr;
  int off = 0;
  if (write_kv) {
    const int page = block_table[(size_t)token_slot[tok] * table_stride + pos / page_size];
    if (page < 0 || page >= num_pages) {
      if (error_word && threadIdx.x == 0) atomicExch(error_word, 1 + tok);
    } else {
      kpage = pool + (size_t)page * page_stride;
      off = pos % page_size;
    }
  }
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cn;
    sincosf((float)pos * inv_freq[i], &sn, &cn);   // (the accurate one: angles reach 10^5 radians)
    cs[i] = cn;
    cs[half + i] = sn;
  }
  __syncthreads();
  __nv_bfloat16* vpage = kpage ? kpage + (size_t)kv_heads * page_size * head_dim : nullptr;
  while (w < items) {
    const int hh = head_of(w), c = (w - hh * chunks) << 3;
    if (w < rot_items) {
      __nv_bfloat16* dst = hh < heads ? q_out + (size_t)tok * q_width + hh * head_dim
                                      : (kpage ? kpage + ((size_t)(hh - heads) * page_size + off) * head_dim : nullptr);
      if (dst) {
        const __nv_bfloat162* l2 = reinterpret_cast<const __nv_bfloat162*>(&araw);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&braw);
        uint4 lo_out, hi_out;
        __nv_bfloat162* lo2 = reinterpret_cast<__nv_bfloat162*>(&lo_out);
        __nv_bfloat162* hi2 = reinterpret_cast<__nv_bfloat162*>(&hi_out);
        float cv[8], sv[8];                                // cos and sin of this item's eight dims: four 16-byte loads
        *reinterpret_cast<float4*>(cv) = *reinterpret_cast<const float4*>(cs + c);
        *reinterpret_cast<float4*>(cv + 4) = *reinterpret_cast<const float4*>(cs + c + 4);
        *reinterpret_cast<float4*>(sv) = *reinterpret_cast<const float4*>(cs + half + c);
        *reinterpret_cast<float4*>(sv + 4) = *reinterpret_cast<const float4*>(cs + half + c + 4);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 lo = bf16x2_floats(l2[k]), hi = bf16x2_floats(h2[k]);
          const float c0 = cv[2 * k], c1 = cv[2 * k + 1], s0 = sv[2 * k], s1 = sv[2 * k + 1];
          lo2[k] = __floats2bfloat162_rn(rope_lo(lo.x, hi.x, c0, s0), rope_lo(lo.y, hi.y, c1, s1));
          hi2[k] = __floats2bfloat162_rn(rope_hi(lo.x, hi.x, c0, s0), rope_hi(lo.y, hi.y, c1, s1));
        }
        *reinterpret_cast<uint4*>(dst + c) = lo_out;
        *reinterpret_cast<uint4*>(dst + half + c) = hi_out;
      }
    } else if (vpage) {
      __nv_bfloat16* dst = vpage + ((size_t)(hh - heads - kv_heads) * page_size + off) * head_dim + 2 * c;
      *reinterpret_cast<uint4*>(dst) = araw;
      *reinterpret_cast<uint4*>(dst + 8) = braw;
    }
    w += blockDim.x;
    if (w < items) {
      const __nv_bfloat16 *a, *b;
      source(w, a, b);
      araw = *reinterpret_cast<const uint4*>(a);
      braw = *reinterpret_cast<const uint4*>(b);
    }
  }
}

}  // namespace tib

using namespace tib;

// qkv: [n_tokens, (heads + 2*kv_heads) * head_dim]; q_out: [n_tokens, heads * head_dim];
// pool: this layer's pages; block_table: [slots, table_stride] page ids.
TIB_API int tib_rope_append(const void* qkv, void* q_out, void* pool, const int* positions,
                            const int* token_slot, const int* block_table, int table_stride,
                            const float* inv_freq, int n_tokens, int heads, int kv_heads,
                            int head_dim, int rot_dim, int interleaved, int page_size,
                            int64_t page_stride, int num_pages, int write_kv, int* error_word,
                            int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return TIB_OK;
  if (!qkv || !q_out || !positions || n_tokens < 0) return TIB_E_ARG;
  if (rot_dim > 0 && !inv_freq) return TIB_E_ARG;
  if (write_kv && (!pool || !token_slot || !block_table || page_size < 1)) return TIB_E_ARG;
  if (heads < 1 || kv_heads < 0 || head_dim < 2 || (head_dim & 1)) return TIB_E_SIZE;
  if (rot_dim < 0 || rot_dim > head_dim || (rot_dim & 1)) return TIB_E_SIZE;
  const int threads = 256;
  const size_t smem = (size_t)rot_dim * sizeof(float);
  if (smem > 48 * 1024) return TIB_E_SMEM;
  int chunk_shift = -1;                                  // log2(head_dim / 16) when that is a power of two
  for (int sft = 0; sft < 16; ++sft)
    if ((16 << sft) == head_dim) chunk_shift = sft;
  if (dtype == TIB_F32)
    TIB_LAUNCH_DEPENDENT(rope_append_kernel<float>, n_tokens, threads, smem, stream,
        (const float*)qkv, (float*)q_out, (float*)pool, positions, token_slot, block_table,
        table_stride, inv_freq, heads, kv_heads, head_dim, rot_dim, interleaved, page_size,
        page_stride, num_pages, write_kv, error_word);
  else if (dtype == TIB_BF16 && rot_dim == head_dim && !interleaved && head_dim % 16 == 0 &&
           (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)pool) & 15) == 0 && (page_stride % 8 == 0 || !write_kv)) {
    // With few tokens (a decode step) a block is all there is on its SM and its latency is the kernel's: it gets as
    // many threads as a token has work items (eight dims of a q or k head and their partners, sixteen of a v head;
    // 32 + 8 + 8 heads of 128 are 448), so that they are done in one pass.  With many tokens smaller blocks share
    // the SMs better: the fewest equal passes of at most 256 threads (two of 224 there: 18.4 us at 2,048 tokens
    // against 19.3 with 256 threads and 23.4 with 448).
    const int items = (heads + (write_kv ? 2 * kv_heads : 0)) * (head_dim / 16);
    const int passes = (items + 255) / 256;
    const int item_threads = n_tokens <= 128 && items <= 1024 ? (items + 31) / 32 * 32 : ((items + passes - 1) / passes + 31) / 32 * 32;
    if (item_threads <= 256)
      TIB_LAUNCH_DEPENDENT(rope_append_bf16x8_kernel<256>, n_tokens, item_threads < 64 ? 64 : item_threads, smem, stream,
          (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)pool, positions, token_slot, block_table,
          table_stride, inv_freq, heads, kv_heads, head_dim, chunk_shift, page_size, page_stride, num_pages, write_kv, error_word);
    else
      TIB_LAUNCH_DEPENDENT(rope_append_bf16x8_kernel<1024>, n_tokens, item_threads, smem, stream,
          (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)pool, positions, token_slot, block_table,
          table_stride, inv_freq, heads, kv_heads, head_dim, chunk_shift, page_size, page_stride, num_pages, write_kv, error_word);
  } else if (dtype == TIB_BF16)
    TIB_LAUNCH_DEPENDENT(rope_append_kernel<__nv_bfloat16>, n_tokens, threads, smem, stream,
        (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)pool, positions,
        token_slot, block_table, table_stride, inv_freq, heads, kv_heads, head_dim, rot_dim,
        interleaved, page_size, page_stride, num_pages, write_kv, error_word);
  else
    return TIB_E_DTYPE;
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}
