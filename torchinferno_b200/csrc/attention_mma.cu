// Paged attention on tensor cores (bf16 in, fp32 softmax and accumulation), for head sizes in steps
// of 16 up to 128 (the tiles in shared memory are 64 or 128 wide; columns past the head's width are
// zeros, which add nothing to a score and are not stored):
//
//   prefill_attention_kernel   portions of prompts: a block owns 64 rows (token, query head) of one
//                              kv head and walks the keys up to the causal edge, flash-attention style
//   decode_attention_kernel    single tokens: the context of one (request, kv head) is split over
//                              blocks ("split-K"); each block streams its keys once for all query heads
//                              of the group and leaves (max, sum, unnormalised output) in scratch
//   decode_merge_kernel        (mma.cuh) combines the partial results exactly (fp32)
//
// Formula as in attention_simt.cu (src/torchinferno/models/llama3/raw_ops.py:44-51; streaming form
// src/torchinferno/kernels/triton_ops.py:2555-2574, whose grid is (batch, kv_heads) with no split
// over the context: triton_ops.py:2661).  Keys and values come from the pages by block table
// (layout [pages][2][kv_heads][page_size][head_dim]); any page size works, since every key row is
// fetched by its own address.  Keys past a block's last query position are never read from memory
// (they may be unwritten): their shared-memory rows are zero-filled, and they are masked.
#include "mma.cuh"
#include <mutex>

namespace tib {

constexpr int kBN = 64;        // keys per tile
constexpr int kMmaThreads = 128;

struct MmaAttnArgs {
  const int* q_start;
  const int* kv_start;
  const int* slots;
  const int* block_table;
  int table_stride;
  int heads, kv_heads, group;
  int head_dim;          // width of a head in memory: a multiple of 16, at most the kernels' D (tiles are padded with zeros)
  int page_size;
  int page_shift;        // log2(page_size) when it is a power of two, else -1
  int64_t page_stride;
  int num_pages;
  int window;
  float scale_log2;      // scale * log2(e)
  int chunk;             // decode: keys per split (multiple of kBN); 0: each request's context / num_splits
  int num_splits;        // decode
  int skip_single;       // prefill: leave single-token entries to the decode kernel
};

// Shared-memory tile [rows][D] of bf16 with the 16-byte chunks of a row XOR-swizzled by (row & 7),
// so that the eight rows an ldmatrix touches fall into different banks.
template <int D> __device__ __forceinline__ __nv_bfloat16* tile_at(__nv_bfloat16* tile, int row, int col) {
  const int chunk = (col >> 3) ^ (row & 7);
  return tile + row * D + chunk * 8 + (col & 7);
}

// Fetch keys [key0, key0 + kBN) of one kv head into k_tile / v_tile.  Keys outside
// [first_key, last_key] and keys whose page is gone are zero-filled.
template <int D>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* k_tile, __nv_bfloat16* v_tile,
                                             const __nv_bfloat16* pool, const int* table, int kvh, int key0,
                                             int first_key, int last_key, const MmaAttnArgs& a) {
  constexpr int CPR = D / 8;                       // 16-byte chunks per key row
  constexpr int ROWS = kMmaThreads / CPR;          // rows fetched by one pass of the block
  constexpr int PASSES = kBN / ROWS;
  const int hd = a.head_dim;
  const int64_t v_off = (int64_t)a.kv_heads * a.page_size * hd;
  const int c = threadIdx.x % CPR, r0 = threadIdx.x / CPR;
  const bool in_head = c * 8 < hd;                 // chunks past the head's width stay zero
  // first all page ids (independent loads, one latency), then all copies
  int page[PASSES], within[PASSES];
#pragma unroll
  for (int i = 0; i < PASSES; ++i) {
    const int kp = key0 + r0 + i * ROWS;
    const bool valid = kp >= first_key && kp <= last_key;
    int idx, off;
    if (a.page_shift >= 0) {
      idx = kp >> a.page_shift;
      off = kp & (a.page_size - 1);
    } else {
      idx = kp / a.page_size;
      off = kp - idx * a.page_size;
    }
    within[i] = off;
    page[i] = valid ? __ldg(table + idx) : -1;
  }
#pragma unroll
  for (int i = 0; i < PASSES; ++i) {
    const int r = r0 + i * ROWS;
    const bool valid = in_head && page[i] >= 0 && page[i] < a.num_pages;
    const __nv_bfloat16* src = valid ? pool + (int64_t)page[i] * a.page_stride + ((int64_t)kvh * a.page_size + within[i]) * hd + c * 8 : pool;
    const int off = r * D + ((c ^ (r & 7)) << 3);
    cp_async16(k_tile + off, src, valid);
    cp_async16(v_tile + off, valid ? src + v_off : pool, valid);
  }
}

// s[8][4] = Q(16 x D) . K(64 keys x D)^T for a whole tile: eight independent accumulators per k step.
template <int D>
__device__ __forceinline__ void qk_tile(float (&s)[kBN / 8][4], const uint32_t (&qf)[D / 16][4], __nv_bfloat16* k_tile,
                                        int lane) {
#pragma unroll
  for (int nt = 0; nt < kBN / 8; ++nt)
#pragma unroll
    for (int j = 0; j < 4; ++j) s[nt][j] = 0.f;
  const int krow = (lane & 7) + ((lane >> 4) << 3);
  const int kcol = ((lane >> 3) & 1) << 3;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
    for (int kk = 0; kk < kBN / 16; ++kk) {
      uint32_t b[4];
      ldmatrix_x4(b, tile_at<D>(k_tile, kk * 16 + krow, ks * 16 + kcol));
      mma_bf16(s[2 * kk], qf[ks], b[0], b[1]);
      mma_bf16(s[2 * kk + 1], qf[ks], b[2], b[3]);
    }
  }
}

// s[2][4] = Q(16 x D) . K(16 keys x D)^T for the keys [slab, slab + 16) of a tile.
template <int D>
__device__ __forceinline__ void qk_slab(float (&s)[2][4], const uint32_t (&qf)[D / 16][4], __nv_bfloat16* k_tile,
                                        int slab, int lane) {
  // even and odd k steps go to accumulators of their own: four independent chains instead of two
  float e[2][4];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int j = 0; j < 4; ++j) s[nt][j] = e[nt][j] = 0.f;
  const int krow = slab + (lane & 7) + ((lane >> 4) << 3);
  const int kcol = ((lane >> 3) & 1) << 3;
#pragma unroll
  for (int ks = 0; ks < D / 16; ks += 2) {
    uint32_t b[4], c[4];
    ldmatrix_x4(b, tile_at<D>(k_tile, krow, ks * 16 + kcol));
    ldmatrix_x4(c, tile_at<D>(k_tile, krow, (ks + 1) * 16 + kcol));
    mma_bf16(s[0], qf[ks], b[0], b[1]);
    mma_bf16(s[1], qf[ks], b[2], b[3]);
    mma_bf16(e[0], qf[ks + 1], c[0], c[1]);
    mma_bf16(e[1], qf[ks + 1], c[2], c[3]);
  }
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int j = 0; j < 4; ++j) s[nt][j] += e[nt][j];
}

// o(16 x D) += P(16 x 16 keys) . V(16 keys x D) for the keys [slab, slab + 16) of a tile.
template <int D>
__device__ __forceinline__ void pv_slab(float (&o)[D / 8][4], const uint32_t (&p)[4], __nv_bfloat16* v_tile, int slab,
                                        int lane) {
  const int vrow = slab + (lane & 7) + (((lane >> 3) & 1) << 3);
  const int vcol = (lane >> 4) << 3;
#pragma unroll
  for (int dn = 0; dn < D / 16; ++dn) {
    uint32_t b[4];
    ldmatrix_x4_trans(b, tile_at<D>(v_tile, vrow, dn * 16 + vcol));
    mma_bf16(o[2 * dn], p, b[0], b[1]);
    mma_bf16(o[2 * dn + 1], p, b[2], b[3]);
  }
}

// ------------------------------------------------------------------ prefill
template <int D, int STAGES>
__global__ void __launch_bounds__(kMmaThreads, D <= 64 ? 4 : 3)
prefill_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pool,
                         __nv_bfloat16* __restrict__ out, MmaAttnArgs a) {
  constexpr int BM = 64;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [STAGES][kBN][D]
  __nv_bfloat16* v_s = k_s + STAGES * kBN * D;
  // The queries only pass through shared memory on their way to registers: they borrow the key buffer of
  // the last stage, which is first filled inside the loop, after every warp has taken its fragments.
  static_assert(BM == kBN, "the query tile borrows one key stage");
  __nv_bfloat16* q_s = k_s + (STAGES - 1) * kBN * D;                 // [BM][D]

  const int entry = blockIdx.z, kvh = blockIdx.y;
  const int row0 = a.q_start[entry];
  const int q_len = a.q_start[entry + 1] - row0;
  if (q_len == 1 && a.skip_single) return;
  const int tok_per_tile = BM / a.group;
  const int tile = gridDim.x - 1 - blockIdx.x;  // the longest tiles start first
  const int t0 = tile * tok_per_tile;
  if (t0 >= q_len) return;
  const int nt = min(tok_per_tile, q_len - t0);
  const int nrows = nt * a.group;
  const int pos0 = a.kv_start[entry] + t0;
  const int last_pos = pos0 + nt - 1;
  const int first_key = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
  const int* table = a.block_table + (size_t)a.slots[entry] * a.table_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hd = a.head_dim;
  const int q_width = a.heads * hd;

  // queries of the tile -> shared memory (rows beyond nrows, and columns beyond the head's width, are zero)
  constexpr int CPR = D / 8;
  for (int idx = threadIdx.x; idx < BM * CPR; idx += kMmaThreads) {
    const int r = idx / CPR, c = idx - r * CPR;
    const bool valid = r < nrows && c * 8 < hd;
    const int t = r / a.group, g = r - t * a.group;
    const __nv_bfloat16* src = valid ? q + (size_t)(row0 + t0 + t) * q_width + (kvh * a.group + g) * hd + c * 8 : q;
    cp_async16(q_s + r * D + ((c ^ (r & 7)) << 3), src, valid);
  }
  cp_async_commit();

  const int kt0 = first_key / kBN, kt1 = last_pos / kBN;
  const int n_tiles = kt1 - kt0 + 1;
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (st < n_tiles)
      load_kv_tile<D>(k_s + st * kBN * D, v_s + st * kBN * D, pool, table, kvh, (kt0 + st) * kBN, first_key, last_pos, a);
    cp_async_commit();
  }

  // the warp's 16 query rows as A fragments
  uint32_t qf[D / 16][4];
  cp_async_wait<STAGES - 1>();
  __syncthreads();
  {
    const int qrow = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
    const int qcol = (lane >> 4) << 3;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) ldmatrix_x4(qf[ks], tile_at<D>(q_s, qrow, ks * 16 + qcol));
  }

  float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[n][j] = 0.f;

  // positions of this thread's two rows (padded rows take the last position: harmless and finite)
  const int g_row = lane >> 2, tig = lane & 3;
  int qpos[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + g_row + 8 * h;
    qpos[h] = r < nrows ? pos0 + r / a.group : last_pos;
  }

  for (int it = 0; it < n_tiles; ++it) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {
      const int nxt = it + STAGES - 1;
      if (nxt < n_tiles) {
        const int st = nxt % STAGES;
        load_kv_tile<D>(k_s + st * kBN * D, v_s + st * kBN * D, pool, table, kvh, (kt0 + nxt) * kBN, first_key, last_pos, a);
      }
      cp_async_commit();
    }
    __nv_bfloat16* k_tile = k_s + (it % STAGES) * kBN * D;
    __nv_bfloat16* v_tile = v_s + (it % STAGES) * kBN * D;
    const int key_base = (kt0 + it) * kBN;
    // tiles wholly inside every row's allowed range need no mask
    const bool need_mask = key_base + kBN - 1 > pos0 || (a.window > 0 && key_base < last_pos - a.window + 1);
    float s[kBN / 8][4];
    qk_tile<D>(s, qf, k_tile, lane);
#pragma unroll
    for (int n2 = 0; n2 < kBN / 8; ++n2)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = s[n2][j] * a.scale_log2;
        if (need_mask) {
          const int key = key_base + n2 * 8 + tig * 2 + (j & 1);
          const int qp = qpos[j >> 1];
          const bool ok = key <= qp && (a.window <= 0 || key > qp - a.window);
          v = ok ? v : -CUDART_INF_F;
        }
        s[n2][j] = v;
      }
    uint32_t p[kBN / 16][4];
    softmax_step<kBN / 8, D / 8>(s, m, l, o, p);
#pragma unroll
    for (int kk = 0; kk < kBN / 16; ++kk) pv_slab<D>(o, p[kk], v_tile, kk * 16, lane);
  }
  cp_async_wait<0>();

  // normalise and store
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float sum = l[h];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    const int r = warp * 16 + g_row + 8 * h;
    if (r >= nrows) continue;
    const float inv = 1.f / sum;
    const int t = r / a.group, g = r - t * a.group;
    __nv_bfloat16* dst = out + (size_t)(row0 + t0 + t) * q_width + (kvh * a.group + g) * hd;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      const uint32_t v = pack_bf16(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
      if (n * 8 < hd) *reinterpret_cast<uint32_t*>(dst + n * 8 + tig * 2) = v;
    }
  }
}

// ------------------------------------------------------------------- decode
// grid: (num_splits, kv_heads * row_tiles, n_entries).  partial_o: [entries][heads][splits][D] fp32,
// partial_ml: [entries][heads][splits][2] fp32 (max in log2 units, sum).
template <int D, int STAGES>
__global__ void __launch_bounds__(kMmaThreads)
decode_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pool,
                        float* __restrict__ partial_o, float* __restrict__ partial_ml,
                        __nv_bfloat16* __restrict__ out, MmaAttnArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [16][D]
  __nv_bfloat16* k_s = q_s + 16 * D;                                 // [STAGES][kBN][D]
  __nv_bfloat16* v_s = k_s + STAGES * kBN * D;

  const int entry = blockIdx.z, split = blockIdx.x;
  const int row_tiles = (a.group + 15) / 16;
  const int kvh = blockIdx.y / row_tiles, rt = blockIdx.y - kvh * row_tiles;
  const int row0 = a.q_start[entry];
  if (a.q_start[entry + 1] - row0 != 1) return;  // portions belong to the prefill kernel
  const int g0 = rt * 16;
  const int nrows = min(16, a.group - g0);
  const int pos = a.kv_start[entry];
  const int first_key = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  // chunk == 0: this request's own context is cut into num_splits equal parts (multiples of kBN),
  // so every split has work whatever bound the host knew when it chose the grid
  const int first_tile_key = first_key / kBN * kBN;
  const int chunk = a.chunk > 0 ? a.chunk
                                : max(kBN, ((pos + 1 - first_tile_key + a.num_splits - 1) / a.num_splits + kBN - 1) / kBN * kBN);
  const int kb = first_tile_key + split * chunk;
  const int ke = min(kb + chunk, pos + 1);  // exclusive
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g_row = lane >> 2, tig = lane & 3;
  const int head0 = kvh * a.group + g0;

  if (kb > pos) {  // nothing in this split: an empty partial, which the merge ignores
    if (a.num_splits > 1 && threadIdx.x < nrows) {
      float* ml = partial_ml + (((size_t)entry * a.heads + head0 + threadIdx.x) * a.num_splits + split) * 2;
      ml[0] = -CUDART_INF_F;
      ml[1] = 0.f;
    }
    return;
  }
  const int* table = a.block_table + (size_t)a.slots[entry] * a.table_stride;

  const int hd = a.head_dim;
  constexpr int CPR = D / 8;
  for (int idx = threadIdx.x; idx < 16 * CPR; idx += kMmaThreads) {
    const int r = idx / CPR, c = idx - r * CPR;
    const bool valid = r < nrows && c * 8 < hd;
    const __nv_bfloat16* src = valid ? q + ((size_t)row0 * a.heads + head0 + r) * hd + c * 8 : q;
    cp_async16(q_s + r * D + ((c ^ (r & 7)) << 3), src, valid);
  }
  cp_async_commit();

  const int n_tiles = (ke - kb + kBN - 1) / kBN;
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (st < n_tiles)
      load_kv_tile<D>(k_s + st * kBN * D, v_s + st * kBN * D, pool, table, kvh, kb + st * kBN, first_key, pos, a);
    cp_async_commit();
  }
  uint32_t qf[D / 16][4];
  cp_async_wait<STAGES - 1>();
  __syncthreads();
  {
    const int qrow = (lane & 7) + (((lane >> 3) & 1) << 3);
    const int qcol = (lane >> 4) << 3;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) ldmatrix_x4(qf[ks], tile_at<D>(q_s, qrow, ks * 16 + qcol));
  }

  float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[n][j] = 0.f;

  for (int it = 0; it < n_tiles; ++it) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {
      const int nxt = it + STAGES - 1;
      if (nxt < n_tiles) {
        const int st = nxt % STAGES;
        load_kv_tile<D>(k_s + st * kBN * D, v_s + st * kBN * D, pool, table, kvh, kb + nxt * kBN, first_key, pos, a);
      }
      cp_async_commit();
    }
    __nv_bfloat16* k_tile = k_s + (it % STAGES) * kBN * D;
    __nv_bfloat16* v_tile = v_s + (it % STAGES) * kBN * D;
    const int key_base = kb + it * kBN + warp * 16;  // each warp takes 16 keys of the tile
    if (key_base > pos) continue;                    // (uniform in the warp)
    float s[2][4];
    qk_slab<D>(s, qf, k_tile, warp * 16, lane);
#pragma unroll
    for (int n2 = 0; n2 < 2; ++n2)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = key_base + n2 * 8 + tig * 2 + (j & 1);
        const bool ok = key <= pos && key >= first_key && key < ke;
        s[n2][j] = ok ? s[n2][j] * a.scale_log2 : -CUDART_INF_F;
      }
    uint32_t p[1][4];
    softmax_step<2, D / 8>(s, m, l, o, p);
    pv_slab<D>(o, p[0], v_tile, warp * 16, lane);
  }
  cp_async_wait<0>();
  __syncthreads();  // all warps are done with the tiles: their memory is reused below

  // merge the four warps (each saw a quarter of the keys) in shared memory
  float* red_o = reinterpret_cast<float*>(k_s);          // [4][16][D]
  float* red_ml = red_o + 4 * 16 * D;                    // [4][16][2]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float sum = l[h];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    const int r = g_row + 8 * h;
    if (tig == 0) {
      red_ml[(warp * 16 + r) * 2] = m[h];
      red_ml[(warp * 16 + r) * 2 + 1] = sum;
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      red_o[(warp * 16 + r) * D + n * 8 + tig * 2] = o[n][2 * h];
      red_o[(warp * 16 + r) * D + n * 8 + tig * 2 + 1] = o[n][2 * h + 1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nrows * D; idx += kMmaThreads) {
    const int r = idx / D, dd = idx - r * D;
    if (dd >= hd) continue;
    float mm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red_ml[(w * 16 + r) * 2]);
    const float base = mm == -CUDART_INF_F ? 0.f : mm;
    float acc = 0.f, sum = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float wgt = exp2f(red_ml[(w * 16 + r) * 2] - base);
      acc += red_o[(w * 16 + r) * D + dd] * wgt;
      sum += red_ml[(w * 16 + r) * 2 + 1] * wgt;
    }
    if (a.num_splits == 1) {
      out[((size_t)row0 * a.heads + head0 + r) * hd + dd] = __float2bfloat16_rn(acc / sum);
    } else {
      const size_t slot = ((size_t)entry * a.heads + head0 + r) * a.num_splits + split;
      partial_o[slot * hd + dd] = acc;
      if (dd == 0) {
        partial_ml[slot * 2] = mm;
        partial_ml[slot * 2 + 1] = sum;
      }
    }
  }
}

template <int D>
static int launch_prefill(const void* q, const void* pool, void* out, const MmaAttnArgs& a, int n_entries,
                          int max_q_len, cudaStream_t stream) {
  constexpr int STAGES = 2;
  const size_t smem = sizeof(__nv_bfloat16) * (2 * (size_t)STAGES * kBN * D);
  auto kern = prefill_attention_kernel<D, STAGES>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int tok_per_tile = 64 / a.group;
  dim3 grid(ceil_div(max_q_len, tok_per_tile), a.kv_heads, n_entries);
  kern<<<grid, kMmaThreads, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)pool, (__nv_bfloat16*)out, a);
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

template <int D>
static int launch_decode(const void* q, const void* pool, float* partial_o, float* partial_ml, void* out,
                         const MmaAttnArgs& a, int n_entries, cudaStream_t stream) {
  constexpr int STAGES = 3;
  size_t smem = sizeof(__nv_bfloat16) * ((size_t)16 * D + 2 * (size_t)STAGES * kBN * D);
  const size_t reduce = sizeof(__nv_bfloat16) * 16 * D + sizeof(float) * (4 * 16 * D + 4 * 16 * 2);
  if (reduce > smem) smem = reduce;
  auto kern = decode_attention_kernel<D, STAGES>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int row_tiles = (a.group + 15) / 16;
  dim3 grid(a.num_splits, a.kv_heads * row_tiles, n_entries);
  kern<<<grid, kMmaThreads, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)pool, partial_o, partial_ml,
                                            (__nv_bfloat16*)out, a);
  TIB_LAUNCH_CHECK();
  if (a.num_splits > 1) {
    dim3 mgrid(a.heads, n_entries);
    decode_merge_kernel<D><<<mgrid, D, (a.num_splits + 1) * sizeof(float), stream>>>(partial_o, partial_ml, (__nv_bfloat16*)out, a.q_start, a.heads, a.num_splits, a.head_dim);
    TIB_LAUNCH_CHECK();
  }
  return TIB_OK;
}

static int fill_args(MmaAttnArgs& a, const int* q_start, const int* kv_start, const int* slots, const int* block_table,
                     int table_stride, int heads, int kv_heads, int head_dim, int page_size, int64_t page_stride,
                     int num_pages, int window, float scale) {
  if (!q_start || !kv_start || !slots || !block_table) return TIB_E_ARG;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads != 0 || page_size < 1) return TIB_E_SIZE;
  if (head_dim < 16 || head_dim > 128 || head_dim % 16 != 0) return TIB_E_SIZE;
  if (page_stride % 8 != 0) return TIB_E_ALIGN;  // 16-byte copies of key rows
  a.q_start = q_start; a.kv_start = kv_start; a.slots = slots; a.block_table = block_table;
  a.table_stride = table_stride; a.heads = heads; a.kv_heads = kv_heads; a.group = heads / kv_heads;
  a.head_dim = head_dim;
  a.page_size = page_size; a.page_shift = -1;
  for (int sft = 0; sft < 31; ++sft) if ((1 << sft) == page_size) a.page_shift = sft;
  a.page_stride = page_stride; a.num_pages = num_pages; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.chunk = kBN; a.num_splits = 1; a.skip_single = 0;
  return TIB_OK;
}

}  // namespace tib

using namespace tib;

// Which head sizes the tensor-core attention kernels are built for.
TIB_API int tib_attention_mma_supports(int head_dim, int group) {
  return head_dim >= 16 && head_dim <= 128 && head_dim % 16 == 0 && group >= 1 && group <= 64;
}

// Portions of prompts (and, unless skip_single, single tokens too).  bf16 only.
TIB_API int tib_prefill_attention(const void* q, const void* pool, void* out, const int* q_start,
                                  const int* kv_start, const int* slots, const int* block_table,
                                  int table_stride, int n_entries, int max_q_len, int heads, int kv_heads,
                                  int head_dim, int page_size, int64_t page_stride, int num_pages, int window,
                                  float scale, int skip_single, cudaStream_t stream) {
  if (n_entries == 0 || max_q_len == 0) return TIB_OK;
  if (!q || !pool || !out) return TIB_E_ARG;
  MmaAttnArgs a;
  int rc = fill_args(a, q_start, kv_start, slots, block_table, table_stride, heads, kv_heads, head_dim, page_size,
                     page_stride, num_pages, window, scale);
  if (rc != TIB_OK) return rc;
  if (a.group > 64 || n_entries > 65535 || kv_heads > 65535) return TIB_E_SIZE;
  a.skip_single = skip_single;
  return head_dim <= 64 ? launch_prefill<64>(q, pool, out, a, n_entries, max_q_len, stream)
                        : launch_prefill<128>(q, pool, out, a, n_entries, max_q_len, stream);
}

// Single-token entries, context split into num_splits parts of `chunk` keys (a multiple of 64;
// num_splits * chunk must cover the longest context), or, with chunk == 0, each request's own
// context split into num_splits equal parts.  scratch_o: [n_entries * heads * num_splits *
// head_dim] floats, scratch_ml: [n_entries * heads * num_splits * 2] floats (unused when num_splits == 1).
TIB_API int tib_decode_attention(const void* q, const void* pool, void* out, float* scratch_o, float* scratch_ml,
                                 const int* q_start, const int* kv_start, const int* slots, const int* block_table,
                                 int table_stride, int n_entries, int heads, int kv_heads, int head_dim,
                                 int page_size, int64_t page_stride, int num_pages, int window, float scale,
                                 int num_splits, int chunk, cudaStream_t stream) {
  if (n_entries == 0) return TIB_OK;
  if (!q || !pool || !out) return TIB_E_ARG;
  if (num_splits < 1 || num_splits > 4096 || chunk < 0 || (chunk > 0 && chunk < kBN) || chunk % kBN != 0) return TIB_E_SIZE;
  if (num_splits > 1 && (!scratch_o || !scratch_ml)) return TIB_E_ARG;
  MmaAttnArgs a;
  int rc = fill_args(a, q_start, kv_start, slots, block_table, table_stride, heads, kv_heads, head_dim, page_size,
                     page_stride, num_pages, window, scale);
  if (rc != TIB_OK) return rc;
  const int row_tiles = (a.group + 15) / 16;
  if (n_entries > 65535 || (int64_t)kv_heads * row_tiles > 65535) return TIB_E_SIZE;
  a.num_splits = num_splits;
  a.chunk = chunk;
  return head_dim <= 64 ? launch_decode<64>(q, pool, scratch_o, scratch_ml, out, a, n_entries, stream)
                        : launch_decode<128>(q, pool, scratch_o, scratch_ml, out, a, n_entries, stream);
}

// ---------------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc (or any allocator) at the time they need
// attention: code that runs inside another framework's memory plan with a fixed budget, a real-time
// loop that may not take the allocator's lock or tolerate its latency, or a plug-in whose host
// forbids allocation after start-up.  tib_decode_attention needs scratch for the partial results of
// its context splits; here that scratch is a fixed array in the library's own device image.
//
//  * The array holds TIB_NOALLOC_SCRATCH_FLOATS floats (16 MiB).  Every GPU that loads this library
//    carries it until the process exits, whether or not this entry point is ever called.
//  * A call needs n_entries * heads * num_splits * (head_dim + 2) floats; a call that needs more is
//    refused with TIB_E_SCRATCH and nothing is launched.  With num_splits == 1 no scratch is used.
//  * The first call on a device looks the array's device address up (cudaGetSymbolAddress, with that
//    device current) and keeps it; make that first call before any stream capture begins.
//  * All calls share the one array, and it keeps what the last call left.  Nothing in it has to
//    start at zero: every call writes each (entry, head, split) record it later reads.  Two calls
//    that overlap on the GPU (different streams, no ordering between them) race on the array; order
//    them on one stream or with events.
//  * No cudaMalloc, cudaFree or allocating library routine is called here.
#define TIB_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)
static __device__ __align__(256) float tib_noalloc_scratch[TIB_NOALLOC_SCRATCH_FLOATS];

static float* noalloc_scratch_address(int* status) {
  // In host code `tib_noalloc_scratch` names a host-side shadow of the symbol, not device memory;
  // the device address must be asked for, once per device, with that device current.
  constexpr int kMaxDevices = 64;
  static float* address[kMaxDevices] = {nullptr};
  static std::mutex guard;                 // (first calls from two host threads would otherwise race on the table)
  std::lock_guard<std::mutex> lock(guard);
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) { *status = (int)e; return nullptr; }
  if (device < 0 || device >= kMaxDevices) { *status = TIB_E_ARG; return nullptr; }
  if (address[device] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, tib_noalloc_scratch);
    if (e != cudaSuccess) { *status = (int)e; return nullptr; }
    address[device] = ptr;
  }
  *status = TIB_OK;
  return address[device];
}

// How many floats of the built-in scratch a call would use (0 when num_splits == 1).
TIB_API long long tib_decode_attention_noalloc_need(int n_entries, int heads, int head_dim, int num_splits) {
  if (num_splits <= 1) return 0;
  return (long long)n_entries * heads * num_splits * (head_dim + 2);
}

TIB_API long long tib_decode_attention_noalloc_capacity(void) { return TIB_NOALLOC_SCRATCH_FLOATS; }

// Same contract as tib_decode_attention, minus the two scratch pointers.  The caller passes inputs
// and outputs; the partial results live in the library's own array (see above).  max_kv_len is the
// longest context of the batch (the largest kv_start + 1): a split that does not cover it is refused.
TIB_API int tib_decode_attention_noalloc(const void* q, const void* pool, void* out, const int* q_start,
                                         const int* kv_start, const int* slots, const int* block_table,
                                         int table_stride, int n_entries, int heads, int kv_heads, int head_dim,
                                         int page_size, int64_t page_stride, int num_pages, int window, float scale,
                                         int num_splits, int chunk, int max_kv_len, cudaStream_t stream) {
  if (n_entries == 0) return TIB_OK;
  if (!q || !pool || !out || n_entries < 0 || max_kv_len < 1) return TIB_E_ARG;
  if (num_splits < 1 || num_splits > 4096 || chunk < kBN || chunk % kBN != 0) return TIB_E_SIZE;
  // the parts must cover the longest context: keys beyond num_splits * chunk would be left out without a sign
  if ((long long)num_splits * chunk < (long long)max_kv_len) return TIB_E_SIZE;
  MmaAttnArgs a;
  int rc = fill_args(a, q_start, kv_start, slots, block_table, table_stride, heads, kv_heads, head_dim, page_size,
                     page_stride, num_pages, window, scale);
  if (rc != TIB_OK) return rc;
  const int row_tiles = (a.group + 15) / 16;
  if (n_entries > 65535 || (int64_t)kv_heads * row_tiles > 65535) return TIB_E_SIZE;
  const long long need = tib_decode_attention_noalloc_need(n_entries, heads, head_dim, num_splits);
  if (need > TIB_NOALLOC_SCRATCH_FLOATS) return TIB_E_SCRATCH;
  float* scratch_o = nullptr;
  float* scratch_ml = nullptr;
  if (num_splits > 1) {
    float* base = noalloc_scratch_address(&rc);
    if (rc != TIB_OK) return rc;
    scratch_o = base;
    scratch_ml = base + (size_t)n_entries * heads * num_splits * head_dim;
  }
  a.num_splits = num_splits;
  a.chunk = chunk;
  return head_dim <= 64 ? launch_decode<64>(q, pool, scratch_o, scratch_ml, out, a, n_entries, stream)
                        : launch_decode<128>(q, pool, scratch_o, scratch_ml, out, a, n_entries, stream);
}
