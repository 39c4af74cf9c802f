// Decode attention over the paged cache with the keys and values brought in by TMA.
//
// One block serves one (request, kv head, part of the context).  Warp 0 is the producer: it looks the
// pages of a 64-key tile up in the block table and has the TMA unit copy them (one box per page and per
// 64-wide half of the head) into a ring of shared-memory stages; no other thread computes an address or
// touches global memory for keys and values.  Warps 1-4 are the consumers: each takes 16 keys of every
// tile, S = Q.K^T and O += P.V on mma.sync (the query rows are the group's heads, padded to 16), with a
// streaming softmax of its own in 32-bit; the four partial results are merged exactly at the end, and the
// parts of a split context by decode_merge_kernel.  Stages are handed over with mbarriers (TMA arrival
// "full", four consumer arrivals "empty"), so there is no block-wide barrier inside the loop, and two
// blocks of three 32 KB stages each keep about 190 KB of copies in flight per SM.
//
// Same formula and contract as decode_attention_kernel in attention_mma.cu (formula:
// src/torchinferno/models/llama3/raw_ops.py:44-51; the reference's decode kernel walks one
// (batch, kv head) per program without a split: src/torchinferno/kernels/triton_ops.py:2555-2574, 2661).
// Takes head sizes 64 and 128, groups up to 16 heads, pages of 8, 16, 32 or 64 tokens packed back to
// back; other shapes stay with the cp.async kernel.
#include "mma.cuh"
#include "tcgen05.cuh"

namespace tib {

constexpr int kDtBN = 64;               // keys per tile
constexpr int kDtConsumers = 4;         // warps; each takes kDtBN / 4 = 16 keys of a tile
constexpr int kDtThreads = 32 * (1 + kDtConsumers);
constexpr int kDtMinPart = 192;         // keys: a context is not cut into parts shorter than this (three tiles)

struct DtArgs {
  const int* q_start;
  const int* kv_start;
  const int* slots;
  const int* block_table;
  int table_stride;
  int heads, kv_heads, group;
  int page_size, page_shift;
  int num_pages;
  int window;
  float scale_log2;
  int chunk, num_splits;
  int* counters;         // [entries * kv_heads] zeros: the parts of a split context count themselves in; or null
  int* error_word;
  // The kernel rotates and stores the newest token itself (ROPE): q points at the unrotated rows of the qkv
  // product (q_stride elements apart; k at column heads * D, v behind it), which the kernel before wrote.
  int q_stride;
  const float* inv_freq;  // [rot_dim / 2]
  int rot_dim, interleaved;
  __nv_bfloat16* pool;    // this layer's pages, to write the newest key and value into
  int64_t page_stride;
};

template <int D>
struct DtSmem {
  static constexpr int kStages = D == 128 ? 3 : 6;
  static constexpr uint32_t kSub = kDtBN * 128;                   // one 64-wide half of a tile: 64 rows of 128 bytes
  static constexpr uint32_t kKV = (D / 64) * kSub;                // keys (or values) of one tile
  static constexpr uint32_t kStage = 2 * kKV;
  static constexpr uint32_t kReduce = sizeof(float) * (kDtConsumers * 16 * D + kDtConsumers * 16 * 2);
  static constexpr uint32_t kData = kStages * kStage > kReduce ? kStages * kStage : kReduce;
  static constexpr uint32_t kRope = 16 * D * 2 + 2 * D * 4;       // rotated queries [16][D] bf16; cos, sin of the position, twice
  static constexpr uint32_t kTotal = 1024 + kData + 16 * kStages + kRope;
};

// Address of element (row, col) of a tile half-by-half in the TMA's 128-byte swizzle: the 16-byte chunk
// index within a 128-byte row is XORed with the row's low three bits.
__device__ __forceinline__ uint32_t dt_at(uint32_t tile, int row, int col) {
  return tile + (uint32_t)(col >> 6) * (kDtBN * 128) + (uint32_t)row * 128 + ((((col >> 3) & 7) ^ (row & 7)) << 4) + ((col & 7) << 1);
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// grid: (num_splits, kv_heads, n_entries).  partial_o: [entries][heads][splits][D] fp32, partial_ml:
// [entries][heads][splits][2] fp32 (max in log2 units, sum).
// ROPE: q holds the unrotated rows of the qkv product.  The four consumer warps rotate the group's queries into
// shared memory (each part of a context does: four heads cost less than a trip to memory), and in the block
// whose part holds the newest position the producer warp rotates that token's key, writes key and value into
// their page and only then has the tile copied (a proxy fence between its stores and the copy); no kernel
// between the qkv product and this one.  Same arithmetic as rope_append_kernel (rope_kv.cu).
template <int D, bool ROPE>
__global__ void __launch_bounds__(kDtThreads)
decode_attention_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const __nv_bfloat16* __restrict__ q,
                            float* __restrict__ partial_o, float* __restrict__ partial_ml,
                            __nv_bfloat16* __restrict__ out, DtArgs a) {
  using L = DtSmem<D>;
  constexpr int STAGES = L::kStages;
  // Placed early (programmatic dependent launch), the block starts copying at once: the kernel before it
  // in the stream writes only the newest token's keys and values and the queries, so everything older may
  // be fetched while that kernel still runs.  pdl_wait() stands before the first read of the newest tile,
  // before the queries are read, and before anything is written.
  pdl_trigger();
  __shared__ int ticket_s;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;     // the swizzle pattern repeats every 1024 bytes
  unsigned char* smem_gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + L::kData;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_gen + L::kData + 16 * STAGES);   // [16][D]
  float* cs_s = reinterpret_cast<float*>(q_s + 16 * D);                                        // consumers' cos | sin
  float* cs_p = cs_s + D;                                                                      // the producer's own
  auto full = [&](int s) { return bars + 8u * s; };
  auto empty = [&](int s) { return bars + 8u * (STAGES + s); };
  auto k_s = [&](int s) { return base + (uint32_t)s * L::kStage; };
  auto v_s = [&](int s) { return base + (uint32_t)s * L::kStage + L::kKV; };

  const int entry = blockIdx.z, split = blockIdx.x, kvh = blockIdx.y;
  if (threadIdx.x == 0) asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_kv) : "memory");
  const int slot = a.slots[entry];                        // (asked for together with the loads below: one latency)
  const int row0 = a.q_start[entry];
  if (a.q_start[entry + 1] - row0 != 1) return;          // portions belong to the prefill kernel
  const int nrows = a.group;
  const int pos = a.kv_start[entry];
  const int first_key = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  // chunk == 0: this request's own context is cut into num_splits equal parts (multiples of a tile)
  const int first_tile_key = first_key / kDtBN * kDtBN;
  // ... but into no more parts than it has stretches of kDtMinPart keys: the grid is sized for the longest
  // context the step may meet, and a short one leaves the blocks past its last part idle.  (Only where the
  // parts merge themselves: the separate merge kernel reads every part.)
  int parts = a.num_splits;
  if (a.chunk == 0 && a.num_splits > 1 && a.counters != nullptr) {
    parts = min(a.num_splits, max(1, (pos + 1 - first_tile_key + kDtMinPart - 1) / kDtMinPart));
    if (split >= parts) return;
  }
  const int chunk = a.chunk > 0 ? a.chunk
                                : max(kDtBN, ((pos + 1 - first_tile_key + parts - 1) / parts + kDtBN - 1) / kDtBN * kDtBN);
  const int kb = first_tile_key + split * chunk;
  const int ke = min(kb + chunk, pos + 1);               // exclusive
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head0 = kvh * a.group;

  const bool empty_part = kb > pos;   // nothing in this part: an empty partial, which the merge ignores
  if (empty_part) {
    pdl_wait();
    if (parts > 1 && threadIdx.x < nrows) {
      float* ml = partial_ml + (((size_t)entry * a.heads + head0 + threadIdx.x) * a.num_splits + split) * 2;
      ml[0] = -CUDART_INF_F;
      ml[1] = 0.f;
    }
  }
  const int n_tiles = empty_part ? 0 : (ke - kb + kDtBN - 1) / kDtBN;
  if (!empty_part) {

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), kDtConsumers);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
  float o[D / 8][4];

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    const int* table = a.block_table + (size_t)slot * a.table_stride;
    const int pages_per_tile = kDtBN >> a.page_shift;
    const int oob_row = a.num_pages * 2 * a.kv_heads * a.page_size;   // past the tensor: the copy fills zeros
    bool ok = true, waited = false;
    for (int it = 0; it < n_tiles; ++it) {
      const int s = it % STAGES;
      const uint32_t round = it / STAGES;
      const int key0 = kb + it * kDtBN;
      if (!waited && key0 + kDtBN > pos) {   // the tile that holds the newest token
        // (what does not depend on the kernel before: the page of the newest position, cos and sin of its angles)
        int page_new = -1;
        if constexpr (ROPE) {
          page_new = __ldg(table + (pos >> a.page_shift));
          const int half = a.rot_dim >> 1;
          for (int i = lane; i < half; i += 32) {
            float sn, cn;
            sincosf((float)pos * a.inv_freq[i], &sn, &cn);
            cs_p[i] = cn;
            cs_p[half + i] = sn;
          }
        }
        pdl_wait();
        waited = true;
        if constexpr (ROPE) {
          // this part holds the newest position: its key (rotated) and value go into their page first
          if (page_new < 0 || page_new >= a.num_pages) {
            if (a.error_word && lane == 0) atomicExch(a.error_word, 1 + entry);
          } else {
            const int half = a.rot_dim >> 1;
            __syncwarp();
            const __nv_bfloat16* ksrc = q + (size_t)row0 * a.q_stride + (size_t)(a.heads + kvh) * D;
            const __nv_bfloat16* vsrc = ksrc + (size_t)a.kv_heads * D;
            __nv_bfloat16* kdst = a.pool + (size_t)page_new * a.page_stride + ((size_t)kvh * a.page_size + (pos & (a.page_size - 1))) * D;
            __nv_bfloat16* vdst = kdst + (size_t)a.kv_heads * a.page_size * D;
            for (int i = lane; i < D / 2; i += 32) {
              if (i < half) {
                const int ia = a.interleaved ? 2 * i : i, ib = a.interleaved ? 2 * i + 1 : i + half;
                const float lo = __bfloat162float(ksrc[ia]), hi = __bfloat162float(ksrc[ib]);
                kdst[ia] = __float2bfloat16_rn(rope_lo(lo, hi, cs_p[i], cs_p[half + i]));
                kdst[ib] = __float2bfloat16_rn(rope_hi(lo, hi, cs_p[i], cs_p[half + i]));
              } else {
                const int ia = a.rot_dim + 2 * (i - half);
                kdst[ia] = ksrc[ia];
                kdst[ia + 1] = ksrc[ia + 1];
              }
            }
            for (int i = lane; i < D / 8; i += 32)
              reinterpret_cast<uint4*>(vdst)[i] = reinterpret_cast<const uint4*>(vsrc)[i];
            // the copy below reads these stores through the async proxy
            asm volatile("fence.proxy.async;\n" ::: "memory");
            __syncwarp();
          }
        }
      }
      int page = -1;
      if (lane < pages_per_tile) {
        const int kp = key0 + lane * a.page_size;
        // pages wholly outside [first_key, pos] are not looked up: they may be gone or never taken
        if (kp <= pos && kp + a.page_size > first_key) page = __ldg(table + (kp >> a.page_shift));
      }
      if (lane == 0) {
        if (round > 0 && !mbar_wait(empty(s), (round - 1) & 1)) {
          if (a.error_word) atomicExch(a.error_word, 0x7C0031);
          ok = false;
        }
        if (ok) mbar_expect_tx(full(s), L::kStage);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < pages_per_tile) {
        const bool have = page >= 0 && page < a.num_pages;
        const int krow = have ? ((page * 2 + 0) * a.kv_heads + kvh) * a.page_size : oob_row;
        const int vrow = have ? ((page * 2 + 1) * a.kv_heads + kvh) * a.page_size : oob_row;
        const uint32_t off = (uint32_t)(lane * a.page_size) * 128u;
#pragma unroll
        for (int h = 0; h < D / 64; ++h) {
          tma_load_2d(k_s(s) + h * L::kSub + off, &map_kv, h * 64, krow, full(s));
          tma_load_2d(v_s(s) + h * L::kSub + off, &map_kv, h * 64, vrow, full(s));
        }
      }
      __syncwarp();
    }
  } else {
    // ----------------------------------------------------------------- consumers
    const int cw = warp - 1;                    // which 16 keys of every tile
    const int g_row = lane >> 2, tig = lane & 3;
    if constexpr (ROPE) {   // (cos and sin of the position's angles do not depend on the kernel before)
      const int ct = threadIdx.x - 32, half = a.rot_dim >> 1;
      for (int i = ct; i < half; i += 32 * kDtConsumers) {
        float sn, cn;
        sincosf((float)pos * a.inv_freq[i], &sn, &cn);
        cs_s[i] = cn;
        cs_s[half + i] = sn;
      }
    }
    pdl_wait();
    if constexpr (ROPE) {
      // the group's queries, rotated, into shared memory: 128 threads, a pair of dims each per pass
      const int ct = threadIdx.x - 32, half = a.rot_dim >> 1;
      asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kDtConsumers) : "memory");
      for (int w = ct; w < nrows * (D / 2); w += 32 * kDtConsumers) {
        const int r = w / (D / 2), i = w - r * (D / 2);
        const __nv_bfloat16* src = q + (size_t)row0 * a.q_stride + (size_t)(head0 + r) * D;
        __nv_bfloat16* dst = q_s + r * D;
        if (i < half) {
          const int ia = a.interleaved ? 2 * i : i, ib = a.interleaved ? 2 * i + 1 : i + half;
          const float lo = __bfloat162float(src[ia]), hi = __bfloat162float(src[ib]);
          dst[ia] = __float2bfloat16_rn(rope_lo(lo, hi, cs_s[i], cs_s[half + i]));
          dst[ib] = __float2bfloat16_rn(rope_hi(lo, hi, cs_s[i], cs_s[half + i]));
        } else {
          const int ia = a.rot_dim + 2 * (i - half);
          dst[ia] = src[ia];
          dst[ia + 1] = src[ia + 1];
        }
      }
      asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kDtConsumers) : "memory");
    }
    // Q fragments (from global memory, or rotated from shared memory): row g_row of the A operand is head head0 + g_row
    uint32_t qf[D / 16][4];
    {
      const __nv_bfloat16* qrow = ROPE ? q_s + g_row * D : q + (size_t)row0 * a.q_stride + (size_t)(head0 + g_row) * D;
      const __nv_bfloat16* qrow8 = qrow + 8 * D;
      const bool v0 = g_row < nrows, v8 = g_row + 8 < nrows;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        qf[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + tig * 2) : 0u;
        qf[ks][1] = v8 ? *reinterpret_cast<const uint32_t*>(qrow8 + ks * 16 + tig * 2) : 0u;
        qf[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + tig * 2) : 0u;
        qf[ks][3] = v8 ? *reinterpret_cast<const uint32_t*>(qrow8 + ks * 16 + 8 + tig * 2) : 0u;
      }
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) o[n][j] = 0.f;

    const int krow = cw * 16 + (lane & 7) + ((lane >> 4) << 3);
    const int kcol = ((lane >> 3) & 1) << 3;
    const int vrow = cw * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
    const int vcol = (lane >> 4) << 3;
    bool ok = true;
    for (int it = 0; it < n_tiles && ok; ++it) {
      const int s = it % STAGES;
      if (!mbar_wait(full(s), (it / STAGES) & 1)) {
        if (a.error_word && lane == 0) atomicExch(a.error_word, 0x7C0032);
        ok = false;
        break;
      }
      const int key_base = kb + it * kDtBN + cw * 16;
      if (key_base <= pos && key_base + 16 > first_key) {           // (uniform in the warp)
        if (key_base + 15 > pos) {
          // value rows of keys past the request's end may never have been written: they must not be NaN
          const int r = lane >> 1;                                   // two lanes per row, half a 128-byte row each
          if (key_base + r > pos) {
#pragma unroll
            for (int h = 0; h < D / 64; ++h) {
              uint4* dst = reinterpret_cast<uint4*>(smem_gen + (v_s(s) - base) + h * L::kSub + (cw * 16 + r) * 128 + (lane & 1) * 64);
#pragma unroll
              for (int c = 0; c < 4; ++c) dst[c] = make_uint4(0u, 0u, 0u, 0u);
            }
          }
          __syncwarp();
        }
        // s = Q(16 x D) . K(16 keys x D)^T, even and odd k steps in accumulators of their own
        float sc[2][4], e[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j) sc[nt][j] = e[nt][j] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ks += 2) {
          uint32_t b[4], c[4];
          ldsm_x4(b, dt_at(k_s(s), krow, ks * 16 + kcol));
          ldsm_x4(c, dt_at(k_s(s), krow, (ks + 1) * 16 + kcol));
          mma_bf16(sc[0], qf[ks], b[0], b[1]);
          mma_bf16(sc[1], qf[ks], b[2], b[3]);
          mma_bf16(e[0], qf[ks + 1], c[0], c[1]);
          mma_bf16(e[1], qf[ks + 1], c[2], c[3]);
        }
#pragma unroll
        for (int n2 = 0; n2 < 2; ++n2)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int key = key_base + n2 * 8 + tig * 2 + (j & 1);
            const bool allowed = key <= pos && key >= first_key && key < ke;
            sc[n2][j] = allowed ? (sc[n2][j] + e[n2][j]) * a.scale_log2 : -CUDART_INF_F;
          }
        uint32_t p[1][4];
        softmax_step<2, D / 8>(sc, m, l, o, p);
#pragma unroll
        for (int dn = 0; dn < D / 16; ++dn) {
          uint32_t b[4];
          ldsm_x4_trans(b, dt_at(v_s(s), vrow, dn * 16 + vcol));
          mma_bf16(o[2 * dn], p[0], b[0], b[1]);
          mma_bf16(o[2 * dn + 1], p[0], b[2], b[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty(s));
    }
  }
  __syncthreads();  // every copy has landed and been read: the stages' memory is reused below
  pdl_wait();

  // merge the four consumer warps (each saw a quarter of the keys) in shared memory
  float* red_o = reinterpret_cast<float*>(smem_gen);                 // [4][16][D]
  float* red_ml = red_o + kDtConsumers * 16 * D;                     // [4][16][2]
  if (warp > 0) {
    const int cw = warp - 1, g_row = lane >> 2, tig = lane & 3;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float sum = l[h];
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      const int r = g_row + 8 * h;
      if (tig == 0) {
        red_ml[(cw * 16 + r) * 2] = m[h];
        red_ml[(cw * 16 + r) * 2 + 1] = sum;
      }
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        red_o[(cw * 16 + r) * D + n * 8 + tig * 2] = o[n][2 * h];
        red_o[(cw * 16 + r) * D + n * 8 + tig * 2 + 1] = o[n][2 * h + 1];
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nrows * D; idx += kDtThreads) {
    const int r = idx / D, dd = idx - r * D;
    float mm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kDtConsumers; ++w) mm = fmaxf(mm, red_ml[(w * 16 + r) * 2]);
    const float basev = mm == -CUDART_INF_F ? 0.f : mm;
    float acc = 0.f, sum = 0.f;
#pragma unroll
    for (int w = 0; w < kDtConsumers; ++w) {
      const float wgt = exp2f(red_ml[(w * 16 + r) * 2] - basev);
      acc += red_o[(w * 16 + r) * D + dd] * wgt;
      sum += red_ml[(w * 16 + r) * 2 + 1] * wgt;
    }
    if (parts == 1) {
      out[(size_t)row0 * a.heads * D + (head0 + r) * D + dd] = __float2bfloat16_rn(acc / sum);
    } else {
      const size_t slot = ((size_t)entry * a.heads + head0 + r) * a.num_splits + split;
      partial_o[slot * D + dd] = acc;
      if (dd == 0) {
        partial_ml[slot * 2] = mm;
        partial_ml[slot * 2 + 1] = sum;
      }
    }
  }
  }  // (!empty_part)

  // The parts of one (request, kv head) count themselves in; the one that arrives last merges them all, so
  // no second kernel is needed.  The counter is left at zero for the next launch.
  if (parts == 1 || a.counters == nullptr) return;
  __syncthreads();                       // every thread's part of the partial result is written ...
  int* counter = a.counters + (size_t)entry * a.kv_heads + kvh;
  if (threadIdx.x == 0) {
    __threadfence();                     // ... and visible to the device before this block counts itself in
    ticket_s = atomicAdd(counter, 1);
  }
  __syncthreads();
  if (ticket_s != parts - 1) return;
  __threadfence();
  const int ns = parts, stride = a.num_splits;
  const size_t slot0 = ((size_t)entry * a.heads + head0) * stride;   // (row r, part sp) is slot0 + r * stride + sp
  if (ns <= 16) {
    // few parts: every thread asks for all it needs at once (its row's maxima and sums and its four output
    // columns of every part), so the merge costs one trip to the L2, not one per dependent step
    for (int idx = threadIdx.x; idx < nrows * (D / 4); idx += kDtThreads) {
      const int r = idx / (D / 4), d4 = idx - r * (D / 4);
      const float2* pm = reinterpret_cast<const float2*>(partial_ml) + slot0 + r * stride;
      const float4* po = reinterpret_cast<const float4*>(partial_o + (slot0 + r * stride) * D) + d4;
      float2 ml[16];
      float4 ov[16];
#pragma unroll
      for (int sp = 0; sp < 16; ++sp) {
        const bool have = sp < ns;
        ml[sp] = have ? __ldcg(pm + sp) : make_float2(-CUDART_INF_F, 0.f);
        ov[sp] = have ? __ldcg(po + (size_t)sp * (D / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      float mm = -CUDART_INF_F;
#pragma unroll
      for (int sp = 0; sp < 16; ++sp) mm = fmaxf(mm, ml[sp].x);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      float sum = 0.f;
#pragma unroll
      for (int sp = 0; sp < 16; ++sp) {
        if (ml[sp].x == -CUDART_INF_F) continue;   // an empty part wrote no output (what was read may be anything)
        const float w = exp2f(ml[sp].x - mm);
        sum += w * ml[sp].y;
        acc.x += w * ov[sp].x; acc.y += w * ov[sp].y; acc.z += w * ov[sp].z; acc.w += w * ov[sp].w;
      }
      const float inv = 1.f / sum;
      uint2 packed;
      packed.x = pack_bf16(acc.x * inv, acc.y * inv);
      packed.y = pack_bf16(acc.z * inv, acc.w * inv);
      *reinterpret_cast<uint2*>(out + (size_t)row0 * a.heads * D + (head0 + r) * D + d4 * 4) = packed;
    }
    if (threadIdx.x == 0) *counter = 0;
    return;
  }
  // weights of the parts first (one load per (row, part), all in flight together), then the sums with the
  // loads of several parts in flight: nothing here waits for one load after another
  float* wgt_s = reinterpret_cast<float*>(smem_gen);                 // [nrows][num_splits] weights, then [nrows] 1 / sum
  for (int r = warp; r < nrows; r += kDtThreads / 32) {
    float mm = -CUDART_INF_F;
    for (int sp = lane; sp < ns; sp += 32) mm = fmaxf(mm, __ldcg(partial_ml + (slot0 + r * stride + sp) * 2));
    mm = warp_max(mm);
    float sum = 0.f;
    for (int sp = lane; sp < ns; sp += 32) {
      const float ms = __ldcg(partial_ml + (slot0 + r * stride + sp) * 2);
      const float w = ms == -CUDART_INF_F ? 0.f : exp2f(ms - mm);     // an empty part wrote no output
      wgt_s[r * ns + sp] = w;
      sum += w == 0.f ? 0.f : w * __ldcg(partial_ml + (slot0 + r * stride + sp) * 2 + 1);
    }
    sum = warp_sum(sum);
    if (lane == 0) wgt_s[nrows * ns + r] = 1.f / sum;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nrows * (D / 4); idx += kDtThreads) {   // four output elements per thread
    const int r = idx / (D / 4), d4 = idx - r * (D / 4);
    const float4* po = reinterpret_cast<const float4*>(partial_o + (slot0 + r * stride) * D) + d4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int sp = 0; sp < ns; ++sp) {
      const float w = wgt_s[r * ns + sp];
      if (w != 0.f) {
        const float4 v = __ldcg(po + (size_t)sp * (D / 4));
        acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
      }
    }
    const float inv = wgt_s[nrows * ns + r];
    uint2 packed;
    packed.x = pack_bf16(acc.x * inv, acc.y * inv);
    packed.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(out + (size_t)row0 * a.heads * D + (head0 + r) * D + d4 * 4) = packed;
  }
  if (threadIdx.x == 0) *counter = 0;
}

template <int D, bool ROPE>
static int launch_decode_tma(const void* q, const void* pool, float* partial_o, float* partial_ml, void* out,
                             const DtArgs& a, int n_entries, cudaStream_t stream) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return TIB_E_ARG;
  CUtensorMap map_kv;
  // one layer's pages as rows of D: [pages * 2 * kv_heads * page_size][D]; a box is 64 dims x one page of one head
  const cuuint64_t rows = (cuuint64_t)a.num_pages * 2 * a.kv_heads * a.page_size;
  const cuuint64_t dims[2] = {(cuuint64_t)D, rows};
  const cuuint64_t strides[1] = {(cuuint64_t)D * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)a.page_size};
  const cuuint32_t elem[2] = {1, 1};
  if (fn(&map_kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return TIB_E_ARG;
  auto kern = decode_attention_tma_kernel<D, ROPE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DtSmem<D>::kTotal);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(a.num_splits, a.kv_heads, n_entries);
  TIB_LAUNCH_DEPENDENT(kern, grid, kDtThreads, DtSmem<D>::kTotal, stream, map_kv, (const __nv_bfloat16*)q, partial_o,
                       partial_ml, (__nv_bfloat16*)out, a);
  TIB_LAUNCH_CHECK();
  if (a.num_splits > 1 && a.counters == nullptr) {
    dim3 mgrid(a.heads, n_entries);
    TIB_LAUNCH_DEPENDENT(decode_merge_kernel<D>, mgrid, D, (a.num_splits + 1) * sizeof(float), stream, (const float*)partial_o, (const float*)partial_ml,
                         (__nv_bfloat16*)out, a.q_start, a.heads, a.num_splits, D);
    TIB_LAUNCH_CHECK();
  }
  return TIB_OK;
}

}  // namespace tib

using namespace tib;

// Whether tib_decode_attention_tma takes these sizes.
TIB_API int tib_decode_attention_tma_supports(int head_dim, int group, int page_size) {
  return (head_dim == 64 || head_dim == 128) && group >= 1 && group <= 16 &&
         (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64);
}

// Same contract as tib_decode_attention (bf16).  page_stride must equal 2 * kv_heads * page_size *
// head_dim (pages packed back to back).  A bounded wait that runs out sets *error_word (0x7C003x).
// counters: n_entries * kv_heads ints that are zero (the kernel leaves them zero): with them the parts of a
// split context are merged by the block that finishes last; without (null) by a second kernel.  Launches
// that may overlap on the GPU need counters of their own.
static int decode_attention_tma(const void* q, int q_stride, const void* pool, void* out, float* scratch_o, float* scratch_ml,
                                const int* q_start, const int* kv_start, const int* slots, const int* block_table,
                                int table_stride, int n_entries, int heads, int kv_heads, int head_dim,
                                int page_size, int64_t page_stride, int num_pages, int window, float scale,
                                int num_splits, int chunk, int* counters, int* error_word, bool rope, const float* inv_freq,
                                int rot_dim, int interleaved, cudaStream_t stream) {
  if (n_entries == 0) return TIB_OK;
  if (!q || !pool || !out || !q_start || !kv_start || !slots || !block_table) return TIB_E_ARG;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads != 0) return TIB_E_SIZE;
  if (!tib_decode_attention_tma_supports(head_dim, heads / kv_heads, page_size)) return TIB_E_SIZE;
  if (num_splits < 1 || num_splits > 1024 || chunk < 0 || chunk % kDtBN != 0) return TIB_E_SIZE;   // (the merge keeps a weight per part in shared memory)
  if (num_splits > 1 && (!scratch_o || !scratch_ml)) return TIB_E_ARG;
  if (page_stride != (int64_t)2 * kv_heads * page_size * head_dim) return TIB_E_ALIGN;
  if ((((uintptr_t)q | (uintptr_t)pool | (uintptr_t)out) & 15) != 0 || q_stride % 8 != 0) return TIB_E_ALIGN;
  if (n_entries > 65535 || kv_heads > 65535) return TIB_E_SIZE;
  if ((int64_t)num_pages * 2 * kv_heads * page_size >= ((int64_t)1 << 31)) return TIB_E_SIZE;   // row coordinates are 32-bit
  if (rope && (rot_dim < 0 || rot_dim > head_dim || (rot_dim & 1) || (rot_dim > 0 && !inv_freq))) return TIB_E_SIZE;
  DtArgs a;
  a.q_start = q_start; a.kv_start = kv_start; a.slots = slots; a.block_table = block_table;
  a.table_stride = table_stride; a.heads = heads; a.kv_heads = kv_heads; a.group = heads / kv_heads;
  a.page_size = page_size; a.page_shift = 0;
  while ((1 << a.page_shift) < page_size) ++a.page_shift;
  a.num_pages = num_pages; a.window = window; a.scale_log2 = scale * 1.4426950408889634f;
  a.chunk = chunk; a.num_splits = num_splits; a.counters = counters; a.error_word = error_word;
  a.q_stride = q_stride; a.inv_freq = inv_freq; a.rot_dim = rot_dim; a.interleaved = interleaved;
  a.pool = (__nv_bfloat16*)const_cast<void*>(pool); a.page_stride = page_stride;
  if (rope)
    return head_dim == 64 ? launch_decode_tma<64, true>(q, pool, scratch_o, scratch_ml, out, a, n_entries, stream)
                          : launch_decode_tma<128, true>(q, pool, scratch_o, scratch_ml, out, a, n_entries, stream);
  return head_dim == 64 ? launch_decode_tma<64, false>(q, pool, scratch_o, scratch_ml, out, a, n_entries, stream)
                        : launch_decode_tma<128, false>(q, pool, scratch_o, scratch_ml, out, a, n_entries, stream);
}

TIB_API int tib_decode_attention_tma(const void* q, const void* pool, void* out, float* scratch_o, float* scratch_ml,
                                     const int* q_start, const int* kv_start, const int* slots, const int* block_table,
                                     int table_stride, int n_entries, int heads, int kv_heads, int head_dim,
                                     int page_size, int64_t page_stride, int num_pages, int window, float scale,
                                     int num_splits, int chunk, int* counters, int* error_word, cudaStream_t stream) {
  return decode_attention_tma(q, heads * head_dim, pool, out, scratch_o, scratch_ml, q_start, kv_start, slots, block_table,
                              table_stride, n_entries, heads, kv_heads, head_dim, page_size, page_stride, num_pages, window,
                              scale, num_splits, chunk, counters, error_word, false, nullptr, 0, 0, stream);
}

// The same for a step of single tokens whose rotary encoding and cache write have not been done: qkv holds the rows
// of the qkv product, [tokens][(heads + 2 kv_heads) * head_dim], unrotated.  The kernel rotates the queries (rot_dim
// leading dims of a head, pairs (i, i + rot_dim / 2) or, interleaved, (2i, 2i + 1); angle = position * inv_freq[i];
// rot_dim 0: no rotation), and writes each token's rotated key and its value into the token's page before it
// attends.  Every entry must bring exactly one token (entries with more are skipped, and their keys not written).
TIB_API int tib_decode_attention_tma_rope(const void* qkv, void* pool, void* out, float* scratch_o, float* scratch_ml,
                                          const int* q_start, const int* kv_start, const int* slots, const int* block_table,
                                          int table_stride, int n_entries, int heads, int kv_heads, int head_dim,
                                          int page_size, int64_t page_stride, int num_pages, int window, float scale,
                                          int num_splits, int chunk, int* counters, int* error_word, const float* inv_freq,
                                          int rot_dim, int interleaved, cudaStream_t stream) {
  return decode_attention_tma(qkv, (heads + 2 * kv_heads) * head_dim, pool, out, scratch_o, scratch_ml, q_start, kv_start, slots,
                              block_table, table_stride, n_entries, heads, kv_heads, head_dim, page_size, page_stride, num_pages,
                              window, scale, num_splits, chunk, counters, error_word, true, inv_freq, rot_dim, interleaved, stream);
}
