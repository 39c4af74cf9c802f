// Causal attention of prompt portions over the paged cache on the 5th-generation tensor cores.
//
// A block owns 128 rows (token, query head of one GQA group) of one kv head and walks the keys in
// tiles of 128 up to the causal edge.  Per tile:
//   S = Q . K^T      `tcgen05.mma` (M 128, N 128, K = head_dim), both operands K-major in 128-byte-
//                    swizzled shared memory, accumulator S in TMEM (128 columns)
//   softmax          eight warps, two threads per row, each with 64 keys of the tile and a running max / sum
//                    (fp32) and an output accumulator of its own: `tcgen05.ld` S, mask, P as bf16 back
//                    into tensor memory over S (the A operand of the next product), O_half in TMEM rescaled
//                    with `tcgen05.ld` / `tcgen05.st` when the row's maximum moved; merged exactly at the end
//   O_h += P_h . V_h `tcgen05.mma` (M 128, N = head_dim, K = 64 keys per half); V is used as it lies in
//                    the cache ([key][head_dim]: an MN-major B operand)
// Warp 0 is the TMA producer of Q (one 3-D tile copy; dims: head_dim, head, token) and of K, the last
// warp that of V, page by page through a 2-D view of the layer's pages ([page rows, head_dim]), each
// into a ring of its own; pages past the block's last query are fetched from an out-of-range
// coordinate, which fills zeros.  Warp 1 (one lane) issues the MMAs.  Every mbarrier wait is bounded; on a timeout a code goes to `error_word`
// and all roles fall through to the common exit.
//
// Formula as in attention_mma.cu / attention_simt.cu (src/torchinferno/models/llama3/raw_ops.py:44-51).
// The reference uses FlashInfer's paged prefill here (src/torchinferno/runtime/paged_serving.py:267-276).
#include "tcgen05.cuh"
#include <math_constants.h>

namespace tib {

constexpr int kFaBM = 128, kFaBN = 128;
constexpr int kFaSoftmaxWarps = 8;                      // two threads per row, each with half the columns
constexpr int kFaThreads = 64 + 32 * kFaSoftmaxWarps + 32;   // key producer, MMA issuer, softmax warps, value producer
constexpr int kFaValueWarp = 2 + kFaSoftmaxWarps;
constexpr int kFaStages = 3;
constexpr float kFaSlack = 8.f;

struct FaArgs {
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
  int skip_single;
  int n_tokens;
  int* error_word;
};

template <int D>
struct FaSmem {
  static constexpr uint32_t kQ = kFaBM * D * 2;          // two sub-tiles of [128 rows][64] when D = 128
  static constexpr uint32_t kKV = kFaBN * D * 2;         // one K or V tile
  static constexpr uint32_t kTotal = 1024 + kQ + kFaStages * 2 * kKV + 256;
};

template <int D>
__global__ void __launch_bounds__(kFaThreads, 1)
prefill_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                                 __nv_bfloat16* __restrict__ out, FaArgs a) {
  using L = FaSmem<D>;
  constexpr int DH = D / 64;                             // 64-wide sub-tiles along head_dim
  constexpr uint32_t kSub = 128 * 64 * 2;                // bytes of one [128][64] sub-tile
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = base;
  auto k_s = [&](int s) { return base + L::kQ + s * 2 * L::kKV; };
  auto v_s = [&](int s) { return base + L::kQ + s * 2 * L::kKV + L::kKV; };
  const uint32_t bars = base + L::kQ + kFaStages * 2 * L::kKV;
  const uint32_t q_full = bars;
  // keys and values have rings of their own: a key stage is free again once S of its tile is computed,
  // long before the values of that tile are used, so the next keys arrive a tile earlier
  auto k_full = [&](int s) { return bars + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bars + 8u * (1 + kFaStages + s); };
  auto v_full = [&](int s) { return bars + 8u * (1 + 2 * kFaStages + s); };
  auto v_empty = [&](int s) { return bars + 8u * (1 + 3 * kFaStages + s); };
  auto s_full = [&](int b) { return bars + 8u * (1 + 4 * kFaStages + b); };
  auto p_full = [&](int b) { return bars + 8u * (3 + 4 * kFaStages + b); };
  const uint32_t pv_done = bars + 8u * (5 + 4 * kFaStages);
  const uint32_t o_final = bars + 8u * (6 + 4 * kFaStages);
  const uint32_t tmem_slot = bars + 8u * (7 + 4 * kFaStages);
  unsigned char* smem_gen = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int entry = blockIdx.y, kvh = blockIdx.x;
  const int row0 = a.q_start[entry];
  const int q_len = a.q_start[entry + 1] - row0;
  const int tok_per_tile = kFaBM / a.group;
  // blocks are handed out x first, z last: with the row tile in z, the longest row tiles of every kv head and
  // request start first and the short ones fill the gaps at the end
  const int tile = gridDim.z - 1 - blockIdx.z;
  const int t0 = tile * tok_per_tile;
  // (uniform exits before any barrier or TMEM use)
  if ((q_len == 1 && a.skip_single) || t0 >= q_len) return;
  const int nt = min(tok_per_tile, q_len - t0);
  const int nrows = nt * a.group;
  const int pos0 = a.kv_start[entry] + t0;
  const int last_pos = pos0 + nt - 1;
  const int first_key = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
  const int kt0 = first_key / kFaBN, kt1 = last_pos / kFaBN;
  const int n_tiles = kt1 - kt0 + 1;
  const int* table = a.block_table + (size_t)a.slots[entry] * a.table_stride;
  constexpr uint32_t kTmemCols = 512;                    // S (two buffers): columns 0..255; O_0, O_1: D columns each from 256

  if (threadIdx.x == 32) {   // (the descriptors are fetched while the barriers are set up)
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_kv) : "memory");
  }
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kFaStages; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full(b), 1);
      mbar_init(p_full(b), 32 * kFaSoftmaxWarps);
    }
    mbar_init(pv_done, 1);
    mbar_init(o_final, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tmem_slot), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_slot_ptr;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 256;   // S buffer b at tmem_s + 128 b

  // Placed early (programmatic dependent launch), the block has set itself up by now; what the kernel before
  // writes (the queries, the newest keys and values) is only touched from here on.
  if (warp != 1) pdl_wait();
  if (warp == 0 || warp == kFaValueWarp) {
    // Two producer warps, one for the keys (and the queries) and one for the values, each with a ring of its
    // own: a copy of one page is one TMA instruction per 64-wide half, and at 16-token pages the issue rate of
    // one warp (about a hundred cycles a box) would otherwise set the pace.  In each, lane 0 waits and arms the
    // barrier, then lane pg looks up page pg of the tile and issues its copies, so the table look-ups of a
    // tile cost one latency.
    const bool values = warp == kFaValueWarp;
    if (!values && lane == 0) {
      // queries: one 3-D box (64 dims, `group` heads, tok_per_tile tokens) per 64-wide half of head_dim
      mbar_expect_tx(q_full, (uint32_t)(tok_per_tile * a.group * D * 2));
#pragma unroll
      for (int h = 0; h < DH; ++h) tma_load_3d(q_s + h * kSub, &map_q, h * 64, kvh * a.group, row0 + t0, q_full);
    }
    const int pages_per_tile = kFaBN >> a.page_shift;
    const int oob_row = a.num_pages * 2 * a.kv_heads * a.page_size;   // first row past the tensor: reads zeros
    for (int it = 0; it < n_tiles; ++it) {
      const int s = it % kFaStages;
      const uint32_t phase = (it / kFaStages) & 1;
      const int key0 = (kt0 + it) * kFaBN;
      // the page id can be fetched while lane 0 waits for the stage
      const int kp = key0 + lane * a.page_size;
      int page = -1;
      if (lane < pages_per_tile && kp <= last_pos && kp + a.page_size > first_key) page = __ldg(table + (kp >> a.page_shift));
      const bool have = page >= 0 && page < a.num_pages;
      const uint32_t off = (uint32_t)(lane * a.page_size) * 128u;        // rows of 128 bytes in a sub-tile
      const uint32_t full = values ? v_full(s) : k_full(s);
      int ok = 1;
      if (lane == 0) {
        ok = mbar_wait(values ? v_empty(s) : k_empty(s), phase ^ 1) ? 1 : 0;
        if (!ok && a.error_word) atomicExch(a.error_word, values ? 0x7C0028 : 0x7C0021);
        if (ok) mbar_expect_tx(full, L::kKV);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < pages_per_tile) {
        const int row = have ? ((page * 2 + (values ? 1 : 0)) * a.kv_heads + kvh) * a.page_size : oob_row;
        const uint32_t dst = (values ? v_s(s) : k_s(s)) + off;
#pragma unroll
        for (int h = 0; h < DH; ++h) tma_load_2d(dst + h * kSub, &map_kv, h * 64, row, full);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kFaBN >> 3) << 17) | ((uint32_t)(kFaBM >> 4) << 24);
      constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) /* B is MN-major */ |
                                   ((uint32_t)(D >> 3) << 17) | ((uint32_t)(kFaBM >> 4) << 24);
      bool ok = mbar_wait(q_full, 0);
      if (!ok && a.error_word) atomicExch(a.error_word, 0x7C0022);
      // O += P . V of tile `j` (its V in stage j % stages, its P in buffer j & 1)
      auto issue_pv = [&](int j) {
        const int s = j % kFaStages;
        if (!mbar_wait(v_full(s), (j / kFaStages) & 1)) {
          if (a.error_word) atomicExch(a.error_word, 0x7C0029);
          return;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < kFaBN / 16; ++kk) {
          // keys 0..63 of the tile go to O_0, keys 64..127 to O_1 (the two halves of a row keep apart); P is
          // read from tensor memory, where each half left it in the first 32 columns of its part of S
          umma_f16_tmem_a(tmem_o + (kk >> 2) * D, tmem_s + (j & 1) * kFaBN + (kk >> 2) * (kFaBN / 2) + (kk & 3) * 8,
                          umma_desc_mn128(v_s(s) + kk * 16 * 128, kSub), idesc_o, (j | (kk & 3)) != 0);
        }
        umma_commit(v_empty(s));    // the value stage goes back to the producer
        umma_commit(pv_done);       // O is at rest again
      };
      for (int it = 0; it < n_tiles && ok; ++it) {
        const int s = it % kFaStages;
        const uint32_t phase = (it / kFaStages) & 1;
        if (!mbar_wait(k_full(s), phase)) {
          if (a.error_word) atomicExch(a.error_word, 0x7C0023);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        // S = Q . K^T over head_dim in steps of 16, into S buffer it & 1: it runs while the softmax warps
        // are still busy with the tile before
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t sub = (kk >> 2) * kSub, inner = (kk & 3) * 32;
          umma_f16_idesc(tmem_s + (it & 1) * kFaBN, umma_desc_k128(q_s + sub + inner), umma_desc_k128(k_s(s) + sub + inner),
                         idesc_s, kk != 0);
        }
        umma_commit(k_empty(s));    // the key stage goes back to the producer
        umma_commit(s_full(it & 1));
        if (it > 0) {
          // P of the tile before (and the rescaled O) are ready: O += P . V
          if (!mbar_wait(p_full((it - 1) & 1), ((it - 1) >> 1) & 1)) {
            if (a.error_word) atomicExch(a.error_word, 0x7C0024);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          issue_pv(it - 1);
        }
      }
      if (ok) {
        const int last = n_tiles - 1;
        if (mbar_wait(p_full(last & 1), (last >> 1) & 1)) {
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          issue_pv(last);
        } else if (a.error_word) {
          atomicExch(a.error_word, 0x7C0024);
        }
      }
      umma_commit(o_final);
    }
  } else {
    // softmax and epilogue: two threads per row.  `half` 0 takes keys 0..63 of every tile, half 1 keys
    // 64..127, each with a running maximum, a sum and an output accumulator (O_half in TMEM) of its own, as
    // if the keys were split between two workers: nothing passes between the two threads of a row until the
    // end, where the two partial results are merged exactly.
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    const int qpos = r < nrows ? pos0 + r / a.group : last_pos;
    constexpr int HC = kFaBN / 2;                          // score columns per thread
    constexpr int OC = D / 2;                              // output columns per thread in the epilogue
    const uint32_t tmem_mine = tmem_o + half * D;          // O_half
    float m = -CUDART_INF_F, l = 0.f;                      // of this half's keys; m in log2 units (scaled)
    bool ok = true;                                        // after a timeout the loop keeps its barriers but does no work
    for (int it = 0; it < n_tiles; ++it) {
      if (ok && !mbar_wait(s_full(it & 1), (it >> 1) & 1)) {
        if (a.error_word && lane == 0) atomicExch(a.error_word, 0x7C0025);
        ok = false;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const int key_base = (kt0 + it) * kFaBN + half * HC;
      const bool need_mask = key_base + HC - 1 > pos0 || (a.window > 0 && key_base < last_pos - a.window + 1);
      if (ok) {
        uint32_t sv[HC];
        {
          uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&sv[0]);
          uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&sv[32]);
          tmem_ld32(tmem_s + lane_sel + (it & 1) * kFaBN + half * HC, lo);
          tmem_ld32(tmem_s + lane_sel + (it & 1) * kFaBN + half * HC + 32, hi);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        }
        float mx = -CUDART_INF_F;
        // two copies of the loop, so that tiles wholly inside the causal triangle pay nothing for the mask
        if (need_mask) {
#pragma unroll
          for (int j = 0; j < HC; ++j) {
            const int key = key_base + j;
            const bool allowed = key <= qpos && (a.window <= 0 || key > qpos - a.window);
            if (!allowed) sv[j] = __float_as_uint(-CUDART_INF_F);
            mx = fmaxf(mx, __uint_as_float(sv[j]));
          }
        } else {
#pragma unroll
          for (int j = 0; j < HC; ++j) mx = fmaxf(mx, __uint_as_float(sv[j]));
        }
        // The running maximum only has to bound the scores loosely: it is moved when a tile exceeds it by more than
        // kFaSlack (in log2 units), so P stays below 2^kFaSlack (fine for bf16 and for the fp32 sums) and the
        // rescaling of O below, with its wait for the product before, becomes rare.  The result is the same
        // quotient either way.  (From -inf any finite maximum is a move; -inf - -inf is NaN and moves nothing.)
        float m_new = fmaxf(m, mx == -CUDART_INF_F ? -CUDART_INF_F : mx * a.scale_log2);
        if (m_new - m <= kFaSlack) m_new = m;
        const float basev = m_new == -CUDART_INF_F ? 0.f : m_new;
        float alpha;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(alpha) : "f"(m - basev));
        m = m_new;
        // O is only touched when some row of the warp moved its maximum; only then must P . V of the tile before
        // be over.  (S of this tile is complete, so every product issued before it is: that of two tiles ago,
        // which read P from the columns written below, among them.)
        const bool rescale = it > 0 && __any_sync(0xffffffffu, alpha != 1.f);
        float sum = 0.f;
        // P (bf16, two keys to a column) goes back into tensor memory over this thread's own part of S: it is
        // the A operand of the next product, and never passes through shared memory
        uint32_t pk[HC / 2];
#pragma unroll
        for (int j = 0; j < HC / 2; ++j) {
          float e0, e1;
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(fmaf(__uint_as_float(sv[2 * j]), a.scale_log2, -basev)));
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(fmaf(__uint_as_float(sv[2 * j + 1]), a.scale_log2, -basev)));
          sum += e0 + e1;
          const __nv_bfloat162 pair = __floats2bfloat162_rn(e0, e1);
          pk[j] = *reinterpret_cast<const uint32_t*>(&pair);
          if (j == HC / 4 - 1) tmem_st16(tmem_s + lane_sel + (it & 1) * kFaBN + half * HC, pk);   // the first half is on its way
        }
        tmem_st16(tmem_s + lane_sel + (it & 1) * kFaBN + half * HC + HC / 4, pk + HC / 4);
        l = l * alpha + sum;
        // O_half of the earlier tiles is scaled to the new maximum, once the P . V of the tile before is done
        if (rescale && !mbar_wait(pv_done, (it - 1) & 1)) {
          if (a.error_word && lane == 0) atomicExch(a.error_word, 0x7C0027);
          ok = false;
        }
        if (ok && rescale) {
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t v[32];
            tmem_ld32(tmem_mine + lane_sel + c * 32, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
            tmem_st32(tmem_mine + lane_sel + c * 32, v);
          }
        }
        asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");   // P (and a rescaled O) are in place
        // values of keys past the block's last query may never have been written: they must not be NaN
        const int tile_base = (kt0 + it) * kFaBN;
        if (tile_base + kFaBN - 1 > last_pos) {
          const int s = it % kFaStages;
          if (!mbar_wait(v_full(s), (it / kFaStages) & 1)) {    // the values must have landed before rows of them are cleared
            if (a.error_word && lane == 0) atomicExch(a.error_word, 0x7C002A);
            ok = false;
          }
          for (int key = max(last_pos + 1, tile_base) + (warp - 2); key < tile_base + kFaBN; key += kFaSoftmaxWarps) {
            const int kr = key - tile_base;
            for (int cb = lane; cb < D / 8; cb += 32)   // 16-byte chunks of the row (all zero, so the swizzle does not matter)
              *reinterpret_cast<uint4*>(smem_gen + (v_s(s) - base) + (cb >> 3) * kSub + kr * 128 + ((cb & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
          }
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // the zeros, before the MMA reads the stage
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      mbar_arrive(p_full(it & 1));
    }
    if (ok && !mbar_wait(o_final, 0)) {
      if (a.error_word && lane == 0) atomicExch(a.error_word, 0x7C0026);
      ok = false;
    }
    // The two halves of a row merge: each passes its (maximum, sum) to the other through the first key stage,
    // which no MMA reads any more, and takes half of the output columns.
    float2* fin = reinterpret_cast<float2*>(smem_gen + (k_s(0) - base));   // [2][128]
    fin[half * 128 + r] = make_float2(m, l);
    asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kFaSoftmaxWarps) : "memory");
    const float2 other = fin[(half ^ 1) * 128 + r];
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const float mm = fmaxf(m, other.x);                  // finite: every row sees at least one key
      const float w_mine = exp2f(m - mm), w_other = exp2f(other.x - mm);
      const float inv = 1.f / (l * w_mine + other.y * w_other);
      const float w0 = (half == 0 ? w_mine : w_other) * inv, w1 = (half == 0 ? w_other : w_mine) * inv;
      const bool store = r < nrows;
      const int t = r / a.group, g = r - t * a.group;
      __nv_bfloat16* dst = out + (size_t)(row0 + t0 + t) * a.heads * D + (kvh * a.group + g) * D + half * OC;
#pragma unroll
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t v0[32], v1[32];
        tmem_ld32(tmem_o + lane_sel + half * OC + c * 32, v0);          // O_0
        tmem_ld32(tmem_o + D + lane_sel + half * OC + c * 32, v1);      // O_1
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        if (store) {
          uint4 packed[4];
          __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(packed);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            p2[j] = __floats2bfloat162_rn(__uint_as_float(v0[2 * j]) * w0 + __uint_as_float(v1[2 * j]) * w1,
                                          __uint_as_float(v0[2 * j + 1]) * w0 + __uint_as_float(v1[2 * j + 1]) * w1);
#pragma unroll
          for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(dst + c * 32)[j] = packed[j];
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

template <int D>
static int launch_fa(const void* q, const void* pool, void* out, FaArgs& a, int n_entries, int max_q_len,
                     int64_t page_stride, cudaStream_t stream) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return TIB_E_ARG;
  const int tok_per_tile = kFaBM / a.group;
  CUtensorMap map_q, map_kv;
  {
    // q: [tokens][heads][D] -> dims (D, heads, tokens); a box is 64 dims x group heads x tok_per_tile tokens
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)a.heads, (cuuint64_t)a.n_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)a.heads * D * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)a.group, (cuuint32_t)tok_per_tile};
    const cuuint32_t elem[3] = {1, 1, 1};
    if (fn(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return TIB_E_ARG;
  }
  {
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
  }
  (void)page_stride;
  auto kern = prefill_attention_tcgen05_kernel<D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FaSmem<D>::kTotal);
  if (e != cudaSuccess) return (int)e;
  const int row_tiles = ceil_div(max_q_len, tok_per_tile);
  if (row_tiles > 65535) return TIB_E_SIZE;
  dim3 grid(a.kv_heads, n_entries, row_tiles);
  TIB_LAUNCH_DEPENDENT(kern, grid, kFaThreads, FaSmem<D>::kTotal, stream, map_q, map_kv, (__nv_bfloat16*)out, a);
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

}  // namespace tib

using namespace tib;

// Whether tib_prefill_attention_tcgen05 takes these sizes: head_dim 64 or 128, a group that divides into
// 128 rows, pages of 8 .. 128 tokens (a power of two), contiguous pages.
TIB_API int tib_prefill_attention_tcgen05_supports(int head_dim, int group, int page_size) {
  const bool pow2 = page_size > 0 && (page_size & (page_size - 1)) == 0;
  return (head_dim == 64 || head_dim == 128) && group >= 1 && group <= 128 && pow2 && page_size >= 8 && page_size <= 128;
}

// Same contract as tib_prefill_attention (bf16).  n_tokens: rows of q / out.  page_stride must equal
// 2 * kv_heads * page_size * head_dim (pages packed back to back).
TIB_API int tib_prefill_attention_tcgen05(const void* q, const void* pool, void* out, const int* q_start,
                                          const int* kv_start, const int* slots, const int* block_table,
                                          int table_stride, int n_entries, int max_q_len, int n_tokens, int heads,
                                          int kv_heads, int head_dim, int page_size, int64_t page_stride, int num_pages,
                                          int window, float scale, int skip_single, int* error_word, cudaStream_t stream) {
  if (n_entries == 0 || max_q_len == 0) return TIB_OK;
  if (!q || !pool || !out || !q_start || !kv_start || !slots || !block_table) return TIB_E_ARG;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads != 0) return TIB_E_SIZE;
  if (!tib_prefill_attention_tcgen05_supports(head_dim, heads / kv_heads, page_size)) return TIB_E_SIZE;
  if (page_stride != (int64_t)2 * kv_heads * page_size * head_dim) return TIB_E_ALIGN;
  if ((((uintptr_t)q | (uintptr_t)pool | (uintptr_t)out) & 15) != 0) return TIB_E_ALIGN;
  if (n_entries > 65535 || kv_heads > 65535) return TIB_E_SIZE;
  FaArgs a;
  a.q_start = q_start; a.kv_start = kv_start; a.slots = slots; a.block_table = block_table;
  a.table_stride = table_stride; a.heads = heads; a.kv_heads = kv_heads; a.group = heads / kv_heads;
  a.page_size = page_size; a.page_shift = 0;
  while ((1 << a.page_shift) < page_size) ++a.page_shift;
  a.num_pages = num_pages; a.window = window; a.scale_log2 = scale * 1.4426950408889634f;
  a.skip_single = skip_single; a.n_tokens = n_tokens; a.error_word = error_word;
  return head_dim == 64 ? launch_fa<64>(q, pool, out, a, n_entries, max_q_len, page_stride, stream)
                        : launch_fa<128>(q, pool, out, a, n_entries, max_q_len, page_stride, stream);
}
