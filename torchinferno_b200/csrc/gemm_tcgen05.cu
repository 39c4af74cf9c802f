// bf16 projections on the 5th-generation tensor cores: out[M, N] = x[M, K] . w[N, K]^T.
//
// A block computes 128 x 256 tiles of the output, one after the other (one block per SM).  Its warps
// have fixed roles:
//   warp 0, one lane   TMA producer: `cp.async.bulk.tensor.2d` copies a 128 x 64 slice of x and a
//                      256 x 64 slice of w into a ring of 128-byte-swizzled shared-memory stages
//   warp 1, one lane   issues `tcgen05.mma.cta_group::1.kind::f16` (M 128, N 256, K 16) on the stages;
//                      `tcgen05.commit` hands a stage back to the producer and, at the end, the
//                      accumulator to the epilogue.  Warp 1 also owns the TMEM allocation.
//   warps 2..5         epilogue: `tcgen05.ld` reads the fp32 accumulator (TMEM lane = output row,
//                      TMEM column = output column), converts and stores it.
// Full / empty mbarriers order producer, MMA and epilogue; two accumulators in TMEM alternate.  Every wait on an mbarrier is bounded: when
// the limit is reached the waiting role records a code in `error_word`, all roles leave their loops,
// the block still meets at the final barrier and frees its TMEM, and the host raises.
//
// The reference sends these products to cuBLAS (src/torchinferno/models/llama3/tensor_parallel.py:11176-11198).
#include "tcgen05.cuh"
#include "cluster.cuh"

namespace tib {

constexpr int kTcBM = 128, kTcBN = 256, kTcBK = 64, kTcStages = 4;
constexpr int kTcThreads = 192;
constexpr uint32_t kTcStageBytes = (kTcBM + kTcBN) * kTcBK * 2;  // 48 KB
constexpr uint32_t kTcSmemBytes = kTcStages * kTcStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;

// Instruction descriptor: D fp32, A and B bf16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTcBN >> 3) << 17) | ((uint32_t)(kTcBM >> 4) << 24);

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate) : "memory");
}
// Persistent: a block walks the tiles t = blockIdx.x, blockIdx.x + gridDim.x, ...  Tile t is row tile
// t % m_tiles of column tile t / m_tiles, so blocks that run together share slices of w (the big
// operand), which then come from HBM once and from L2 for the other row tiles.  Two accumulators
// (2 x 256 TMEM columns) alternate, so the epilogue of one tile runs under the MMAs of the next.
template <typename TOut>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    TOut* __restrict__ out, int M, int N, int K, int64_t ldo, int* __restrict__ error_word) {
  extern __shared__ unsigned char smem_raw[];
  // stages must start on 1024-byte boundaries (128-byte swizzle repeats every 8 rows of 128 bytes)
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + kTcStages * kTcStageBytes;       // full[4], empty[4], acc_full[2], acc_empty[2], tmem slot
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kTcStages + s); };
  auto acc_full_bar = [&](int b) { return bars + 8u * (2 * kTcStages + b); };
  auto acc_empty_bar = [&](int b) { return bars + 8u * (2 * kTcStages + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * kTcStages + 4);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = K / kTcBK;
  const int m_tiles = (M + kTcBM - 1) / kTcBM, n_tiles = (N + kTcBN - 1) / kTcBN;
  const int num_tiles = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 4);   // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tmem_slot), "r"(2u * kTcBN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;   // k blocks issued so far: picks the stage and its phase
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m0 = (t % m_tiles) * kTcBM, n0 = (t / m_tiles) * kTcBN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kTcStages;
          const uint32_t phase = (it / kTcStages) & 1;
          if (!mbar_wait(empty_bar(s), phase ^ 1)) {
            if (error_word) atomicExch(error_word, 0x7C0001);
            ok = false;
            break;
          }
          mbar_expect_tx(full_bar(s), kTcStageBytes);
          const uint32_t a_dst = base + s * kTcStageBytes, b_dst = a_dst + kTcBM * kTcBK * 2;
          tma_load_2d(a_dst, &map_x, kb * kTcBK, m0, full_bar(s));
          tma_load_2d(b_dst, &map_w, kb * kTcBK, n0, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      int j = 0;         // tiles done by this block: picks the accumulator and its phase
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++j) {
        const int b = j & 1;
        const uint32_t tmem_acc = tmem_base + b * kTcBN;
        if (!mbar_wait(acc_empty_bar(b), ((j >> 1) & 1) ^ 1)) {   // the epilogue has drained this accumulator
          if (error_word) atomicExch(error_word, 0x7C0004);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kTcStages;
          const uint32_t phase = (it / kTcStages) & 1;
          if (!mbar_wait(full_bar(s), phase)) {
            if (error_word) atomicExch(error_word, 0x7C0002);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t a_src = base + s * kTcStageBytes, b_src = a_src + kTcBM * kTcBK * 2;
#pragma unroll
          for (int k = 0; k < kTcBK / 16; ++k) {
            // 16 bf16 = 32 bytes further along K inside the 128-byte swizzle atom
            umma_f16(tmem_acc, umma_desc_k128(a_src + k * 32), umma_desc_k128(b_src + k * 32), (kb | k) != 0);
          }
          umma_commit(empty_bar(s));   // the stage is free once these MMAs have read it
        }
        umma_commit(acc_full_bar(b));  // (also on failure, so that the epilogue does not wait in vain)
      }
    }
  } else {
    // epilogue: warp w may touch TMEM lanes 32 * (w % 4) .. + 31
    const int quarter = warp & 3;
    int j = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++j) {
      const int m0 = (t % m_tiles) * kTcBM, n0 = (t / m_tiles) * kTcBN;
      const int b = j & 1;
      const int row = m0 + quarter * 32 + lane;
      if (!mbar_wait(acc_full_bar(b), (j >> 1) & 1)) {
        if (error_word && lane == 0) atomicExch(error_word, 0x7C0003);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
      for (int c = 0; c < kTcBN / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + b * kTcBN + c * 32, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        const int col = n0 + c * 32;
        if (row < M && col < N) {
          TOut* dst = out + (size_t)row * ldo + col;
          if (col + 32 <= N) {
            if constexpr (sizeof(TOut) == 2) {
              uint4 packed[4];
              __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(packed);
#pragma unroll
              for (int q = 0; q < 16; ++q) p2[q] = __floats2bfloat162_rn(__uint_as_float(v[2 * q]), __uint_as_float(v[2 * q + 1]));
#pragma unroll
              for (int q = 0; q < 4; ++q) reinterpret_cast<uint4*>(dst)[q] = packed[q];
            } else {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                reinterpret_cast<uint4*>(dst)[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            }
          } else {
            for (int q = 0; q < 32 && col + q < N; ++q) dst[q] = from_f32<TOut>(__uint_as_float(v[q]));
          }
        }
      }
      // this warp has read its quarter of the accumulator: hand it back to the MMA warp
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(b));
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(2u * kTcBN) : "memory");
  }
}

// ------------------------------------------------------------------ few rows (decode): swap A and B
// With at most 64 rows of x the product is a stream of w.  Here w is the 128-row operand of the MMA
// (a tile of 128 output features) and the rows of x are its N dimension (padded to 16 .. 64), so the
// accumulator is the transposed output tile: TMEM lane = feature, column = token.
//
// The kernel is persistent: `clusters` thread-block clusters of `splits` blocks (one block per SM) walk
// the feature tiles; block r of a cluster streams the r-th part of K of every tile its cluster takes.
// The producer runs ahead across tiles, two accumulators alternate, and the partial tiles of a cluster
// meet in distributed shared memory: every block owns a band of the 128 features, receives that band
// from its peers with st.shared::cluster, sums it and stores it.  The hand-over is done with mbarriers
// that peers arrive on remotely, so only the epilogue warps take part.  No scratch in global memory,
// no second kernel.
constexpr uint32_t kSwWBytes = 128 * kTcBK * 2;   // 16 KB of w per stage
constexpr int kSwRedRows = 136;                   // splits * ceil(128 / splits) <= 135 for up to 8 splits
// Stages of the w / x ring.  More bytes in flight are not better: with every SM streaming, about 16 to 20 MB on
// their way (6 to 8 stages of 18 KB on each of 135 to 148 SMs) stream fastest; with 11 stages the same loop was
// 5 % slower, with 3 stages 15 %.  (At more rows a stage is larger and fewer fit.)
constexpr int sw_stages(int npad) { return npad <= 16 ? 7 : npad <= 32 ? 8 : npad <= 48 ? 6 : 5; }

// NPAD: rows of x padded to a multiple of 16 (16, 32, 48 or 64).  WKN: w is stored [K, N] (the layout the library
// prefers at few rows), so a slice of it is an MN-major A operand: two boxes of 64 features x 64 k.
template <int NPAD, typename TOut, bool WKN>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tcgen05_swapab_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                           TOut* __restrict__ out, int M, int N, int K, int64_t ldo, int* __restrict__ error_word) {
  constexpr int kStages = sw_stages(NPAD);
  constexpr uint32_t kXBytes = NPAD * kTcBK * 2;
  constexpr uint32_t kStage = kSwWBytes + ((kXBytes + 1023u) & ~1023u);   // both parts start on 1024-byte boundaries
  constexpr uint32_t kTmemCols = NPAD <= 16 ? 32 : NPAD <= 32 ? 64 : 128;  // two accumulators of NPAD columns
  constexpr int kRedStride = NPAD + 4;                                     // floats per row of a reduction buffer
  constexpr uint32_t kRedBytes = kSwRedRows * kRedStride * 4;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t red = base + kStages * kStage;                            // 2 x [splits][rows_per][kRedStride] floats
  const uint32_t bars = red + 2 * kRedBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kStages + s); };
  auto acc_full_bar = [&](int b) { return bars + 8u * (2 * kStages + b); };
  auto acc_empty_bar = [&](int b) { return bars + 8u * (2 * kStages + 2 + b); };
  auto red_full_bar = [&](int b) { return bars + 8u * (2 * kStages + 4 + b); };   // peers' partial bands have arrived
  auto red_free_bar = [&](int b) { return bars + 8u * (2 * kStages + 6 + b); };   // every block has summed its band
  const uint32_t tmem_slot = bars + 8u * (2 * kStages + 8);
  unsigned char* smem_gen = smem_raw + (base - smem_u32(smem_raw));        // generic pointer to `base`
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t splits = cluster_size(), rank = cluster_rank();
  const int cluster_id = blockIdx.x / splits, clusters = gridDim.x / splits;
  const int n_tiles = (N + 127) / 128;
  const int k_blocks = K / kTcBK;
  const int kb0 = (int)((int64_t)k_blocks * rank / splits), kb1 = (int)((int64_t)k_blocks * (rank + 1) / splits);
  const int rows_per = (128 + splits - 1) / splits;                        // features each block of the cluster owns

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 4);           // one arrival per epilogue warp
      mbar_init(red_full_bar(b), 4 * splits);   // one arrival per epilogue warp of every block of the cluster
      mbar_init(red_free_bar(b), 4 * splits);   // likewise, once they have summed their share of the band
    }
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
  if (splits > 1) cluster_sync_all();   // every block of the cluster runs and has its barriers: peers may touch them
  auto load_w = [&](uint32_t dst, int t, int kb, uint32_t bar) {
    if constexpr (WKN) {
      tma_load_2d(dst, &map_w, t * 128, kb * kTcBK, bar);
      tma_load_2d(dst + kSwWBytes / 2, &map_w, t * 128 + 64, kb * kTcBK, bar);
    } else {
      tma_load_2d(dst, &map_w, kb * kTcBK, t * 128, bar);
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      // The weights do not depend on the kernel before this one, the rows of x do: the first ring of weight
      // tiles is requested at once, and pdl_wait() stands before the first copy of x.
      uint32_t it = 0, ahead = 0;
      bool ok = true;
      for (int t = cluster_id; t < n_tiles && ahead < (uint32_t)kStages; t += clusters)
        for (int kb = kb0; kb < kb1 && ahead < (uint32_t)kStages; ++kb, ++ahead) {
          mbar_expect_tx(full_bar(ahead), kSwWBytes + kXBytes);
          load_w(base + ahead * kStage, t, kb, full_bar(ahead));
        }
      pdl_wait();
      for (int t = cluster_id; t < n_tiles && ok; t += clusters) {
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1;
          const uint32_t w_dst = base + s * kStage, x_dst = w_dst + kSwWBytes;
          if (it < ahead) {   // (its weights are on their way)
            tma_load_2d(x_dst, &map_x, kb * kTcBK, 0, full_bar(s));
            continue;
          }
          if (!mbar_wait(empty_bar(s), phase ^ 1)) {
            if (error_word) atomicExch(error_word, 0x7C0011);
            ok = false;
            break;
          }
          mbar_expect_tx(full_bar(s), kSwWBytes + kXBytes);
          load_w(w_dst, t, kb, full_bar(s));
          tma_load_2d(x_dst, &map_x, kb * kTcBK, 0, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // (bit 15: the A operand is MN-major)
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (WKN ? (1u << 15) : 0u) | ((uint32_t)(NPAD >> 3) << 17) |
                                 ((uint32_t)(128 >> 4) << 24);
      uint32_t it = 0;
      bool ok = true;
      int j = 0;
      for (int t = cluster_id; t < n_tiles && ok; t += clusters, ++j) {
        const int b = j & 1;
        if (!mbar_wait(acc_empty_bar(b), ((j >> 1) & 1) ^ 1)) {
          if (error_word) atomicExch(error_word, 0x7C0014);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1;
          if (!mbar_wait(full_bar(s), phase)) {
            if (error_word) atomicExch(error_word, 0x7C0012);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t w_src = base + s * kStage, x_src = w_src + kSwWBytes;
#pragma unroll
          for (int k = 0; k < kTcBK / 16; ++k) {
            const uint64_t adesc = WKN ? umma_desc_mn128(w_src + k * 16 * 128, kSwWBytes / 2) : umma_desc_k128(w_src + k * 32);
            umma_f16_idesc(tmem_base + b * NPAD, adesc, umma_desc_k128(x_src + k * 32), idesc, (kb > kb0) || (k > 0));
          }
          umma_commit(empty_bar(s));
        }
        umma_commit(acc_full_bar(b));
      }
    }
  } else {
    pdl_wait();                                        // `out` may be memory the kernel before still reads
    const int quarter = warp & 3;
    const int f = quarter * 32 + lane;                 // feature (row of w) within the tile
    const int et = threadIdx.x - 64;                   // 0 .. 127 among the epilogue threads
    const int first = rank * rows_per;
    const int mine = max(0, min(rows_per, 128 - first));
    int j = 0;
    for (int t = cluster_id; t < n_tiles; t += clusters, ++j) {
      const int b = j & 1;
      const uint32_t par = (j >> 1) & 1;
      const int n0 = t * 128;
      float acc[NPAD];
      if (kb1 > kb0) {
        if (!mbar_wait(acc_full_bar(b), par)) {
          if (error_word && lane == 0) atomicExch(error_word, 0x7C0013);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
        for (int c = 0; c < NPAD / 16; ++c) {
          uint32_t v[16];
          tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + b * NPAD + c * 16, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
          for (int q = 0; q < 16; ++q) acc[c * 16 + q] = __uint_as_float(v[q]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty_bar(b));   // the MMA warp may reuse this accumulator
      } else {
#pragma unroll
        for (int q = 0; q < NPAD; ++q) acc[q] = 0.f;    // a block without k blocks adds nothing
      }
      if (splits == 1) {
        if (n0 + f < N) {
#pragma unroll
          for (int m = 0; m < NPAD; ++m)
            if (m < M) out[(size_t)m * ldo + n0 + f] = from_f32<TOut>(acc[m]);   // lanes = consecutive features
        }
        continue;
      }
      // exchange: this block's partial rows go to the blocks that own them
      if (!mbar_wait_cluster(red_free_bar(b), par ^ 1)) {           // every block is done with buffer b of two tiles ago
        if (error_word && lane == 0) atomicExch(error_word, 0x7C0015);
        break;
      }
      const uint32_t red_b = red + b * kRedBytes;
      {
        const uint32_t owner = f / rows_per, local = f - owner * rows_per;
        const uint32_t dst = map_to_cta(red_b + ((rank * rows_per + local) * kRedStride) * 4, owner);
#pragma unroll
        for (int q = 0; q < NPAD; q += 4) st_cluster_f32x4(dst + q * 4, acc[q], acc[q + 1], acc[q + 2], acc[q + 3]);
      }
      __syncwarp();
      if (lane < splits) mbar_arrive_remote(map_to_cta(red_full_bar(b), lane));   // this warp's rows are written, everywhere
      if (!mbar_wait_cluster(red_full_bar(b), par)) {
        if (error_word && lane == 0) atomicExch(error_word, 0x7C0016);
        break;
      }
      const float* red_gen = reinterpret_cast<const float*>(smem_gen + (red_b - base));
      for (int idx = et; idx < mine * M; idx += 128) {
        const int m = idx / mine, lr = idx - m * mine;   // consecutive threads = consecutive features
        float sum = 0.f;
        for (uint32_t sp = 0; sp < splits; ++sp) sum += red_gen[(sp * rows_per + lr) * kRedStride + m];
        if (n0 + first + lr < N) out[(size_t)m * ldo + n0 + first + lr] = from_f32<TOut>(sum);
      }
      // this warp has read its share of the band: tell every block (this one included)
      __syncwarp();
      if (lane < splits) mbar_arrive_remote(map_to_cta(red_free_bar(b), lane));
    }
  }
  __syncwarp();
  if (splits > 1) cluster_sync_all();   // no block leaves while a peer may still write to it or arrive on its barriers
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------ host side
}  // namespace tib

using namespace tib;

// Whether tib_gemm_tcgen05 takes this shape: K a multiple of 64, N a multiple of 8.
TIB_API int tib_gemm_tcgen05_supports(int M, int N, int K) {
  return M >= 1 && N >= 8 && N % 8 == 0 && K >= 64 && K % 64 == 0;
}

template <int NPAD, typename TOut, bool WKN>
static int launch_swapab(const CUtensorMap& map_w, const CUtensorMap& map_x, void* out, int M, int N, int K, int64_t ldo,
                         int splits, int* error_word, cudaStream_t stream) {
  constexpr uint32_t x_bytes = NPAD * kTcBK * 2;
  constexpr uint32_t stage = kSwWBytes + ((x_bytes + 1023u) & ~1023u);
  constexpr uint32_t smem = 1024 + sw_stages(NPAD) * stage + 2 * kSwRedRows * (NPAD + 4) * 4 + 256;
  auto kern = gemm_tcgen05_swapab_kernel<NPAD, TOut, WKN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ceil_div(N, 128), k_blocks = K / kTcBK;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // (see launch_dependent in common.cuh)
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // How many clusters of s blocks can run at once (one block per SM), asked once per s.
  static int resident[9] = {0};
  auto clusters_of = [&](int s) {
    if (resident[s] == 0) {
      attr[0].val.clusterDim.x = (unsigned)s;
      cfg.gridDim = dim3((unsigned)s);
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) n = 1;
      resident[s] = n;
    }
    return resident[s];
  };
  if (splits <= 0) {
    // Every block streams tile_bytes / s of each tile its cluster takes; the clusters take the tiles in
    // rounds.  Fewest rounds x bytes per round wins; a split costs a little for the exchange.
    double best = 1e30;
    splits = 1;
    for (int s = 1; s <= 8 && (s == 1 || s * 2 <= k_blocks); ++s) {
      const int rounds = ceil_div(tiles, clusters_of(s));
      const double cost = rounds * (1.0 / s + 0.02) + (s > 1 ? 0.03 : 0.0);
      if (cost < best - 1e-12) {
        best = cost;
        splits = s;
      }
    }
  }
  if (splits > 8 || splits > k_blocks) return TIB_E_SIZE;
  const int clusters = tiles < clusters_of(splits) ? tiles : clusters_of(splits);
  attr[0].val.clusterDim.x = (unsigned)splits;
  cfg.gridDim = dim3((unsigned)(clusters * splits));
  cfg.numAttrs = dependent_launch_flag() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map_w, map_x, (TOut*)out, M, N, K, ldo, error_word);
  if (e != cudaSuccess) return (int)e;
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

// Whether tib_gemm_tcgen05_swapab takes this shape: at most 64 rows, K a multiple of 64, N a multiple of 8.
TIB_API int tib_gemm_tcgen05_swapab_supports(int M, int N, int K) {
  return M >= 1 && M <= 64 && N >= 8 && N % 8 == 0 && K >= 64 && K % 64 == 0;
}

// Few rows (decode): x: [M <= 64, K] bf16, w: [N, K] (w_kn 0) or [K, N] (w_kn 1) bf16, out: [M, N] bf16 or fp32.
// splits: 0 lets the library choose how many blocks share K (1..8), else that many.
TIB_API int tib_gemm_tcgen05_swapab(const void* x, const void* w, void* out, int M, int N, int K, int64_t ldx,
                                    int64_t ldw, int64_t ldo, int w_kn, int out_dtype, int splits, int* error_word,
                                    cudaStream_t stream) {
  if (M == 0 || N == 0) return TIB_OK;
  if (!x || !w || !out) return TIB_E_ARG;
  if (!tib_gemm_tcgen05_swapab_supports(M, N, K)) return TIB_E_SIZE;
  if ((((uintptr_t)x | (uintptr_t)w) & 15) || ldx % 8 || ldw % 8) return TIB_E_ALIGN;
  if (out_dtype != TIB_BF16 && out_dtype != TIB_F32) return TIB_E_DTYPE;
  const int npad = (M + 15) / 16 * 16;
  if (splits > 8 || splits > K / kTcBK) return TIB_E_SIZE;
  CUtensorMap map_w, map_x;
  int rc = w_kn ? make_map(&map_w, w, K, N, ldw, 64) : make_map(&map_w, w, N, K, ldw, 128);
  if (rc != TIB_OK) return rc;
  rc = make_map(&map_x, x, M, K, ldx, npad);
  if (rc != TIB_OK) return rc;
#define TIB_SWAPAB_T(NP, T) \
  (w_kn ? launch_swapab<NP, T, true>(map_w, map_x, out, M, N, K, ldo, splits, error_word, stream) \
        : launch_swapab<NP, T, false>(map_w, map_x, out, M, N, K, ldo, splits, error_word, stream))
#define TIB_SWAPAB(NP) (out_dtype == TIB_BF16 ? TIB_SWAPAB_T(NP, __nv_bfloat16) : TIB_SWAPAB_T(NP, float))
  switch (npad) {
    case 16: return TIB_SWAPAB(16);
    case 32: return TIB_SWAPAB(32);
    case 48: return TIB_SWAPAB(48);
    default: return TIB_SWAPAB(64);
  }
#undef TIB_SWAPAB
#undef TIB_SWAPAB_T
}

// x: [M, K] bf16 (row stride ldx), w: [N, K] bf16 (row stride ldw), out: [M, N] bf16 or fp32 (row stride ldo).
// Base addresses and row strides must be multiples of 16 bytes.  error_word (device, optional) receives a
// non-zero code if a bounded wait inside the kernel ran out.
TIB_API int tib_gemm_tcgen05(const void* x, const void* w, void* out, int M, int N, int K, int64_t ldx, int64_t ldw,
                             int64_t ldo, int out_dtype, int* error_word, cudaStream_t stream) {
  if (M == 0 || N == 0) return TIB_OK;
  if (!x || !w || !out) return TIB_E_ARG;
  if (!tib_gemm_tcgen05_supports(M, N, K)) return TIB_E_SIZE;
  if ((((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) || ldx % 8 || ldw % 8 || ldo % 8) return TIB_E_ALIGN;
  CUtensorMap map_x, map_w;
  int rc = make_map(&map_x, x, M, K, ldx, kTcBM);
  if (rc != TIB_OK) return rc;
  rc = make_map(&map_w, w, N, K, ldw, kTcBN);
  if (rc != TIB_OK) return rc;
  const int64_t tiles = (int64_t)ceil_div(M, kTcBM) * ceil_div(N, kTcBN);
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return TIB_E_ARG;
  if (tiles > 0x7fffffff) return TIB_E_SIZE;
  dim3 grid((unsigned)(tiles < sms ? tiles : sms));
  cudaError_t e;
  if (out_dtype == TIB_BF16) {
    auto kern = gemm_tcgen05_kernel<__nv_bfloat16>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemBytes);
    if (e != cudaSuccess) return (int)e;
    kern<<<grid, kTcThreads, kTcSmemBytes, stream>>>(map_x, map_w, (__nv_bfloat16*)out, M, N, K, ldo, error_word);
  } else if (out_dtype == TIB_F32) {
    auto kern = gemm_tcgen05_kernel<float>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemBytes);
    if (e != cudaSuccess) return (int)e;
    kern<<<grid, kTcThreads, kTcSmemBytes, stream>>>(map_x, map_w, (float*)out, M, N, K, ldo, error_word);
  } else {
    return TIB_E_DTYPE;
  }
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}
