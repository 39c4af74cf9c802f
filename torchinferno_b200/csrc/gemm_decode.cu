// Products of a decode step: out[M, N] = x[M, K] . w with at most 64 rows of x and the weight stored [K, N]
// (the layout the engine keeps under its default backend).  The product is a stream of w, so the kernel is built
// around that stream:
//
//   * w is the 128-row operand of `tcgen05.mma` (MN-major: 64 features of one k are contiguous), the rows of x
//     are its N dimension (padded to 16 .. 64); the accumulator in tensor memory is the transposed output tile
//     (lane = feature, column = row of x).
//   * A block takes tiles of FT = 128 or 256 features (256: two MMAs and two accumulators per k step).  With 256
//     features and all of K per block, a wide matrix (gate/up: 28,672 features) is one tile per block on 112 SMs
//     with 192 KB of weights in flight on each: no rounds of tiles whose last is part empty, no exchange.
//     Narrow matrices (4,096 features) split K over a thread-block cluster of up to 8 blocks whose partial tiles
//     meet in distributed shared memory, as in gemm_tcgen05.cu.
//   * warp 0 / one lane: TMA producer into a ring of stages; it requests its first ring of weights before
//     `griddepcontrol.wait`, while the kernel before this one is still running (the weights do not depend on it).
//     warp 1 / one lane: MMA issue and TMEM ownership.  warps 2..5: epilogue; with tiles of 256 features four such
//     sets of four warps (a warp reaches only its quarter of the lanes of tensor memory, so the sets share the work
//     by accumulator and by odd and even rows): the epilogue is not overlapped with anything when a block has one tile.
//   * Epilogues: plain (bf16 or fp32 rows), or SwiGLU: the matrix holds gate and up columns interleaved
//     (feature 2i = gate i, 2i + 1 = up i), adjacent lanes exchange by shuffle and row i of the activation
//     silu(gate) * up is written directly (src/torchinferno/kernels/triton_ops.py:16-68 is the reference's
//     stand-alone kernel; gate in fp32, silu(g) = g / (1 + exp(-g))).
//
// Every wait is bounded and reports in the error word; TMEM is freed on every path.
// The reference sends these products to the library (src/torchinferno/models/llama3/tensor_parallel.py:11176-11239).
#include "cluster.cuh"

namespace tib {

constexpr int kDgBK = 64;
__host__ __device__ constexpr int dg_epilogue_sets(int ft) { return ft == 256 ? 4 : 1; }
__host__ __device__ constexpr int dg_threads(int ft) { return 64 + 128 * dg_epilogue_sets(ft); }
constexpr int kDgRedRows = 136;                   // splits * ceil(128 / splits) <= 135 for up to 8 splits
enum DecodeEpilogue : int { DG_PLAIN = 0, DG_SWIGLU = 1 };

__host__ __device__ constexpr uint32_t dg_x_bytes(int npad) { return ((uint32_t)npad * kDgBK * 2 + 1023u) & ~1023u; }
__host__ __device__ constexpr uint32_t dg_stage_bytes(int npad, int ft) { return (uint32_t)ft * kDgBK * 2 + dg_x_bytes(npad); }
// Ring depth: 128 features: the depth that streamed fastest with every SM at work (about 18 MB on their way);
// 256 features: what fits (six stages of 34 KB at 16 rows).
__host__ __device__ constexpr int dg_stages(int npad, int ft) {
  return ft == 256 ? (npad <= 16 ? 6 : npad <= 48 ? 5 : 4) : (npad <= 16 ? 7 : npad <= 32 ? 8 : npad <= 48 ? 6 : 5);
}

constexpr int kDgMaxStages = 16;

// kStages: the depth of the ring (1 .. kDgMaxStages), chosen by the host: the depth that streams fastest for a matrix
// that is mostly stream, fewer where the kernel after this one should fit on the SM beside it and fetch ahead (the
// decode attention after the qkv product), more where a block's whole share of a small matrix then fits the ring
// and is on its way before the kernel before this one has ended.
template <int NPAD, int FT, int EPI, typename TOut>
__global__ void __launch_bounds__(dg_threads(FT), 1)
gemm_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   TOut* __restrict__ out, int M, int N, int K, int64_t ldo, int kStages, int* __restrict__ error_word) {
  constexpr int H = FT / 128;                                              // accumulators (and MMAs per k step) of a tile
  constexpr uint32_t kWBytes = (uint32_t)FT * kDgBK * 2;
  constexpr uint32_t kXBytes = NPAD * kDgBK * 2;
  constexpr uint32_t kStage = dg_stage_bytes(NPAD, FT);
  constexpr uint32_t kCols = 2u * H * NPAD;                                // two tiles' accumulators
  constexpr uint32_t kTmemCols = kCols <= 32 ? 32 : kCols <= 64 ? 64 : kCols <= 128 ? 128 : 256;
  constexpr int kRedStride = NPAD + 4;                                     // floats per row of a reduction buffer
  constexpr uint32_t kRedBytes = FT == 128 ? kDgRedRows * kRedStride * 4 : 0;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t red = base + kStages * kStage;                            // 2 x [splits][rows_per][kRedStride] floats
  const uint32_t bars = red + 2 * kRedBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kDgMaxStages + s); };
  auto acc_full_bar = [&](int b) { return bars + 8u * (2 * kDgMaxStages + b); };
  auto acc_empty_bar = [&](int b) { return bars + 8u * (2 * kDgMaxStages + 2 + b); };
  auto red_full_bar = [&](int b) { return bars + 8u * (2 * kDgMaxStages + 4 + b); };   // peers' partial bands have arrived
  auto red_free_bar = [&](int b) { return bars + 8u * (2 * kDgMaxStages + 6 + b); };   // every block has summed its band
  const uint32_t tmem_slot = bars + 8u * (2 * kDgMaxStages + 8);
  unsigned char* smem_gen = smem_raw + (base - smem_u32(smem_raw));        // generic pointer to `base`
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t splits = FT == 128 ? cluster_size() : 1u, rank = FT == 128 ? cluster_rank() : 0u;
  const int cluster_id = blockIdx.x / splits, clusters = gridDim.x / splits;
  const int n_tiles = (N + FT - 1) / FT;
  const int k_blocks = K / kDgBK;
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
      mbar_init(acc_empty_bar(b), 4 * dg_epilogue_sets(FT));   // one arrival per epilogue warp
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
#pragma unroll
    for (int b = 0; b < FT / 64; ++b) tma_load_2d(dst + b * 8192, &map_w, t * FT + b * 64, kb * kDgBK, bar);
  };

  if (warp == 0) {
    if (lane == 0) {
      // The weights do not depend on the kernel before this one, the rows of x do: the first ring of weight
      // tiles is requested at once, and pdl_wait() stands before the first copy of x.
      uint32_t it = 0, ahead = 0;
      bool ok = true;
      for (int t = cluster_id; t < n_tiles && ahead < (uint32_t)kStages; t += clusters)
        for (int kb = kb0; kb < kb1 && ahead < (uint32_t)kStages; ++kb, ++ahead) {
          mbar_expect_tx(full_bar(ahead), kWBytes + kXBytes);
          load_w(base + ahead * kStage, t, kb, full_bar(ahead));
        }
      pdl_wait();
      int s = 0;                 // stage and phase of iteration `it`, counted along (no division in the loop)
      uint32_t phase = 0;
      for (int t = cluster_id; t < n_tiles && ok; t += clusters) {
        for (int kb = kb0; kb < kb1; ++kb, ++it, phase ^= (s + 1 == kStages), s = (s + 1 == kStages ? 0 : s + 1)) {
          const uint32_t w_dst = base + s * kStage, x_dst = w_dst + kWBytes;
          if (it < ahead) {   // (its weights are on their way)
            tma_load_2d(x_dst, &map_x, kb * kDgBK, 0, full_bar(s));
            continue;
          }
          if (!mbar_wait(empty_bar(s), phase ^ 1)) {
            if (error_word) atomicExch(error_word, 0x7C0041);
            ok = false;
            break;
          }
          mbar_expect_tx(full_bar(s), kWBytes + kXBytes);
          load_w(w_dst, t, kb, full_bar(s));
          tma_load_2d(x_dst, &map_x, kb * kDgBK, 0, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // D fp32, A and B bf16, A MN-major (bit 15), B K-major, N = NPAD, M = 128
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((uint32_t)(NPAD >> 3) << 17) |
                                 ((uint32_t)(128 >> 4) << 24);
      bool ok = true;
      int j = 0, s = 0;
      uint32_t phase = 0;
      for (int t = cluster_id; t < n_tiles && ok; t += clusters, ++j) {
        const int b = j & 1;
        if (!mbar_wait(acc_empty_bar(b), ((j >> 1) & 1) ^ 1)) {
          if (error_word) atomicExch(error_word, 0x7C0044);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        for (int kb = kb0; kb < kb1; ++kb, phase ^= (s + 1 == kStages), s = (s + 1 == kStages ? 0 : s + 1)) {
          if (!mbar_wait(full_bar(s), phase)) {
            if (error_word) atomicExch(error_word, 0x7C0042);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t w_src = base + s * kStage, x_src = w_src + kWBytes;
#pragma unroll
          for (int k = 0; k < kDgBK / 16; ++k) {
            const uint64_t bdesc = umma_desc_k128(x_src + k * 32);
#pragma unroll
            for (int h = 0; h < H; ++h)
              umma_f16_idesc(tmem_base + (b * H + h) * NPAD, umma_desc_mn128(w_src + h * 16384 + k * 16 * 128, 8192), bdesc, idesc,
                             (kb > kb0) || (k > 0));
          }
          umma_commit(empty_bar(s));
        }
        umma_commit(acc_full_bar(b));
      }
    }
  } else {
    pdl_wait();                                        // `out` may be memory the kernel before still reads
    const int quarter = warp & 3;
    const int et = threadIdx.x - 64;                   // 0 .. 127 among the epilogue threads (of the one set of FT = 128)
    // this warp's share of a tile: its quarter of the lanes of one accumulator; with four sets (FT = 256), set s takes
    // accumulator s & 1 and the rows of x of parity s >> 1
    constexpr int kSets = dg_epilogue_sets(FT);
    const int set = (warp - 2) >> 2;
    const int h = kSets > 1 ? (set & (H - 1)) : 0;
    const int m_first = kSets > 1 ? set / H : 0;
    constexpr int kRowStep = kSets / H;
    const int first = rank * rows_per;
    const int mine = max(0, min(rows_per, 128 - first));
    int j = 0;
    for (int t = cluster_id; t < n_tiles; t += clusters, ++j) {
      const int b = j & 1;
      const uint32_t par = (j >> 1) & 1;
      float acc[NPAD];
      if (kb1 > kb0) {
        if (!mbar_wait(acc_full_bar(b), par)) {
          if (error_word && lane == 0) atomicExch(error_word, 0x7C0043);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
        for (int c = 0; c < NPAD / 16; ++c) {
          uint32_t v[16];
          tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (b * H + h) * NPAD + c * 16, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
          for (int q = 0; q < 16; ++q) acc[c * 16 + q] = __uint_as_float(v[q]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty_bar(b));   // the MMA warp may reuse this accumulator
      } else {
#pragma unroll
        for (int q = 0; q < NPAD; ++q) acc[q] = 0.f;      // a block without k blocks adds nothing
      }
      if (splits == 1) {
        const int f = t * FT + h * 128 + quarter * 32 + lane;     // feature (column of w)
        if constexpr (EPI == DG_SWIGLU) {
          // even lanes hold gate i, odd lanes up i (i = f / 2): the pair meets by shuffle
#pragma unroll
          for (int mm = 0; mm < NPAD; mm += kRowStep) {
            const int m = mm + m_first;
            if (m >= M) break;                                     // (the same for every lane)
            const float g = kRowStep == 2 && m_first ? acc[mm + kRowStep - 1] : acc[mm];   // (row m, by constant indices)
            const float other = __shfl_xor_sync(0xffffffffu, g, 1);
            const float act = __fdividef(g, 1.0f + __expf(-g)) * other;
            if (!(lane & 1) && f < N) out[(size_t)m * ldo + (f >> 1)] = from_f32<TOut>(act);
          }
        } else {
          if (f < N) {
#pragma unroll
            for (int mm = 0; mm < NPAD; mm += kRowStep) {
              const int m = mm + m_first;
              if (m >= M) break;
              out[(size_t)m * ldo + f] = from_f32<TOut>(kRowStep == 2 && m_first ? acc[mm + kRowStep - 1] : acc[mm]);   // lanes = consecutive features
            }
          }
        }
        continue;
      }
      if constexpr (FT == 128 && EPI == DG_PLAIN) {
        const int f = quarter * 32 + lane;
        const int n0 = t * 128;
        // exchange: this block's partial rows go to the blocks that own them
        if (!mbar_wait_cluster(red_free_bar(b), par ^ 1)) {           // every block is done with buffer b of two tiles ago
          if (error_word && lane == 0) atomicExch(error_word, 0x7C0045);
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
          if (error_word && lane == 0) atomicExch(error_word, 0x7C0046);
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

// Bytes of shared memory a block with a ring of `stages` takes.
template <int NPAD, int FT>
static constexpr uint32_t dg_smem(int stages) {
  return 1024u + (uint32_t)stages * dg_stage_bytes(NPAD, FT) + (FT == 128 ? 2u * kDgRedRows * (NPAD + 4) * 4 : 0u) + 8u * (2 * kDgMaxStages + 10);
}
template <int NPAD, int FT>
static constexpr int dg_most_stages() {
  int n = kDgMaxStages;
  while (n > 1 && dg_smem<NPAD, FT>(n) > 232448u) --n;
  return n;
}

template <int NPAD, int FT, int EPI, typename TOut>
static int launch_decode_gemm(const CUtensorMap& map_w, const CUtensorMap& map_x, void* out, int M, int N, int K, int64_t ldo,
                              int splits, int stages, int* error_word, cudaStream_t stream) {
  constexpr int most = dg_most_stages<NPAD, FT>();
  if (stages <= 0) stages = dg_stages(NPAD, FT);
  if (stages > most) stages = most;
  const uint32_t smem = dg_smem<NPAD, FT>(stages);
  auto kern = gemm_decode_kernel<NPAD, FT, EPI, TOut>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dg_smem<NPAD, FT>(most));
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ceil_div(N, FT);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(dg_threads(FT));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // (see launch_dependent in common.cuh)
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // How many clusters of `splits` blocks can run at once (one block per SM), asked once per size.
  static int resident[9] = {0};
  if (resident[splits] == 0) {
    cfg.numAttrs = 1;
    cfg.dynamicSmemBytes = dg_smem<NPAD, FT>(most);
    cfg.gridDim = dim3((unsigned)splits);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) n = 1;
    resident[splits] = n;
  }
  const int clusters = tiles < resident[splits] ? tiles : resident[splits];
  cfg.dynamicSmemBytes = smem;
  cfg.gridDim = dim3((unsigned)(clusters * splits));
  cfg.numAttrs = dependent_launch_flag() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map_w, map_x, (TOut*)out, M, N, K, ldo, stages, error_word);
  if (e != cudaSuccess) return (int)e;
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

}  // namespace tib

using namespace tib;

// Whether tib_gemm_decode takes this: at most 64 rows, K a multiple of 64, N a multiple of 8 (of 2 x 8 for the SwiGLU
// epilogue, whose output has N / 2 columns); tiles of 128 features with K split over 1..8 blocks, or of 256 features
// unsplit; the SwiGLU epilogue only unsplit.
TIB_API int tib_gemm_decode_supports(int M, int N, int K, int features, int splits, int epilogue) {
  if (!(M >= 1 && M <= 64 && N >= 8 && N % 8 == 0 && K >= 64 && K % 64 == 0)) return 0;
  if (features != 128 && features != 256) return 0;
  if (splits < 1 || splits > 8 || splits > K / kDgBK || (features == 256 && splits != 1)) return 0;
  if (epilogue == DG_SWIGLU) return splits == 1 && N % 16 == 0;
  return epilogue == DG_PLAIN;
}

// x: [M <= 64, K] bf16 (row stride ldx); w: [K, N] bf16 (row stride ldw); out: [M, N] bf16 or fp32, or with the
// SwiGLU epilogue [M, N / 2] (row stride ldo).  features: 128 or 256 per tile; splits: blocks that share K;
// stages: depth of the ring (0: the default for the tile; more than fits is cut to what fits).
TIB_API int tib_gemm_decode(const void* x, const void* w, void* out, int M, int N, int K, int64_t ldx, int64_t ldw,
                            int64_t ldo, int out_dtype, int features, int splits, int epilogue, int stages, int* error_word,
                            cudaStream_t stream) {
  if (M == 0 || N == 0) return TIB_OK;
  if (!x || !w || !out) return TIB_E_ARG;
  if (!tib_gemm_decode_supports(M, N, K, features, splits, epilogue)) return TIB_E_SIZE;
  if ((((uintptr_t)x | (uintptr_t)w) & 15) || ldx % 8 || ldw % 8) return TIB_E_ALIGN;
  if (out_dtype != TIB_BF16 && out_dtype != TIB_F32) return TIB_E_DTYPE;
  if (stages < 0 || stages > kDgMaxStages) return TIB_E_SIZE;
  const int npad = (M + 15) / 16 * 16;
  CUtensorMap map_w, map_x;
  int rc = make_map(&map_w, w, K, N, ldw, 64);
  if (rc != TIB_OK) return rc;
  rc = make_map(&map_x, x, M, K, ldx, npad);
  if (rc != TIB_OK) return rc;
#define TIB_DG_E(NP, FT, T) \
  (epilogue == DG_SWIGLU ? launch_decode_gemm<NP, FT, DG_SWIGLU, T>(map_w, map_x, out, M, N, K, ldo, splits, stages, error_word, stream) \
                         : launch_decode_gemm<NP, FT, DG_PLAIN, T>(map_w, map_x, out, M, N, K, ldo, splits, stages, error_word, stream))
#define TIB_DG_F(NP, T) (features == 256 ? TIB_DG_E(NP, 256, T) : TIB_DG_E(NP, 128, T))
#define TIB_DG(NP) (out_dtype == TIB_BF16 ? TIB_DG_F(NP, __nv_bfloat16) : TIB_DG_F(NP, float))
  switch (npad) {
    case 16: return TIB_DG(16);
    case 32: return TIB_DG(32);
    case 48: return TIB_DG(48);
    default: return TIB_DG(64);
  }
#undef TIB_DG
#undef TIB_DG_F
#undef TIB_DG_E
}
