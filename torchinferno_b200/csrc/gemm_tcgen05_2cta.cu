// bf16 projections for many rows on pairs of SMs: out[M, N] = x[M, K] . w[N, K]^T with `tcgen05.mma.cta_group::2`.
//
// Two blocks (a cluster of two, on neighbouring SMs) compute one 256 x 256 tile together.  Block r of the pair
// holds rows r * 128 .. of the x slice and rows r * 128 .. of the w slice in its shared memory; one MMA
// instruction, issued by a single thread of the even block, multiplies the pair's 256 x 64 of x by its
// 256 x 64 of w (the tensor cores of the two SMs read the halves of w from each other's shared memory), and
// leaves rows r * 128 .. of the 256-column accumulator in block r's tensor memory.
// Against one block per 128 x 256 tile this halves the shared-memory bytes written and read per flop, which
// is what bounds the one-block kernel in gemm_tcgen05.cu.
//
// Roles per block: warp 0 (one lane) TMA producer into a six-stage ring; warp 1 owns the TMEM allocation and,
// in the even block only, issues the MMAs; warps 2..5 epilogue.  Barriers: `full` lives in the even block and
// collects the bytes of both blocks' copies (the copies name it through the cluster address space); `empty`
// and `acc_full` exist in both blocks and are arrived on together by `tcgen05.commit ... multicast::cluster`;
// `acc_empty` lives in the even block and counts the epilogue warps of both (the odd block arrives remotely).
// Every wait is bounded and reports in `error_word`; no block leaves before its partner is done.  Every copy
// lands in the shared memory of the block that issued it.
//
// The reference sends these products to cuBLAS (src/torchinferno/models/llama3/tensor_parallel.py:11176-11198).
#include "tcgen05.cuh"

namespace tib {

// The tile is 256 rows by BN columns, BN = 256 or 224: with 74 pairs of SMs a shape whose tiles do not fill the
// last round runs that round nearly empty, and the narrower tile can make the rounds come out even (the gate/up
// projection at 2,048 rows: 896 tiles = 12.1 rounds of 256 columns, or 1,024 tiles = 13.8 rounds of 224).
constexpr int kT2BM = 256, kT2BK = 64, kT2Stages = 6;
constexpr int kT2Threads = 192;
constexpr uint32_t kT2ABytes = 128 * kT2BK * 2;                   // this block's rows of x: 16 KB
constexpr uint32_t kT2StageBytes = kT2ABytes + 128 * kT2BK * 2;   // and at most 128 rows of w
constexpr uint32_t kT2SmemBytes = kT2Stages * kT2StageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr int kT2AccStride = 256;                                 // TMEM columns between the two accumulators
// D fp32, A and B bf16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24 (M = 256 over the pair)
constexpr uint32_t t2_idesc(int bn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(kT2BM >> 4) << 24);
}

__device__ __forceinline__ uint32_t t2_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t t2_map(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void t2_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// A tile copy whose completion is counted on a barrier given by its cluster address (the even block's).
__device__ __forceinline__ void t2_tma_load(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void t2_umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive, once the MMAs issued so far are done, on the barrier at this offset in both blocks of the pair.
__device__ __forceinline__ void t2_commit_both(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void t2_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ bool t2_wait_cluster(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 18); ++i) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(1000u) : "memory");
    if (ok) return true;
  }
  return false;
}

// Persistent: pair p walks the tiles t = p, p + pairs, ...; tile t is row tile t % m_tiles of column tile
// t / m_tiles, so pairs that run together share slices of w through the L2.
template <int BN, typename TOut>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kT2Threads, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         TOut* __restrict__ out, int M, int N, int K, int64_t ldo, int* __restrict__ error_word) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + kT2Stages * kT2StageBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kT2Stages + s); };
  auto acc_full_bar = [&](int b) { return bars + 8u * (2 * kT2Stages + b); };
  auto acc_empty_bar = [&](int b) { return bars + 8u * (2 * kT2Stages + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * kT2Stages + 4);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = t2_cluster_rank();                 // 0: the even block of the pair, which issues the MMAs
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int k_blocks = K / kT2BK;
  constexpr uint32_t kBBytes = (BN / 2) * kT2BK * 2;       // this block's rows of w
  const int m_tiles = (M + kT2BM - 1) / kT2BM, n_tiles = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kT2Stages; ++s) {
      mbar_init(full_bar(s), 1);          // (used in the even block: its producer's arrival, plus the bytes of both)
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 8);     // (used in the even block: four epilogue warps of each block)
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tmem_slot), "r"(2u * kT2AccStride) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  t2_cluster_sync();                                       // both blocks have their barriers before either is signalled
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += pairs) {
        const int m0 = (t % m_tiles) * kT2BM + (int)rank * 128, n0 = (t / m_tiles) * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kT2Stages;
          const uint32_t phase = (it / kT2Stages) & 1;
          if (!mbar_wait(empty_bar(s), phase ^ 1)) {
            if (error_word) atomicExch(error_word, 0x7C0041);
            ok = false;
            break;
          }
          if (rank == 0) mbar_expect_tx(full_bar(s), 2 * (kT2ABytes + kBBytes));
          const uint32_t a_dst = base + s * kT2StageBytes, b_dst = a_dst + kT2ABytes;
          const uint32_t bar0 = t2_map(full_bar(s), 0);
          t2_tma_load(a_dst, &map_x, kb * kT2BK, m0, bar0);
          t2_tma_load(b_dst, &map_w, kb * kT2BK, n0, bar0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      uint32_t it = 0;
      bool ok = true;
      int j = 0;
      for (int t = pair; t < num_tiles && ok; t += pairs, ++j) {
        const int b = j & 1;
        const uint32_t tmem_acc = tmem_base + b * kT2AccStride;
        if (!t2_wait_cluster(acc_empty_bar(b), ((j >> 1) & 1) ^ 1)) {   // both epilogues have drained this accumulator
          if (error_word) atomicExch(error_word, 0x7C0044);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kT2Stages;
          const uint32_t phase = (it / kT2Stages) & 1;
          if (!t2_wait_cluster(full_bar(s), phase)) {
            if (error_word) atomicExch(error_word, 0x7C0042);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t a_src = base + s * kT2StageBytes, b_src = a_src + kT2ABytes;
#pragma unroll
          for (int k = 0; k < kT2BK / 16; ++k)
            t2_umma(tmem_acc, umma_desc_k128(a_src + k * 32), umma_desc_k128(b_src + k * 32), t2_idesc(BN), (kb | k) != 0);
          t2_commit_both(empty_bar(s));   // the stage is free in both blocks once these MMAs have read it
        }
        t2_commit_both(acc_full_bar(b));  // (also on failure, so that the epilogues do not wait in vain)
      }
    }
  } else {
    const int quarter = warp & 3;
    int j = 0;
    for (int t = pair; t < num_tiles; t += pairs, ++j) {
      const int m0 = (t % m_tiles) * kT2BM + (int)rank * 128, n0 = (t / m_tiles) * BN;
      const int b = j & 1;
      const int row = m0 + quarter * 32 + lane;
      if (!mbar_wait(acc_full_bar(b), (j >> 1) & 1)) {
        if (error_word && lane == 0) atomicExch(error_word, 0x7C0043);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + b * kT2AccStride + c * 32, v);
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
      // this warp has read its quarter of the accumulator: tell the MMA thread (in the even block)
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) t2_arrive_cluster(t2_map(acc_empty_bar(b), 0));
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  t2_cluster_sync();   // neither block leaves (or frees tensor memory) while its partner may still signal it
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(2u * kT2AccStride) : "memory");
  }
}

static int make_map_2cta(CUtensorMap* map, const void* ptr, int rows, int K, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return TIB_E_ARG;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kT2BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? TIB_OK : TIB_E_ARG;
}

static int t2_pairs() {
  static int pairs = 0;
  if (pairs == 0) {
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    pairs = sms / 2 > 0 ? sms / 2 : 1;
  }
  return pairs;
}

// The tile width whose rounds over the pairs of SMs cost least: rounds x (width + a little for each tile's start).
static int t2_tile_width(int M, int N) {
  const int pairs = t2_pairs(), m_tiles = ceil_div(M, kT2BM);
  const int widths[2] = {256, 224};
  int best = 256;
  long best_cost = -1;
  for (int bn : widths) {
    const long rounds = ceil_div(m_tiles * ceil_div(N, bn), pairs);
    const long cost = rounds * (bn + 16);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

template <int BN, typename TOut>
static int launch_2cta(const void* x, const void* w, void* out, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo,
                       int* error_word, cudaStream_t stream) {
  CUtensorMap map_x, map_w;
  int rc = make_map_2cta(&map_x, x, M, K, ldx, 128);
  if (rc != TIB_OK) return rc;
  rc = make_map_2cta(&map_w, w, N, K, ldw, BN / 2);
  if (rc != TIB_OK) return rc;
  auto kern = gemm_tcgen05_2cta_kernel<BN, TOut>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kT2SmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ceil_div(M, kT2BM) * ceil_div(N, BN);
  const int pairs = tiles < t2_pairs() ? tiles : t2_pairs();
  kern<<<2 * pairs, kT2Threads, kT2SmemBytes, stream>>>(map_x, map_w, (TOut*)out, M, N, K, ldo, error_word);
  TIB_LAUNCH_CHECK();
  return TIB_OK;
}

}  // namespace tib

using namespace tib;

// Whether tib_gemm_tcgen05_2cta takes this shape: K a multiple of 64, N a multiple of 8.
TIB_API int tib_gemm_tcgen05_2cta_supports(int M, int N, int K) {
  return M >= 1 && N >= 8 && N % 8 == 0 && K >= 64 && K % 64 == 0;
}

// x: [M, K] bf16, w: [N, K] bf16, out: [M, N] bf16 or fp32; row strides in elements.
TIB_API int tib_gemm_tcgen05_2cta(const void* x, const void* w, void* out, int M, int N, int K, int64_t ldx, int64_t ldw,
                                  int64_t ldo, int out_dtype, int* error_word, cudaStream_t stream) {
  if (M == 0 || N == 0) return TIB_OK;
  if (!x || !w || !out) return TIB_E_ARG;
  if (!tib_gemm_tcgen05_2cta_supports(M, N, K)) return TIB_E_SIZE;
  if ((((uintptr_t)x | (uintptr_t)w) & 15) || ldx % 8 || ldw % 8) return TIB_E_ALIGN;
  if (out_dtype == TIB_BF16 && ((((uintptr_t)out) & 15) || ldo % 8)) return TIB_E_ALIGN;
  if (out_dtype == TIB_F32 && ((((uintptr_t)out) & 15) || ldo % 4)) return TIB_E_ALIGN;
  if (out_dtype != TIB_BF16 && out_dtype != TIB_F32) return TIB_E_DTYPE;
  const bool wide = t2_tile_width(M, N) == 256;
  if (out_dtype == TIB_BF16)
    return wide ? launch_2cta<256, __nv_bfloat16>(x, w, out, M, N, K, ldx, ldw, ldo, error_word, stream)
                : launch_2cta<224, __nv_bfloat16>(x, w, out, M, N, K, ldx, ldw, ldo, error_word, stream);
  return wide ? launch_2cta<256, float>(x, w, out, M, N, K, ldx, ldw, ldo, error_word, stream)
              : launch_2cta<224, float>(x, w, out, M, N, K, ldx, ldw, ldo, error_word, stream);
}
