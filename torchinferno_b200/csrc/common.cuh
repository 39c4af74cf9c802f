// Shared helpers for the engine's CUDA kernels (sm_100a).
//
// Every launcher is an `extern "C"` function that takes raw device pointers,
// sizes and a stream, and returns 0 on success, a positive cudaError_t when the
// launch failed, or a negative TIB_E_* code when it refuses its arguments.
// A refused size is an error, never a wrong result.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TIB_API extern "C" __attribute__((visibility("default")))

// Element types of activations, weights and cache pages.
enum TibDtype : int { TIB_F32 = 0, TIB_BF16 = 1 };

// Argument errors (negative so they cannot collide with cudaError_t).
enum TibError : int {
  TIB_OK = 0,
  TIB_E_DTYPE = -1,      // unknown dtype code
  TIB_E_SIZE = -2,       // a size the kernel does not take
  TIB_E_ALIGN = -3,      // a pointer or stride that is not aligned as required
  TIB_E_SMEM = -4,       // needs more shared memory than an SM offers
  TIB_E_ARG = -5,        // null pointer or inconsistent arguments
  TIB_E_WAIT = -6,       // a bounded device-side wait ran out
  TIB_E_SCRATCH = -7,    // needs more scratch than the library's built-in array holds
};

// The fixed-size record every live request has on the device, one row of int32 words per request slot.
// The host writes a whole record when a request is opened; after that a decode step reads its inputs from it and
// the sampler reads its parameters from it and leaves the drawn token in it, with no host copy in between.
enum TibRequestRecord : int {
  TIB_REC_LENGTH = 0,       // tokens of the request in the cache = position of its next input token
  TIB_REC_LAST_TOKEN = 1,   // its next input token (the one drawn last)
  TIB_REC_SEED_LO = 2,      // sampling seed, low and high half
  TIB_REC_SEED_HI = 3,
  TIB_REC_TEMPERATURE = 4,  // bits of a float; <= 0: greedy
  TIB_REC_DRAWN = 5,        // tokens drawn for the request so far
  TIB_REC_WORDS = 8,        // (two words spare)
};

// kernel<<<grid, block, smem, stream>>>(args) as a programmatic dependent launch (see launch_dependent below)
#define TIB_LAUNCH_DEPENDENT(kernel, grid, block, smem, stream, ...)                                              \
  do {                                                                                                            \
    cudaError_t le__ = tib::launch_dependent(kernel, dim3(grid), dim3(block), (size_t)(smem), stream, __VA_ARGS__); \
    if (le__ != cudaSuccess) return (int)le__;                                                                    \
  } while (0)

#define TIB_LAUNCH_CHECK()                         \
  do {                                             \
    cudaError_t e__ = cudaGetLastError();          \
    if (e__ != cudaSuccess) return (int)e__;       \
  } while (0)

namespace tib {

// The two halves of a bf16 pair as floats, by shift and mask (a bf16 is the upper half of the float it stands for).
// `__bfloat1622float2` compiles to two conversion instructions here, which run on the special-function unit at an
// eighth of the rate: in a kernel that only unpacks, computes a little and packs, that unit was 61 % busy.
__device__ __forceinline__ float2 bf16x2_floats(const __nv_bfloat162 v) {
  const uint32_t u = *reinterpret_cast<const uint32_t*>(&v);
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// One rotated pair of the rotary encoding, with the roundings spelled out so that every kernel that rotates
// (the stand-alone one, and the decode attention kernel that rotates the newest token itself) gives the same bits.
__device__ __forceinline__ float rope_lo(float lo, float hi, float c, float s) { return __fmaf_rn(lo, c, -__fmul_rn(hi, s)); }
__device__ __forceinline__ float rope_hi(float lo, float hi, float c, float s) { return __fmaf_rn(hi, c, __fmul_rn(lo, s)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds at least 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// --- programmatic dependent launch -------------------------------------------------------------
// A kernel launched through launch_dependent() may be placed on the SMs while the kernel before it
// in the stream is still draining; it must call pdl_wait() before it reads anything an earlier
// kernel wrote (or writes anything an earlier kernel reads).  pdl_wait() returns once every kernel
// before it has completed and its writes are visible; in a kernel launched the ordinary way it
// returns at once.  pdl_trigger() lets the kernel after this one be placed early in the same way.
// Every kernel of this library that is launched this way waits first thing, so completion is
// transitive along the stream.  The switch is process-wide (tib_set_dependent_launch).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

inline int& dependent_launch_flag() {
  static int on = 1;
  return on;
}

template <typename... P, typename... A>
static inline cudaError_t launch_dependent(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                           A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr = {};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = dependent_launch_flag() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace tib
