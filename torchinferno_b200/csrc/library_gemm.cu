// The library matrix product (cuBLAS), called from this library instead of through the framework's
// operator: the same kernels at a fraction of the host cost per call, and callable from the native
// layer sequence in block.cu without going back to the interpreter.
//
// cuBLAS is not linked: the process that loads this library has it loaded already (PyTorch brings its
// own copy), so its entry points are looked up at run time (dlopen of the same SONAME returns the copy
// in the process).  One handle per device, made at tib_blas_init, which also hands cuBLAS a workspace
// that the caller owns: with a workspace of its own cuBLAS never allocates inside a stream capture.
//
// The reference sends every projection to this library through F.linear
// (src/torchinferno/models/llama3/pipeline.py:206-208).
#include "common.cuh"
#include <cublas_v2.h>
#include <dlfcn.h>

namespace tib {

constexpr int kBlasError = 20000;   // returned as kBlasError + cublasStatus_t

struct Blas {
  decltype(&cublasCreate_v2) create = nullptr;
  decltype(&cublasSetStream_v2) set_stream = nullptr;
  decltype(&cublasSetWorkspace_v2) set_workspace = nullptr;
  // (the header overloads cublasGemmEx for C++, so its C signature is spelled out)
  cublasStatus_t (*gemm_ex)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*, const void*,
                            cudaDataType, int, const void*, cudaDataType, int, const void*, void*, cudaDataType, int,
                            cublasComputeType_t, cublasGemmAlgo_t) = nullptr;
  bool loaded = false;
  static constexpr int kMaxDevices = 64;
  cublasHandle_t handle[kMaxDevices] = {nullptr};
  void* workspace[kMaxDevices] = {nullptr};
  size_t workspace_bytes[kMaxDevices] = {0};
};

static Blas& blas() {
  static Blas b;
  return b;
}

static int load_blas() {
  Blas& b = blas();
  if (b.loaded) return TIB_OK;
  void* lib = dlopen("libcublas.so.12", RTLD_NOW | RTLD_NOLOAD);
  if (!lib) lib = dlopen("libcublas.so.12", RTLD_NOW);
  if (!lib) lib = dlopen("libcublas.so", RTLD_NOW);
  if (!lib) return TIB_E_ARG;
  b.create = (decltype(b.create))dlsym(lib, "cublasCreate_v2");
  b.set_stream = (decltype(b.set_stream))dlsym(lib, "cublasSetStream_v2");
  b.set_workspace = (decltype(b.set_workspace))dlsym(lib, "cublasSetWorkspace_v2");
  b.gemm_ex = (decltype(b.gemm_ex))dlsym(lib, "cublasGemmEx");
  if (!b.create || !b.set_stream || !b.set_workspace || !b.gemm_ex) return TIB_E_ARG;
  b.loaded = true;
  return TIB_OK;
}

// out[M, N] = x[M, K] . w^T with w stored [N, K] (w_kn == 0) or [K, N] (w_kn == 1); bf16 operands, fp32
// accumulation, out bf16 or fp32.  Row-major operands are the library's column-major ones transposed:
// out^T [N, M] = op(w) [N, K] . x^T [K, M].
int blas_gemm_bf16(const void* x, const void* w, void* out, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo,
                   int w_kn, int out_dtype, cudaStream_t stream) {
  Blas& b = blas();
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= Blas::kMaxDevices || !b.loaded || !b.handle[device]) return TIB_E_ARG;
  cublasHandle_t h = b.handle[device];
  cublasStatus_t st = b.set_stream(h, stream);
  if (st != CUBLAS_STATUS_SUCCESS) return kBlasError + (int)st;
  // (setting the stream resets the workspace to the library's own: hand ours back)
  st = b.set_workspace(h, b.workspace[device], b.workspace_bytes[device]);
  if (st != CUBLAS_STATUS_SUCCESS) return kBlasError + (int)st;
  const float alpha = 1.f, beta = 0.f;
  st = b.gemm_ex(h, w_kn ? CUBLAS_OP_N : CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, w, CUDA_R_16BF, (int)ldw, x, CUDA_R_16BF,
                 (int)ldx, &beta, out, out_dtype == TIB_F32 ? CUDA_R_32F : CUDA_R_16BF, (int)ldo, CUBLAS_COMPUTE_32F,
                 CUBLAS_GEMM_DEFAULT_TENSOR_OP);
  return st == CUBLAS_STATUS_SUCCESS ? TIB_OK : kBlasError + (int)st;
}

}  // namespace tib

using namespace tib;

// Make the handle of the current device and give it `bytes` of device memory at `workspace` (256-byte
// aligned, owned by the caller and kept for as long as products are launched).  Calling it again replaces
// the workspace.
TIB_API int tib_blas_init(void* workspace, size_t bytes) {
  int rc = load_blas();
  if (rc != TIB_OK) return rc;
  if (!workspace || ((uintptr_t)workspace & 255) != 0) return TIB_E_ALIGN;
  Blas& b = blas();
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= Blas::kMaxDevices) return TIB_E_ARG;
  if (!b.handle[device]) {
    cublasStatus_t st = b.create(&b.handle[device]);
    if (st != CUBLAS_STATUS_SUCCESS) return kBlasError + (int)st;
  }
  b.workspace[device] = workspace;
  b.workspace_bytes[device] = bytes;
  return TIB_OK;
}

// x: [M, K] bf16 (row stride ldx), w: [N, K] (w_kn 0) or [K, N] (w_kn 1) bf16 (row stride ldw), out: [M, N]
// bf16 or fp32 (row stride ldo).  tib_blas_init must have been called on this device.
TIB_API int tib_blas_gemm(const void* x, const void* w, void* out, int M, int N, int K, int64_t ldx, int64_t ldw,
                          int64_t ldo, int w_kn, int out_dtype, cudaStream_t stream) {
  if (M == 0 || N == 0) return TIB_OK;
  if (!x || !w || !out || M < 0 || N < 0 || K < 1) return TIB_E_ARG;
  if (out_dtype != TIB_BF16 && out_dtype != TIB_F32) return TIB_E_DTYPE;
  return blas_gemm_bf16(x, w, out, M, N, K, ldx, ldw, ldo, w_kn, out_dtype, stream);
}
