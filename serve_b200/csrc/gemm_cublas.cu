// Library matrix products: out[M,N] = a[M,K] * w[N,K]^T through cuBLAS, which
// is what the reference's nn.Linear layers call (serve/model.py:95-97, 80-82,
// 159). float runs with the pedantic float compute type (no TF32 or other
// reduced-precision mode); bfloat16 inputs accumulate in float and write
// bfloat16 or float.
//
// One handle and one fixed workspace per device, made at the first call on
// that device (make that call before any stream capture).
#include <cublas_v2.h>

#include "common.cuh"

namespace {
constexpr int kMaxDevices = 16;
constexpr size_t kWorkspaceBytes = 64u << 20;
cublasHandle_t g_handle[kMaxDevices];
void* g_workspace[kMaxDevices];
bool g_ready[kMaxDevices];

int ensure_handle(int dev) {
  if (dev < 0 || dev >= kMaxDevices) return SB_ERR_LIMIT;
  if (g_ready[dev]) return 0;
  if (cublasCreate(&g_handle[dev]) != CUBLAS_STATUS_SUCCESS) return -100;
  if (cudaMalloc(&g_workspace[dev], kWorkspaceBytes) != cudaSuccess) return -101;
  if (cublasSetWorkspace(g_handle[dev], g_workspace[dev], kWorkspaceBytes) != CUBLAS_STATUS_SUCCESS) return -102;
  cublasSetMathMode(g_handle[dev], CUBLAS_DEFAULT_MATH);
  g_ready[dev] = true;
  return 0;
}
}  // namespace

SB_EXPORT int sb_linear(const void* a, const void* w, void* out, int M, int N, int K, int in_dtype, int out_dtype,
                        cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return SB_ERR_SHAPE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -103;
  int rc = ensure_handle(dev);
  if (rc) return rc;
  cublasHandle_t h = g_handle[dev];
  if (cublasSetStream(h, stream) != CUBLAS_STATUS_SUCCESS) return -104;
  const float alpha = 1.f, beta = 0.f;
  cudaDataType_t in_t, out_t;
  cublasComputeType_t comp;
  if (in_dtype == SB_DTYPE_F32) {
    if (out_dtype != SB_DTYPE_F32) return SB_ERR_DTYPE;
    in_t = CUDA_R_32F; out_t = CUDA_R_32F; comp = CUBLAS_COMPUTE_32F_PEDANTIC;
  } else if (in_dtype == SB_DTYPE_BF16) {
    in_t = CUDA_R_16BF; comp = CUBLAS_COMPUTE_32F;
    if (out_dtype == SB_DTYPE_BF16) out_t = CUDA_R_16BF;
    else if (out_dtype == SB_DTYPE_F32) out_t = CUDA_R_32F;
    else return SB_ERR_DTYPE;
  } else {
    return SB_ERR_DTYPE;
  }
  // row-major out[M,N] is column-major [N,M]: out^T = w (as op T of col-major [K,N]) * a^T (col-major [K,M])
  cublasStatus_t st = cublasGemmEx(h, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, w, in_t, K, a, in_t, K, &beta, out, out_t, N, comp,
                                   CUBLAS_GEMM_DEFAULT);
  if (st != CUBLAS_STATUS_SUCCESS) return -200 - (int)st;
  return 0;
}
