// Shared pieces of the two GEMM kernels (CUDA-core fp32 and tcgen05 bf16).
#pragma once

#include "hx_common.cuh"

namespace hx {
namespace gemm {

enum : int { kEpiNone = 0, kEpiSilu = 1, kEpiSoftplus = 2, kEpiSiluFast = 3, kEpiAccumulate = 4 };  // 4: C += A W^T (fp32 C)

template <int EPI> __device__ __forceinline__ float apply_epilogue(float v) {
    if constexpr (EPI == kEpiSilu) return silu_acc(v);
    else if constexpr (EPI == kEpiSoftplus) return softplus_acc(v);
    else if constexpr (EPI == kEpiSiluFast) return silu_fast(v);
    else return v;
}

// The few-rows kernel (gemm_skinny.cu): M <= 64, K a multiple of 32, operands 16-byte aligned with row strides
// that are multiples of 8 elements.
hx_status launch_skinny(const void *A, int64_t lda, const void *W, int64_t ldw, const float *bias, void *C, int64_t ldc,
                        int c_dtype, int M, int N, int K, int epi, int epi_col0, cudaStream_t st);

// The short-inner-dimension kernel (gemm_lowk.cu): K <= 64 and a multiple of 8, N a multiple of 8, bf16 C with a
// 16-byte aligned base and row stride, no bias, no epilogue.
hx_status launch_lowk(const void *A, int64_t lda, const void *W, int64_t ldw, void *C, int64_t ldc, int M, int N, int K,
                      cudaStream_t st);

hx_status validate_gemm(const void *A, int64_t lda, const void *W, int64_t ldw, void *C, int64_t ldc, int M, int N, int K);

}  // namespace gemm
}  // namespace hx
