// Shared pieces of the two GEMM kernels (CUDA-core fp32 and tcgen05 bf16).
#pragma once

#include "hx_common.cuh"

namespace hx {
namespace gemm {

enum : int { kEpiNone = 0, kEpiSilu = 1, kEpiSoftplus = 2 };

template <int EPI> __device__ __forceinline__ float apply_epilogue(float v) {
    if constexpr (EPI == kEpiSilu) return silu_acc(v);
    else if constexpr (EPI == kEpiSoftplus) return softplus_acc(v);
    else return v;
}

hx_status validate_gemm(const void *A, int64_t lda, const void *W, int64_t ldw, void *C, int64_t ldc, int M, int N, int K);

}  // namespace gemm
}  // namespace hx
