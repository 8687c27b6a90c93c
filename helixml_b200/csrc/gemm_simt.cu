// fp32 CUDA-core GEMM: C[M,N] = A[M,K] . W[N,K]^T (+ bias, + activation).  Any alignment, fp32 or
// bf16 operands, fp32 accumulation.  It serves the fp32 (reference-precision) path and the shapes
// too small or too ragged for the tensor-core kernel.
#include "gemm.cuh"

namespace hx {
namespace gemm {

template <typename TA, typename TC, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA *A, int64_t lda, const TA *W, int64_t ldw, const float *bias, TC *C, int64_t ldc, int M, int N,
                 int K) {
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    // each thread loads 4 elements of each tile per k-step: row = tid / 4, k = (tid % 4) * 4 .. +3
    const int lr = threadIdx.x / 4, lk = (threadIdx.x % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int m = m0 + lr, n = n0 + lr;
            As[lk + e][lr] = (m < M && k < K) ? ld_f32(A + (int64_t)m * lda + k) : 0.f;
            Ws[lk + e][lr] = (n < N && k < K) ? ld_f32(W + (int64_t)n * ldw + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j] + (bias ? bias[n] : 0.f);
            v = apply_epilogue<EPI>(v);
            st_f32(C + (int64_t)m * ldc + n, v);
        }
    }
}

template <typename TA, typename TC>
static hx_status launch_simt(const void *A, int64_t lda, const void *W, int64_t ldw, const float *bias, void *C,
                             int64_t ldc, int M, int N, int K, int epi, cudaStream_t st) {
    dim3 grid((N + 63) / 64, (M + 63) / 64), block(256);
    HX_REQUIRE(grid.y <= 65535, HX_ERR_INVALID_DIMENSION, "M %d too large for the SIMT GEMM grid", M);
    auto a = static_cast<const TA *>(A);
    auto w = static_cast<const TA *>(W);
    auto c = static_cast<TC *>(C);
    switch (epi) {
        case kEpiNone: gemm_simt_kernel<TA, TC, kEpiNone><<<grid, block, 0, st>>>(a, lda, w, ldw, bias, c, ldc, M, N, K); break;
        case kEpiSilu: gemm_simt_kernel<TA, TC, kEpiSilu><<<grid, block, 0, st>>>(a, lda, w, ldw, bias, c, ldc, M, N, K); break;
        case kEpiSoftplus: gemm_simt_kernel<TA, TC, kEpiSoftplus><<<grid, block, 0, st>>>(a, lda, w, ldw, bias, c, ldc, M, N, K); break;
        default: return fail(HX_ERR_INVALID_INPUT, "unknown epilogue %d", epi);
    }
    return check_launch("gemm_simt_kernel");
}

hx_status validate_gemm(const void *A, int64_t lda, const void *W, int64_t ldw, void *C, int64_t ldc, int M, int N, int K) {
    HX_REQUIRE(M >= 0 && N >= 0 && K >= 0, HX_ERR_INVALID_DIMENSION, "negative GEMM dimension (%d, %d, %d)", M, N, K);
    if (M == 0 || N == 0) return HX_OK;
    HX_REQUIRE(A && W && C, HX_ERR_INVALID_INPUT, "A, W and C must not be NULL");
    HX_REQUIRE(lda >= K && ldw >= K && ldc >= N, HX_ERR_SHAPE_MISMATCH,
               "leading dimension too small (lda %lld, ldw %lld, ldc %lld for K %d, N %d)", (long long)lda,
               (long long)ldw, (long long)ldc, K, N);
    return HX_OK;
}

}  // namespace gemm
}  // namespace hx

extern "C" hx_status hx_gemm_simt(const void *A, int64_t lda, const void *W, int64_t ldw, const float *bias, void *C,
                                  int64_t ldc, int32_t ab_dtype, int32_t c_dtype, int32_t M, int32_t N, int32_t K,
                                  int32_t epilogue, void *stream) {
    using namespace hx::gemm;
    hx_status s = validate_gemm(A, lda, W, ldw, C, ldc, M, N, K);
    if (s != HX_OK) return s;
    if (M == 0 || N == 0) return HX_OK;
    HX_REQUIRE((ab_dtype == HX_F32 || ab_dtype == HX_BF16) && (c_dtype == HX_F32 || c_dtype == HX_BF16),
               HX_ERR_DTYPE_MISMATCH, "dtype unsupported (ab %d, c %d)", ab_dtype, c_dtype);
    cudaStream_t st = (cudaStream_t)stream;
    const bool ab = ab_dtype == HX_BF16, cb = c_dtype == HX_BF16;
    if (ab && cb) return launch_simt<__nv_bfloat16, __nv_bfloat16>(A, lda, W, ldw, bias, C, ldc, M, N, K, epilogue, st);
    if (ab) return launch_simt<__nv_bfloat16, float>(A, lda, W, ldw, bias, C, ldc, M, N, K, epilogue, st);
    if (cb) return launch_simt<float, __nv_bfloat16>(A, lda, W, ldw, bias, C, ldc, M, N, K, epilogue, st);
    return launch_simt<float, float>(A, lda, W, ldw, bias, C, ldc, M, N, K, epilogue, st);
}
