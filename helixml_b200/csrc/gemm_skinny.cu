// gemm_skinny_kernel: C[M,N] = A[M,K] . W[N,K]^T for a handful of rows (M <= 64), the shape of a decode step.
// With so few rows the GEMM is a stream over the weights: every byte of W is needed once and nothing is
// reused, so the persistent tcgen05 kernel (one 128-row tile, one CTA per 256 columns) spends its time in
// set-up, and what matters is how many weight bytes are in flight.  A CTA owns 8 output columns; its 16 warps
// split K in blocks of 32 (round-robin), each warp runs mma.sync.m16n8k16 (bf16 in, fp32 accumulate) over its
// blocks with all of its loads issued up front, and the 16 partial tiles are summed through shared memory.
// The grid is N/8 CTAs, so every SM streams a slice of W and the whole kernel is about one memory round trip.
//
// Operand loads are 16 bytes per lane.  The MMA does not care in which order the k indices are presented as
// long as A and B agree, so inside a block of 32 k values lane (g, tid) loads the 8 consecutive elements
// k = 8 tid .. 8 tid + 7 of its row and uses them as the two k-halves of two MMAs:
//   MMA j (j = 0, 1): "k pair 2 tid" = elements 4 j + {0, 1}, "k pair 2 tid + 8" = elements 4 j + {2, 3}.
// A comes straight from global memory (it is M x K, a few tens of KB, shared by every CTA through L2/L1).
#include "gemm.cuh"

namespace hx {
namespace gemm {

constexpr int kSkinnyWarps = 16;

template <int MT, typename TC, int EPI>
__global__ void __launch_bounds__(kSkinnyWarps * 32)
gemm_skinny_kernel(const __nv_bfloat16 *__restrict__ A, int64_t lda, const __nv_bfloat16 *__restrict__ W, int64_t ldw,
                   const float *__restrict__ bias, TC *__restrict__ C, int64_t ldc, int M, int N, int K, int epi_col0) {
    __shared__ float partial[kSkinnyWarps * MT * 128];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tid = lane & 3;
    const int n0 = blockIdx.x * 8;
    const int n = n0 + g;                                   // the W row this lane loads
    const bool n_ok = n < N;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    const __nv_bfloat16 *wrow = W + (int64_t)(n_ok ? n : 0) * ldw + tid * 8;
    const __nv_bfloat16 *arow[MT][2];
    bool a_ok[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = mt * 16 + h * 8 + g;
            a_ok[mt][h] = r < M;
            arow[mt][h] = A + (int64_t)(a_ok[mt][h] ? r : 0) * lda + tid * 8;
        }
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;

    // this warp's k-blocks: warp, warp + 16, ... ; two blocks per trip so that their loads overlap
    for (int k0 = warp * 32; k0 < K; k0 += kSkinnyWarps * 64) {
        uint4 b[2], a[2][MT][2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int k = k0 + u * kSkinnyWarps * 32;
            const bool k_ok = k < K;
            b[u] = (n_ok && k_ok) ? *reinterpret_cast<const uint4 *>(wrow + k) : zero4;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    a[u][mt][h] = (a_ok[mt][h] && k_ok) ? *reinterpret_cast<const uint4 *>(arow[mt][h] + k) : zero4;
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                // fragment registers: a0 = (row g, k pair), a1 = (row g+8, k pair), a2 = (row g, k pair + 8), a3 = (row g+8, ...)
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                             "{%0, %1, %2, %3};"
                             : "+f"(acc[mt][0]), "+f"(acc[mt][1]), "+f"(acc[mt][2]), "+f"(acc[mt][3])
                             : "r"(a[u][mt][0].x), "r"(a[u][mt][1].x), "r"(a[u][mt][0].y), "r"(a[u][mt][1].y), "r"(b[u].x), "r"(b[u].y));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                             "{%0, %1, %2, %3};"
                             : "+f"(acc[mt][0]), "+f"(acc[mt][1]), "+f"(acc[mt][2]), "+f"(acc[mt][3])
                             : "r"(a[u][mt][0].z), "r"(a[u][mt][1].z), "r"(a[u][mt][0].w), "r"(a[u][mt][1].w), "r"(b[u].z), "r"(b[u].w));
            }
    }
    // partial[warp][mt][lane][i]; accumulator layout: i = 0, 1 -> (row g, columns 2 tid, 2 tid + 1); i = 2, 3 -> row g + 8
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
        *reinterpret_cast<float4 *>(&partial[((warp * MT + mt) * 32 + lane) * 4]) =
            make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]);
    __syncthreads();
    const int t = threadIdx.x;
    if (t >= MT * 128) return;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kSkinnyWarps; ++w) v += partial[w * MT * 128 + t];
    const int mt = t >> 7, ln = (t & 127) >> 2, i = t & 3;
    const int r = mt * 16 + (i >> 1) * 8 + (ln >> 2);
    const int c = n0 + 2 * (ln & 3) + (i & 1);
    if (r < M && c < N) {
        if (bias) v += bias[c];
        if constexpr (EPI == kEpiAccumulate) C[(int64_t)r * ldc + c] += TC(v);  // fp32 C; this thread owns the element
        else st_f32(C + (int64_t)r * ldc + c, c >= epi_col0 ? apply_epilogue<EPI>(v) : v);
    }
}

template <int MT, typename TC>
static hx_status launch_skinny_epi(const void *A, int64_t lda, const void *W, int64_t ldw, const float *bias, void *C, int64_t ldc,
                                   int M, int N, int K, int epi, int epi_col0, cudaStream_t st) {
    const dim3 grid((unsigned)((N + 7) / 8)), block(kSkinnyWarps * 32);
    auto a = static_cast<const __nv_bfloat16 *>(A), w = static_cast<const __nv_bfloat16 *>(W);
    auto c = static_cast<TC *>(C);
    switch (epi) {
        case kEpiNone: gemm_skinny_kernel<MT, TC, kEpiNone><<<grid, block, 0, st>>>(a, lda, w, ldw, bias, c, ldc, M, N, K, epi_col0); break;
        case kEpiSilu: gemm_skinny_kernel<MT, TC, kEpiSilu><<<grid, block, 0, st>>>(a, lda, w, ldw, bias, c, ldc, M, N, K, epi_col0); break;
        case kEpiSoftplus: gemm_skinny_kernel<MT, TC, kEpiSoftplus><<<grid, block, 0, st>>>(a, lda, w, ldw, bias, c, ldc, M, N, K, epi_col0); break;
        case kEpiSiluFast: gemm_skinny_kernel<MT, TC, kEpiSiluFast><<<grid, block, 0, st>>>(a, lda, w, ldw, bias, c, ldc, M, N, K, epi_col0); break;
        case kEpiAccumulate:
            if constexpr (sizeof(TC) == 4) gemm_skinny_kernel<MT, TC, kEpiAccumulate><<<grid, block, 0, st>>>(a, lda, w, ldw, bias, c, ldc, M, N, K, epi_col0);
            else return fail(HX_ERR_DTYPE_MISMATCH, "accumulating GEMM needs an fp32 C");
            break;
        default: return fail(HX_ERR_INVALID_INPUT, "unknown epilogue %d", epi);
    }
    return check_launch("gemm_skinny_kernel");
}

// M <= 64, K a multiple of 32, lda / ldw multiples of 8 and 16-byte aligned bases (checked by the caller).
hx_status launch_skinny(const void *A, int64_t lda, const void *W, int64_t ldw, const float *bias, void *C, int64_t ldc,
                        int c_dtype, int M, int N, int K, int epi, int epi_col0, cudaStream_t st) {
#define HX_SKINNY(MT)                                                                                                   \
    return c_dtype == HX_BF16 ? launch_skinny_epi<MT, __nv_bfloat16>(A, lda, W, ldw, bias, C, ldc, M, N, K, epi, epi_col0, st)    \
                              : launch_skinny_epi<MT, float>(A, lda, W, ldw, bias, C, ldc, M, N, K, epi, epi_col0, st)
    if (M <= 16) { HX_SKINNY(1); }
    if (M <= 32) { HX_SKINNY(2); }
    HX_SKINNY(4);
#undef HX_SKINNY
}

}  // namespace gemm
}  // namespace hx
