// gemm_lowk_kernel: C[M,N] = A[M,K] . W[N,K]^T for a short inner dimension (K <= 64), the shape of dt_proj
// (K = dt_rank = 48, N = d_inner): 2 K flops per output element, so the product is bound by WRITING C, and the
// 128 x 256 tcgen05 tile kernel, whose main loop is a single k-block here, spends its time in the epilogue
// (87 us for 65 536 x 1536 x 48 against 31 us of stores at the measured copy bandwidth).
//
// A CTA owns RT row tiles of 16 rows (2 to 8, chosen so that the grid is a whole number of waves) and all N
// columns.  Its A rows ([RT * 16, K], a few KB) are staged in shared
// memory once.  A warp takes blocks of 64 columns: it loads the W fragments of the block into registers once
// (8 column tiles x K / 16 k-steps x 2 registers), then runs over the CTA's row tiles with mma.sync.m16n8k16
// (bf16 in, fp32 accumulate), rounds the 16 x 64 result to bf16 into a small per-warp staging tile and writes it
// out as whole 128-byte row segments (16-byte stores, four rows per instruction).
#include "gemm.cuh"

namespace hx {
namespace gemm {

constexpr int kLowkWarps = 8;

constexpr int kLowkMaxRowTiles = 8;

template <int KS>  // KS: k-steps of 16 (K <= 16 KS); RT: row tiles of 16 per CTA (<= kLowkMaxRowTiles)
__global__ void __launch_bounds__(kLowkWarps * 32)
gemm_lowk_kernel(const __nv_bfloat16 *__restrict__ A, int64_t lda, const __nv_bfloat16 *__restrict__ W, int64_t ldw,
                 __nv_bfloat16 *__restrict__ C, int64_t ldc, int M, int N, int K, int RT) {
    constexpr int AK = KS * 16 + 8;              // A row pitch in elements: the pad spreads the fragment loads over the banks
    constexpr int SP = 64 + 8;                   // staging row pitch
    __shared__ __align__(16) __nv_bfloat16 sA[kLowkMaxRowTiles * 16 * AK];
    __shared__ __align__(16) __nv_bfloat16 sOut[kLowkWarps][16 * SP];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tid = lane & 3;
    const int m0 = blockIdx.x * RT * 16;

    // stage the CTA's A rows (zero beyond M and beyond K)
    for (int i = threadIdx.x; i < RT * 16 * (KS * 8); i += blockDim.x) {
        const int r = i / (KS * 8), kp = i % (KS * 8);  // element pair
        const int k = 2 * kp;
        uint32_t v = 0u;
        if (m0 + r < M && k < K) v = *reinterpret_cast<const uint32_t *>(A + (int64_t)(m0 + r) * lda + k);
        *reinterpret_cast<uint32_t *>(&sA[r * AK + k]) = v;
    }
    __syncthreads();

    __nv_bfloat16 *so = sOut[warp];
    for (int cb = warp; cb * 64 < N; cb += kLowkWarps) {
        const int n0 = cb * 64;
        // W fragments of this column block: b0 = (k 2 tid, 2 tid + 1; column g), b1 = (k 2 tid + 8, + 9; column g)
        uint32_t bf[8][KS][2];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int n = n0 + nt * 8 + g;
            const __nv_bfloat16 *wr = W + (int64_t)(n < N ? n : 0) * ldw;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int k = ks * 16 + 2 * tid;
                bf[nt][ks][0] = (n < N && k < K) ? __ldg(reinterpret_cast<const uint32_t *>(wr + k)) : 0u;
                bf[nt][ks][1] = (n < N && k + 8 < K) ? __ldg(reinterpret_cast<const uint32_t *>(wr + k + 8)) : 0u;
            }
        }
#pragma unroll 2
        for (int rt = 0; rt < RT; ++rt) {
            if (m0 + rt * 16 >= M) break;
            uint32_t af[KS][4];
            const __nv_bfloat16 *ar = sA + (rt * 16 + g) * AK + 2 * tid;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                af[ks][0] = *reinterpret_cast<const uint32_t *>(ar + ks * 16);
                af[ks][1] = *reinterpret_cast<const uint32_t *>(ar + 8 * AK + ks * 16);
                af[ks][2] = *reinterpret_cast<const uint32_t *>(ar + ks * 16 + 8);
                af[ks][3] = *reinterpret_cast<const uint32_t *>(ar + 8 * AK + ks * 16 + 8);
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks)
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                                 "{%0, %1, %2, %3};"
                                 : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
                                 : "r"(af[ks][0]), "r"(af[ks][1]), "r"(af[ks][2]), "r"(af[ks][3]), "r"(bf[nt][ks][0]), "r"(bf[nt][ks][1]));
                // accumulator: (row g, columns 2 tid, 2 tid + 1) and (row g + 8, same columns)
                const __nv_bfloat162 lo = __floats2bfloat162_rn(c0, c1), hi = __floats2bfloat162_rn(c2, c3);
                *reinterpret_cast<__nv_bfloat162 *>(&so[g * SP + nt * 8 + 2 * tid]) = lo;
                *reinterpret_cast<__nv_bfloat162 *>(&so[(g + 8) * SP + nt * 8 + 2 * tid]) = hi;
            }
            __syncwarp();
            // 16 rows x 8 chunks of 16 bytes: four rows per warp-wide store, each row segment 128 contiguous bytes
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int id = it * 32 + lane, r = id >> 3, c = id & 7;
                const int row = m0 + rt * 16 + r, col = n0 + c * 8;
                if (row < M && col < N)
                    *reinterpret_cast<uint4 *>(C + (int64_t)row * ldc + col) = *reinterpret_cast<const uint4 *>(&so[r * SP + c * 8]);
            }
            __syncwarp();
        }
    }
}

// K <= 64 and a multiple of 8, N a multiple of 8, bf16 C with a 16-byte aligned base and row stride; lda, ldw even
// and the bases 4-byte aligned (checked by the caller).
hx_status launch_lowk(const void *A, int64_t lda, const void *W, int64_t ldw, void *C, int64_t ldc, int M, int N, int K,
                      cudaStream_t st) {
    auto a = static_cast<const __nv_bfloat16 *>(A), w = static_cast<const __nv_bfloat16 *>(W);
    auto c = static_cast<__nv_bfloat16 *>(C);
    const int ks = (K + 15) / 16;
    // Row tiles per CTA: the kernel is bound by its stores and two CTAs fit an SM, so the grid should be a whole
    // number of waves of 2 x SMs CTAs; among 2 .. 8 tiles take the count with the least waves x tiles.
    const int slots = 2 * sm_count();
    int rt = 2;
    long best = -1;
    for (int r = 2; r <= kLowkMaxRowTiles; ++r) {
        const long ctas = ((long)M + 16 * r - 1) / (16 * r);
        const long cost = ((ctas + slots - 1) / slots) * r;
        if (best < 0 || cost < best || (cost == best && r > rt)) { best = cost; rt = r; }
    }
    const unsigned grid = (unsigned)(((long)M + 16 * rt - 1) / (16 * rt));
    const dim3 block(kLowkWarps * 32);
    if (ks == 1) gemm_lowk_kernel<1><<<grid, block, 0, st>>>(a, lda, w, ldw, c, ldc, M, N, K, rt);
    else if (ks == 2) gemm_lowk_kernel<2><<<grid, block, 0, st>>>(a, lda, w, ldw, c, ldc, M, N, K, rt);
    else if (ks == 3) gemm_lowk_kernel<3><<<grid, block, 0, st>>>(a, lda, w, ldw, c, ldc, M, N, K, rt);
    else gemm_lowk_kernel<4><<<grid, block, 0, st>>>(a, lda, w, ldw, c, ldc, M, N, K, rt);
    return check_launch("gemm_lowk_kernel");
}

}  // namespace gemm
}  // namespace hx
