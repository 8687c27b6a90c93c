// bf16 GEMM on the 5th-generation tensor cores (tcgen05) for sm_100a:
//   C[M,N] = A[M,K] . W[N,K]^T (+ bias[N]) (+ activation), fp32 accumulation in tensor memory.
// Both operands are K-major (row-major A, row-major nn::Linear weight [out, in]), so no transposes.
//
// Persistent kernel, one CTA per SM, 6 warps:
//   warp 0      TMA producer: [128 x 64] A boxes and [BN x 64] W boxes, 128-byte swizzle, into a
//               multi-stage shared-memory ring (full/empty mbarriers).
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (M=128, N=BN, K=16, four per
//               64-wide k-block) and commits completion to the ring's empty barriers and, at the end
//               of a tile, to the accumulator-full barrier.  Two accumulators (2*BN columns) let the
//               next tile's main loop overlap this tile's epilogue.
//   warps 2..5  epilogue: tcgen05.ld 32 lanes x 32 columns at a time, bias/activation in registers,
//               16-byte stores to C.
// Out-of-range rows/columns/k are zero-filled by TMA and masked in the epilogue, so M, N, K need
// not be tile multiples (K and the leading dimensions must be multiples of 8 for the 16-byte rule).
// Every wait is bounded; a wait that runs out raises the per-device status word, the CTA drains,
// frees its tensor memory and returns.
#include <atomic>
#include <cstdlib>
#include "gemm.cuh"
#include "hx_tma.cuh"
#include "hx_tcgen05.cuh"

namespace hx {
namespace gemm {

using namespace hx::tc;

// Status word of this translation unit: a bounded wait that ran out ORs kWaitGemm in.
__device__ int g_gemm_status = 0;
constexpr int kWaitGemm = 32;
constexpr int BM = 128, BK = 64;
#ifndef HX_GEMM_PAIR_DEFAULT
#define HX_GEMM_PAIR_DEFAULT 1
#endif

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (int i = 0; i < kMaxTries; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    atomicOr(&g_gemm_status, kWaitGemm);
    return false;
}

// ---- CTA pairs (PAIR = 1): two CTAs of a cluster share one [256 x BN] tile.  Each CTA loads its own 128 rows of A
// and HALF of the W tile (BN/2 rows); the leader (cluster rank 0) issues tcgen05.mma.cta_group::2 (M = 256), which
// reads both CTAs' shared memory at the same offsets and leaves rows r*128.. of the tile in CTA r's tensor memory.
// Per FLOP a CTA pulls two thirds of the operand bytes of the single-CTA form, and the ring holds six stages.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory whose completion is counted on a barrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *m, uint32_t bar_cluster, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(bar_cluster)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on ONE barrier (of either CTA, by its shared::cluster address) when the pair's MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory");
}

template <int BN, int PAIR = 0> struct TcCfg {
    static constexpr int STAGES = PAIR ? 6 : (BN == 256 ? 4 : 6);
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_ROWS = PAIR ? BN / 2 : BN;   // W rows this CTA loads per stage
    static constexpr int B_BYTES = B_ROWS * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TMEM_COLS = 2 * BN;
    static constexpr int OUT_STAGE_BYTES = 32 * 128;  // one epilogue warp's [32 rows x 128 bytes] staging tile
    static constexpr int OUT_BUFS = 2;                // staging tiles per epilogue warp (more of them change nothing)
    static constexpr int OUT_BYTES = 4 * OUT_BUFS * OUT_STAGE_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_BYTES + 256 + 1024;
    static_assert(SMEM_BYTES <= 232448, "more shared memory than a CTA can have");
    static_assert((2 * STAGES + 4) * 8 + 8 <= 256, "barrier block too small");
    static constexpr int THREADS = 192;
};

template <int BN, typename TC, int EPI, int PAIR>
__device__ __forceinline__ void gemm_tc_body(const CUtensorMap &tm_a, const CUtensorMap &tm_w, const CUtensorMap &tm_c,
                                             const float *bias, TC *C, int64_t ldc, int M, int N, int K, int epi_col0,
                                             int vec_ok) {
    using Cfg = TcCfg<BN, PAIR>;
    constexpr int TILE_M = PAIR ? 2 * BM : BM;   // rows of C one tile covers (both CTAs of a pair)
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ __align__(16) char smem_raw[];
    char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);  // keeps the shared address space
    char *out_stage = smem + STAGES * Cfg::STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(out_stage + Cfg::OUT_BYTES);
    // barriers: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]; then the TMEM base and the abort flag
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto bar_full = [&](int s) { return bar0 + 8u * s; };
    auto bar_empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto bar_acc_full = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
    auto bar_acc_empty = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_m = (M + TILE_M - 1) / TILE_M, num_n = (N + BN - 1) / BN;
    const int tiles = num_m * num_n;
    const int kblocks = (K + BK - 1) / BK;
    // a pair walks the tile list together: cluster i is CTAs 2i and 2i+1
    const uint32_t crank = PAIR ? cluster_ctarank() : 0u;
    const int tile0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int tile_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_acc_full(a), 1);
            mbar_init(bar_acc_empty(a), PAIR ? 8 : 4);   // the leader's barrier also counts the peer's epilogue warps
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if constexpr (PAIR) {
        // the peer is running and its barriers are initialised before anything is allocated or signalled across
        __syncthreads();
        cluster_sync_all();
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            // one warp of EACH CTA of the pair performs the allocation (and, below, the release) together
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                         "r"((uint32_t)Cfg::TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                         "r"((uint32_t)Cfg::TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ============================================================ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tm_a);
            tma_prefetch_desc(&tm_w);
            int it = 0;
            bool ok = true;
            for (int tile = tile0; tile < tiles && ok; tile += tile_step) {
                const int m0 = (tile / num_n) * TILE_M + (int)crank * BM, n0 = (tile % num_n) * BN + (int)crank * Cfg::B_ROWS;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!wait_or_abort(bar_empty(s), ((it / STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
                    if constexpr (PAIR) {
                        // both CTAs' bytes are counted on the LEADER's full barrier, which its MMA lane waits on
                        const uint32_t full_leader = map_to_cta(bar_full(s), 0);
                        if (crank == 0) mbar_expect_tx(bar_full(s), 2 * Cfg::STAGE_BYTES);
                        tma_load_2d_pair(sa, &tm_a, full_leader, kb * BK, m0);
                        tma_load_2d_pair(sa + Cfg::A_BYTES, &tm_w, full_leader, kb * BK, n0);
                    } else {
                        mbar_expect_tx(bar_full(s), Cfg::STAGE_BYTES);
                        tma_load_2d(sa, &tm_a, bar_full(s), kb * BK, m0);
                        tma_load_2d(sa + Cfg::A_BYTES, &tm_w, bar_full(s), kb * BK, n0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ============================================================ MMA issuer
        if (lane == 0 && crank == 0) {   // in a pair only the leader issues
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                       ((uint32_t)(TILE_M >> 4) << 24);
            int it = 0, tc = 0;
            bool ok = true;
            for (int tile = tile0; tile < tiles && ok; tile += tile_step, ++tc) {
                const int acc = tc & 1;
                if (!wait_or_abort(bar_acc_empty(acc), ((tc >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!wait_or_abort(bar_full(s), (it / STAGES) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
                    const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + Cfg::A_BYTES);
                    if constexpr (PAIR) {
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            umma_bf16_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) ? 1u : 0u);
                        umma_commit_pair(map_to_cta(bar_empty(s), 0));  // the stage is free in both CTAs once these
                        umma_commit_pair(map_to_cta(bar_empty(s), 1));  // MMAs have read it
                    } else {
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            umma_bf16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) ? 1u : 0u);
                        umma_commit(bar_empty(s));  // the stage is free once these MMAs have read it
                    }
                }
                if (ok) {
                    if constexpr (PAIR) {
                        umma_commit_pair(map_to_cta(bar_acc_full(acc), 0));
                        umma_commit_pair(map_to_cta(bar_acc_full(acc), 1));
                    } else {
                        umma_commit(bar_acc_full(acc));
                    }
                }
            }
        }
    } else {
        // ============================================================ epilogue warps
        const int wq = warp & 3;  // TMEM lane quarter this warp may read
        int tc = 0, sc = 0;       // tiles done; staged blocks issued (selects the staging buffer)
        bool ok = true;
        for (int tile = tile0; tile < tiles && ok; tile += tile_step, ++tc) {
            const int acc = tc & 1;
            const int m0 = (tile / num_n) * TILE_M + (int)crank * BM, n0 = (tile % num_n) * BN;
            if (!wait_or_abort(bar_acc_full(acc), (tc >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int m = m0 + wq * 32 + lane;
            if (vec_ok) {
                // Coalesced path: 128 bytes of each of the warp's 32 rows go to a swizzled staging tile and
                // leave with one TMA store; out-of-range rows and columns are clipped by the tensor map.
                constexpr int CPB = 128 / (int)sizeof(TC);  // columns per staged block: 64 bf16 / 32 fp32
                char *my_stage = out_stage + (warp - 2) * Cfg::OUT_BUFS * Cfg::OUT_STAGE_BYTES;
#pragma unroll 1
                for (int cb = 0; cb < BN / CPB; ++cb) {
                    const int nb = n0 + cb * CPB;
                    if (nb >= N) break;  // warp-uniform
                    char *buf = my_stage + (sc % Cfg::OUT_BUFS) * Cfg::OUT_STAGE_BYTES;
                    ++sc;
                    // both halves of the block are fetched from tensor memory before anything waits
                    constexpr int HALVES = CPB / 32;
                    uint32_t r[HALVES][32];
#pragma unroll
                    for (int half = 0; half < HALVES; ++half)
                        tmem_ld32(tmem_base + acc * BN + cb * CPB + half * 32 + ((uint32_t)(wq * 32) << 16), r[half]);
                    if (lane == 0) tma_store_wait_read<Cfg::OUT_BUFS - 1>();  // the store that last read this buffer is done
                    tmem_ld_wait();
                    __syncwarp();
#pragma unroll
                    for (int half = 0; half < HALVES; ++half) {
                        float v[32];
                        const bool act = nb + half * 32 >= epi_col0;  // warp-uniform: epi_col0 is a multiple of 32
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            float x = __uint_as_float(r[half][j]);
                            const int n = nb + half * 32 + j;
                            if (bias) x += (n < N) ? __ldg(bias + n) : 0.f;
                            v[j] = x;
                        }
                        if (EPI != kEpiNone && act) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = apply_epilogue<EPI>(v[j]);
                        }
                        // 16-byte pieces of this lane's row, XOR-swizzled with the row index like the TMA box
                        if constexpr (sizeof(TC) == 2) {
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4) {
                                uint32_t w[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[q4 * 8 + 2 * e], v[q4 * 8 + 2 * e + 1]);
                                    w[e] = *reinterpret_cast<const uint32_t *>(&h2);
                                }
                                const int chunk = half * 4 + q4;
                                *reinterpret_cast<uint4 *>(buf + lane * 128 + ((chunk ^ (lane & 7)) << 4)) =
                                    make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        } else {
#pragma unroll
                            for (int q4 = 0; q4 < 8; ++q4)
                                *reinterpret_cast<float4 *>(buf + lane * 128 + ((q4 ^ (lane & 7)) << 4)) =
                                    make_float4(v[q4 * 4], v[q4 * 4 + 1], v[q4 * 4 + 2], v[q4 * 4 + 3]);
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (m0 + wq * 32 < M) {   // a box that starts below the last row has nothing to write
                            if constexpr (EPI == kEpiAccumulate) tma_reduce_add_2d(&tm_c, smem_u32(buf), nb, m0 + wq * 32);
                            else tma_store_2d(&tm_c, smem_u32(buf), nb, m0 + wq * 32);
                        }
                        tma_store_commit();
                    }
                }
            } else {
            TC *crow = C + (int64_t)m * ldc;
#pragma unroll 1
            for (int ch = 0; ch < BN / 32; ++ch) {
                const int nb = n0 + ch * 32;
                if (nb >= N) break;  // warp-uniform
                uint32_t r[32];
                tmem_ld32(tmem_base + acc * BN + ch * 32 + ((uint32_t)(wq * 32) << 16), r);
                tmem_ld_wait();
                if (m < M) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float x = __uint_as_float(r[j]);
                        if (nb + j < N) {
                            if (bias) x += __ldg(bias + nb + j);
                            if constexpr (EPI == kEpiAccumulate) crow[nb + j] += x;  // this thread owns the element
                            else st_f32(crow + nb + j, nb + j >= epi_col0 ? apply_epilogue<EPI>(x) : x);
                        }
                    }
                }
            }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if constexpr (PAIR) mbar_arrive_cluster(map_to_cta(bar_acc_empty(acc), 0));
                else mbar_arrive(bar_acc_empty(acc));
            }
        }
        if (lane == 0) tma_store_wait_all<0>();  // staging tiles must outlive their TMA stores
    }

    // teardown: everybody meets, then the allocating warp frees tensor memory
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();   // the peer no longer reads tensor memory or signals this CTA's barriers
    if (warp == 1) {
        tc_fence_after();
        if constexpr (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS)
                         : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS)
                         : "memory");
    }
    if constexpr (PAIR) {
        __syncthreads();
        cluster_sync_all();   // neither CTA leaves while the other still releases tensor memory
    }
}

template <int BN, typename TC, int EPI>
__global__ void __launch_bounds__(192, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
               const __grid_constant__ CUtensorMap tm_c, const float *bias, TC *C, int64_t ldc, int M, int N, int K, int epi_col0,
               int vec_ok) {
    gemm_tc_body<BN, TC, EPI, 0>(tm_a, tm_w, tm_c, bias, C, ldc, M, N, K, epi_col0, vec_ok);
}

// The same kernel run by CTA pairs: grid = 2 x pairs, cluster (2, 1, 1).
template <int BN, typename TC, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                    const __grid_constant__ CUtensorMap tm_c, const float *bias, TC *C, int64_t ldc, int M, int N, int K,
                    int epi_col0, int vec_ok) {
    gemm_tc_body<BN, TC, EPI, 1>(tm_a, tm_w, tm_c, bias, C, ldc, M, N, K, epi_col0, vec_ok);
}

template <int BN, typename TC, int EPI>
static hx_status launch_tc_inst(const CUtensorMap &ma, const CUtensorMap &mw, const CUtensorMap &mc, const float *bias, void *C,
                                int64_t ldc, int M, int N, int K, int epi_col0, int vec_ok, cudaStream_t st) {
    using Cfg = TcCfg<BN>;
    auto kern = gemm_tc_kernel<BN, TC, EPI>;
    static std::atomic<bool> attr_set[64];  // zero-initialised; setting the attribute twice is harmless
    int dev = 0;
    HX_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
        HX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_set[dev].store(true, std::memory_order_release);
    }
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    kern<<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(ma, mw, mc, bias, static_cast<TC *>(C), ldc, M, N, K, epi_col0, vec_ok);
    return check_launch("gemm_tc_kernel");
}

// How many CTA pairs of the pair kernel can be resident at once on the current device (0: pairs cannot be used).
template <int BN, typename TC, int EPI> static int pair_capacity() {
    using Cfg = TcCfg<BN, 1>;
    static std::atomic<int> cap[64];   // 0 = not asked yet, -1 = unusable, else pairs
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    int c = cap[dev].load(std::memory_order_acquire);
    if (c == 0) {
        auto kern = gemm_tc_pair_kernel<BN, TC, EPI>;
        c = -1;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2 * sm_count());
            cfg.blockDim = dim3(Cfg::THREADS);
            cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
            cudaLaunchAttribute at;
            at.id = cudaLaunchAttributeClusterDimension;
            at.val.clusterDim.x = 2;
            at.val.clusterDim.y = 1;
            at.val.clusterDim.z = 1;
            cfg.attrs = &at;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) c = n;
        }
        (void)cudaGetLastError();
        cap[dev].store(c, std::memory_order_release);
    }
    return c > 0 ? c : 0;
}

template <int BN, typename TC, int EPI>
static hx_status launch_tc_pair_inst(const CUtensorMap &ma, const CUtensorMap &mw, const CUtensorMap &mc, const float *bias,
                                     void *C, int64_t ldc, int M, int N, int K, int epi_col0, int pairs, cudaStream_t st) {
    using Cfg = TcCfg<BN, 1>;
    const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
    const int grid = 2 * (tiles < pairs ? tiles : pairs);
    gemm_tc_pair_kernel<BN, TC, EPI><<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(ma, mw, mc, bias, static_cast<TC *>(C), ldc, M,
                                                                                 N, K, epi_col0, 1);
    return check_launch("gemm_tc_pair_kernel");
}

// 0: single CTAs only; 1: CTA pairs where they measured faster; 2: pairs wherever the shape allows.
// HX_GEMM_PAIR in the environment sets the initial mode.
static std::atomic<int> g_pair_mode{-1};   // -1: not set through hx_gemm_pair_mode
static int pair_mode() {
    const int m = g_pair_mode.load(std::memory_order_relaxed);
    if (m >= 0) return m;
    static const int mode = [] {
        const char *e = getenv("HX_GEMM_PAIR");
        return e ? atoi(e) : HX_GEMM_PAIR_DEFAULT;
    }();
    return mode;
}

template <int BN, typename TC>
static hx_status launch_tc_epi(const CUtensorMap &ma, const CUtensorMap &mw, const CUtensorMap &mc, const float *bias, void *C,
                               int64_t ldc, int M, int N, int K, int vec_ok, int epi, int epi_col0, cudaStream_t st) {
    switch (epi) {
        case kEpiNone: return launch_tc_inst<BN, TC, kEpiNone>(ma, mw, mc, bias, C, ldc, M, N, K, epi_col0, vec_ok, st);
        case kEpiSilu: return launch_tc_inst<BN, TC, kEpiSilu>(ma, mw, mc, bias, C, ldc, M, N, K, epi_col0, vec_ok, st);
        case kEpiSoftplus: return launch_tc_inst<BN, TC, kEpiSoftplus>(ma, mw, mc, bias, C, ldc, M, N, K, epi_col0, vec_ok, st);
        case kEpiSiluFast: return launch_tc_inst<BN, TC, kEpiSiluFast>(ma, mw, mc, bias, C, ldc, M, N, K, epi_col0, vec_ok, st);
        case kEpiAccumulate:
            if constexpr (sizeof(TC) == 4) return launch_tc_inst<BN, TC, kEpiAccumulate>(ma, mw, mc, bias, C, ldc, M, N, K, epi_col0, vec_ok, st);
            else return fail(HX_ERR_DTYPE_MISMATCH, "accumulating GEMM needs an fp32 C");
        default: return fail(HX_ERR_INVALID_INPUT, "unknown epilogue %d", epi);
    }
}

}  // namespace gemm

hx_status read_status_gemm(int *v, bool clear) {
    HX_CUDA(cudaMemcpyFromSymbol(v, gemm::g_gemm_status, sizeof(int)));
    if (clear && *v != 0) {
        const int zero = 0;
        HX_CUDA(cudaMemcpyToSymbol(gemm::g_gemm_status, &zero, sizeof(int)));
    }
    return HX_OK;
}

}  // namespace hx

extern "C" hx_status hx_gemm_pair_mode(int32_t mode, int32_t *pairs) {
    if (mode >= 0) hx::gemm::g_pair_mode.store(mode > 2 ? 2 : mode, std::memory_order_relaxed);
    if (pairs) *pairs = hx::gemm::pair_capacity<256, __nv_bfloat16, hx::gemm::kEpiNone>();
    return HX_OK;
}

extern "C" hx_status hx_gemm_bf16(const void *A, int64_t lda, const void *W, int64_t ldw, const float *bias, void *C,
                                  int64_t ldc, int32_t c_dtype, int32_t M, int32_t N, int32_t K, int32_t epilogue,
                                  void *stream) {
    return hx_gemm_bf16_cols(A, lda, W, ldw, bias, C, ldc, c_dtype, M, N, K, epilogue, 0, stream);
}

extern "C" hx_status hx_gemm_bf16_acc(const void *A, int64_t lda, const void *W, int64_t ldw, float *C, int64_t ldc, int32_t M,
                                      int32_t N, int32_t K, void *stream) {
    return hx_gemm_bf16_cols(A, lda, W, ldw, nullptr, C, ldc, HX_F32, M, N, K, hx::gemm::kEpiAccumulate, 0, stream);
}

extern "C" hx_status hx_gemm_bf16_cols(const void *A, int64_t lda, const void *W, int64_t ldw, const float *bias, void *C,
                                       int64_t ldc, int32_t c_dtype, int32_t M, int32_t N, int32_t K, int32_t epilogue,
                                       int32_t epilogue_first_col, void *stream) {
    using namespace hx::gemm;
    const int epi_col0 = epilogue_first_col;
    HX_REQUIRE(epi_col0 >= 0 && epi_col0 % 32 == 0, HX_ERR_INVALID_INPUT,
               "epilogue_first_col must be a non-negative multiple of 32 (got %d)", epi_col0);
    hx_status s = validate_gemm(A, lda, W, ldw, C, ldc, M, N, K);
    if (s != HX_OK) return s;
    if (M == 0 || N == 0) return HX_OK;
    HX_REQUIRE(c_dtype == HX_F32 || c_dtype == HX_BF16, HX_ERR_DTYPE_MISMATCH, "c_dtype %d unsupported", c_dtype);
    HX_REQUIRE(K >= 1, HX_ERR_INVALID_DIMENSION, "K must be positive");
    HX_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0, HX_ERR_UNSUPPORTED_OPERATION,
               "hx_gemm_bf16 needs K, lda and ldw to be multiples of 8 (got %d, %lld, %lld)", K, (long long)lda,
               (long long)ldw);
    cudaStream_t st = (cudaStream_t)stream;
    // a handful of rows (a decode step): stream the weights through many small CTAs instead of one 128-row tile
    if (M <= 64 && K % 32 == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0)
        return launch_skinny(A, lda, W, ldw, bias, C, ldc, c_dtype, M, N, K, epilogue, epi_col0, st);
    // a short inner dimension (dt_proj, K = dt_rank): bound by writing C, which a store-shaped kernel does at twice the
    // rate of the tile kernel's epilogue
    if (K <= 64 && M > 64 && N % 8 == 0 && N >= 64 && c_dtype == HX_BF16 && bias == nullptr && epilogue == kEpiNone &&
        (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc * 2) % 16 == 0)
        return launch_lowk(A, lda, W, ldw, C, ldc, M, N, K, st);
    const int BN = N > 128 ? 256 : 128;
    CUtensorMap ma, mw;
    const uint64_t dims_a[2] = {(uint64_t)K, (uint64_t)M}, dims_w[2] = {(uint64_t)K, (uint64_t)N};
    const uint64_t str_a[1] = {(uint64_t)lda * 2}, str_w[1] = {(uint64_t)ldw * 2};
    const uint32_t box_a[2] = {(uint32_t)BK, (uint32_t)BM}, box_w[2] = {(uint32_t)BK, (uint32_t)BN};
    if ((s = hx::encode_tensor_map(&ma, HX_BF16, 2, A, dims_a, str_a, box_a, true)) != HX_OK) return s;
    if ((s = hx::encode_tensor_map(&mw, HX_BF16, 2, W, dims_w, str_w, box_w, true)) != HX_OK) return s;
    const int es = c_dtype == HX_BF16 ? 2 : 4;
    // C leaves through TMA when its base and row stride meet the 16-byte rule; otherwise by plain stores
    const int vec_ok = ((reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc * es) % 16 == 0) ? 1 : 0;
    CUtensorMap mc = ma;
    if (vec_ok) {
        const uint64_t dims_c[2] = {(uint64_t)N, (uint64_t)M};
        const uint64_t str_c[1] = {(uint64_t)ldc * es};
        const uint32_t box_c[2] = {(uint32_t)(128 / es), 32};
        if ((s = hx::encode_tensor_map(&mc, c_dtype, 2, C, dims_c, str_c, box_c, true)) != HX_OK) return s;
    }
    // CTA pairs for the wide shapes: [256 x 256] tiles, each CTA loading 128 rows of the W tile.  Measured against
    // single CTAs on a B200 (65 536 rows, sustained): equal within 2 % where C is written (K = 768: 253-257 against
    // 248-253 us), 5-10 % faster for the accumulating epilogue at K = 1536 (134-145 against 145-152 us; 3.35 against
    // 3.72 ms over the 24 blocks of the byte-LM step), slower below four waves of tiles.  [256 x 128] pair tiles
    // were measured too and dropped (in_proj 388 us: the pair instruction does not speed up with the narrower N).
    // Mode 1 therefore takes pairs for the accumulating epilogue on at least four waves of them, mode 2 wherever the
    // shape allows.
    const int pm = pair_mode();
    if (BN == 256 && vec_ok && pm != 0 && M >= 4 * BM && (epilogue == kEpiNone || (epilogue == kEpiAccumulate && c_dtype == HX_F32))) {
        const bool accum = epilogue == kEpiAccumulate;
        const int64_t pair_tiles = (int64_t)((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
        int pairs = 0;
        if (accum) pairs = pair_capacity<256, float, kEpiAccumulate>();
        else if (pm >= 2) pairs = c_dtype == HX_BF16 ? pair_capacity<256, __nv_bfloat16, kEpiNone>() : pair_capacity<256, float, kEpiNone>();
        if (pairs > 0 && (pm >= 2 || pair_tiles >= 4 * (int64_t)pairs)) {
            CUtensorMap mwh;
            const uint32_t box_wh[2] = {(uint32_t)BK, (uint32_t)(BN / 2)};
            if ((s = hx::encode_tensor_map(&mwh, HX_BF16, 2, W, dims_w, str_w, box_wh, true)) != HX_OK) return s;
            if (accum) return launch_tc_pair_inst<256, float, kEpiAccumulate>(ma, mwh, mc, bias, C, ldc, M, N, K, epi_col0, pairs, st);
            if (c_dtype == HX_BF16)
                return launch_tc_pair_inst<256, __nv_bfloat16, kEpiNone>(ma, mwh, mc, bias, C, ldc, M, N, K, epi_col0, pairs, st);
            return launch_tc_pair_inst<256, float, kEpiNone>(ma, mwh, mc, bias, C, ldc, M, N, K, epi_col0, pairs, st);
        }
    }
    if (BN == 256) {
        if (c_dtype == HX_BF16) return launch_tc_epi<256, __nv_bfloat16>(ma, mw, mc, bias, C, ldc, M, N, K, vec_ok, epilogue, epi_col0, st);
        return launch_tc_epi<256, float>(ma, mw, mc, bias, C, ldc, M, N, K, vec_ok, epilogue, epi_col0, st);
    }
    if (c_dtype == HX_BF16) return launch_tc_epi<128, __nv_bfloat16>(ma, mw, mc, bias, C, ldc, M, N, K, vec_ok, epilogue, epi_col0, st);
    return launch_tc_epi<128, float>(ma, mw, mc, bias, C, ldc, M, N, K, vec_ok, epilogue, epi_col0, st);
}
