// Causal depthwise conv + SiLU and the x_proj product of a Mamba block in ONE kernel (bf16, sm_100a):
//   u[b,t,:]     = silu(conv_b + sum_k conv_w[:,k] * x[b,t-3+k,:])        (nn::ssm::MambaBlock::conv1d + silu)
//   x_dbl[b,t,:] = u[b,t,:] . W_x^T                                      (x_proj, [dt_low | B | C] of the row)
// As two kernels u is written by the conv and read again by the GEMM (2 bytes per element each way, 201 MB per
// block of the byte LM); here the tile of u the conv produces in shared memory IS the GEMM's A operand, so u is
// written once (the scan reads it) and never read back.
//
// One CTA per 128 consecutive steps of one sequence (64 where that leaves SMs idle), all channels, walked in blocks
// of 64 channels:
//   warp 0      TMA producer: [131 steps x 64 channels] boxes of x (3 steps of history in front; steps before the
//               sequence start are zero-filled by TMA, which is the conv's causal padding) and [n_out x 64] boxes
//               of W_x (128-byte swizzle), each in a small ring.
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (M = 128, N = n_out, K = 16, four per block)
//               on the u tile and the W_x tile and commits to the barriers that free them.
//   warps 2..9  conv + SiLU: a thread owns two adjacent channels and 16 steps (8 with 64-step tiles), loads its rows
//               of the x box, slides the 4-tap window down them and writes bf16 pairs into the u tile in the 128-byte-swizzled K-major layout the tensor core
//               reads.  The same tile then leaves for global memory with one TMA store.  After the last block
//               four of these warps drain the accumulator: tcgen05.ld, bf16, 16-byte stores of the x_dbl rows.
// Two CTAs fit an SM (105 KB of shared memory, 128 columns of tensor memory each; three with 64-step tiles), so one
// CTA's loads and stores run under the other's arithmetic.  The arithmetic of u is that of the strip kernel of elementwise.cu, so u is
// bit-identical to it; x_dbl accumulates in fp32 over ascending k like the tcgen05 GEMM.
// Every wait is bounded; a wait that runs out raises the status word, the CTA drains, frees its tensor memory and
// returns.
#include <atomic>

#include "hx_common.cuh"
#include "hx_tcgen05.cuh"
#include "hx_tma.cuh"

namespace hx {
namespace cx {

using namespace hx::tc;

__device__ int g_cx_status = 0;
constexpr int kWaitConvX = 64;

constexpr int KC = 64;             // channels per block (128 bytes of bf16: one swizzle row)
constexpr int HALO = 3;            // history steps of a 4-tap causal conv
constexpr int MMA_M = 128;
#ifndef HX_CX_XS
#define HX_CX_XS 3
#endif
#ifndef HX_CX_WS
#define HX_CX_WS 2
#endif
#ifndef HX_CX_AB
#define HX_CX_AB 2
#endif
constexpr int XS = HX_CX_XS, WS = HX_CX_WS;   // ring depths of the x boxes and the W_x boxes
constexpr int AB = HX_CX_AB;                   // u tiles: one being written, the others read by the MMA / the store
constexpr int COMPUTE_THREADS = 256;
constexpr int THREADS = 64 + COMPUTE_THREADS;
constexpr int NBARS = 2 * XS + 2 * WS + 2 * AB + 1;

// TM = steps per CTA: 128, or 64 where 128-step tiles would leave SMs without a CTA.  The MMA is always M = 128; with
// 64 steps its upper 64 rows read whatever follows the tile in shared memory and their results are dropped.
template <int TM> struct Cfg {
    static_assert(TM == 64 || TM == 128, "64 or 128 steps per CTA");
    static constexpr int A_BYTES = TM * KC * 2;
    static constexpr int X_BOX_ROWS = TM + HALO;
    static constexpr int X_BOX_BYTES = X_BOX_ROWS * KC * 2;
    static constexpr int X_STAGE_BYTES = (X_BOX_BYTES + 127) / 128 * 128;
    static constexpr int ROWS_PER_THREAD = TM / (COMPUTE_THREADS / 32);
    static constexpr int CTAS_PER_SM = TM == 64 ? 3 : 2;
};

__host__ __device__ constexpr int w_stage_bytes(int n_out) { return (n_out * KC * 2 + 1023) / 1024 * 1024; }
template <int TM> __host__ __device__ constexpr int smem_bytes(int n_out) {
    return AB * Cfg<TM>::A_BYTES + WS * w_stage_bytes(n_out) + XS * Cfg<TM>::X_STAGE_BYTES + 256 + 1024;
}

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (int i = 0; i < kMaxTries; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    atomicOr(&g_cx_status, kWaitConvX);
    return false;
}

// Barrier 1 among the compute threads that also ORs a predicate, so that all of them leave the block loop together.
__device__ __forceinline__ bool compute_sync_or(bool v) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\t"
        "barrier.cta.red.or.pred p, 1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)v), "n"(COMPUTE_THREADS)
        : "memory");
    return r != 0;
}

template <int TM>
__global__ void __launch_bounds__(THREADS, Cfg<TM>::CTAS_PER_SM)
conv_xproj_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                  const __grid_constant__ CUtensorMap tm_u, const float *__restrict__ cw, const float *__restrict__ cb,
                  __nv_bfloat16 *__restrict__ xd, int64_t ldxd, int L, int E, int n_out, int n_mma, int tiles_per_seq,
                  uint32_t tmem_cols) {
    constexpr int A_BYTES = Cfg<TM>::A_BYTES, X_BOX_BYTES = Cfg<TM>::X_BOX_BYTES, X_STAGE_BYTES = Cfg<TM>::X_STAGE_BYTES;
    constexpr int ROWS_PER_THREAD = Cfg<TM>::ROWS_PER_THREAD;
    extern __shared__ __align__(16) char smem_raw[];
    char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int wbytes = w_stage_bytes(n_mma);   // n_mma: n_out rounded up to the MMA's multiple of 16 (rows >= n_out are zero)
    char *a_tile = smem;                          // AB x [128 steps x 64 channels], swizzled
    char *w_tile = a_tile + AB * A_BYTES;         // WS x [n_out x 64 channels], swizzled
    char *x_tile = w_tile + WS * wbytes;          // XS x [131 steps x 64 channels], plain rows of 128 bytes
    uint64_t *bars = reinterpret_cast<uint64_t *>(x_tile + XS * X_STAGE_BYTES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + NBARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto bar_x_full = [&](int s) { return bar0 + 8u * s; };
    auto bar_x_empty = [&](int s) { return bar0 + 8u * (XS + s); };
    auto bar_w_full = [&](int s) { return bar0 + 8u * (2 * XS + s); };
    auto bar_w_empty = [&](int s) { return bar0 + 8u * (2 * XS + WS + s); };
    auto bar_a_full = [&](int a) { return bar0 + 8u * (2 * XS + 2 * WS + a); };
    auto bar_a_done = [&](int a) { return bar0 + 8u * (2 * XS + 2 * WS + AB + a); };
    const uint32_t bar_acc_full = bar0 + 8u * (2 * XS + 2 * WS + 2 * AB);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x / tiles_per_seq;
    const int t0 = (blockIdx.x % tiles_per_seq) * TM;
    const int kblocks = E / KC;

    if (threadIdx.x == 0) {
        for (int i = 0; i < NBARS; ++i) mbar_init(bar0 + 8u * i, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ============================================================ TMA producer
        // lane 0 feeds the x ring, lane 1 the W_x ring: neither waits for the other's consumer
        if (lane == 0) {
            tma_prefetch_desc(&tm_x);
            for (int kb = 0; kb < kblocks; ++kb) {
                const int sx = kb % XS;
                if (!wait_or_abort(bar_x_empty(sx), ((kb / XS) & 1) ^ 1, abort_flag)) break;
                mbar_expect_tx(bar_x_full(sx), X_BOX_BYTES);
                tma_load_3d(smem_u32(x_tile + sx * X_STAGE_BYTES), &tm_x, bar_x_full(sx), kb * KC, t0 - HALO, b);
            }
        } else if (lane == 1) {
            tma_prefetch_desc(&tm_w);
            for (int kb = 0; kb < kblocks; ++kb) {
                const int sw = kb % WS;
                if (!wait_or_abort(bar_w_empty(sw), ((kb / WS) & 1) ^ 1, abort_flag)) break;
                mbar_expect_tx(bar_w_full(sw), (uint32_t)(n_mma * KC * 2));
                tma_load_2d(smem_u32(w_tile + sw * wbytes), &tm_w, bar_w_full(sw), kb * KC, 0);
            }
        }
    } else if (warp == 1) {
        // ============================================================ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = idesc_bf16(MMA_M, n_mma);
            bool ok = true;
            for (int kb = 0; kb < kblocks; ++kb) {
                const int ab = kb % AB, sw = kb % WS;
                if (!wait_or_abort(bar_a_full(ab), (kb / AB) & 1, abort_flag) ||
                    !wait_or_abort(bar_w_full(sw), (kb / WS) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint64_t da = make_smem_desc(smem_u32(a_tile + ab * A_BYTES));
                const uint64_t db = make_smem_desc(smem_u32(w_tile + sw * wbytes));
#pragma unroll
                for (int k = 0; k < KC / 16; ++k)
                    umma_bf16(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) ? 1u : 0u);
                umma_commit(bar_w_empty(sw));  // both tiles are free once these MMAs have read them
                umma_commit(bar_a_done(ab));
            }
            if (ok) umma_commit(bar_acc_full);
        }
    } else {
        // ============================================================ conv + SiLU warps, then the epilogue
        const int ct = threadIdx.x - 64;
        const int cp = ct & 31;                         // pair of adjacent channels within the block
        const int r0 = (ct >> 5) * ROWS_PER_THREAD;     // first of this thread's steps
        const float4 *cw4 = reinterpret_cast<const float4 *>(cw);
        bool bad = false;
        // this block's taps and bias; the next block's are fetched while this one is computed
        float4 wa_n = __ldg(cw4 + 2 * cp), wb_n = __ldg(cw4 + 2 * cp + 1);
        float ba_n = cb ? __ldg(cb + 2 * cp) : 0.f, bb_n = cb ? __ldg(cb + 2 * cp + 1) : 0.f;
        for (int kb = 0; kb < kblocks; ++kb) {
            const int sx = kb % XS, ab = kb % AB;
            const float4 wa = wa_n, wb = wb_n;
            const float ba = ba_n, bb = bb_n;
            if (kb + 1 < kblocks) {
                const int cn = (kb + 1) * KC + 2 * cp;
                wa_n = __ldg(cw4 + cn); wb_n = __ldg(cw4 + cn + 1);
                if (cb) { ba_n = __ldg(cb + cn); bb_n = __ldg(cb + cn + 1); }
            }
            bool ok = wait_or_abort(bar_x_full(sx), (kb / XS) & 1, abort_flag);
            ok = ok && wait_or_abort(bar_a_done(ab), ((kb / AB) & 1) ^ 1, abort_flag);
            if (ok) {
                // box row j holds step t0 - 3 + j: output step r reads rows r .. r+3
                const char *xs = x_tile + sx * X_STAGE_BYTES + cp * 4;
                char *at = a_tile + ab * A_BYTES;
                // all of this thread's box rows first: a load issued after a store to the tile would have to wait
                // for it (both are shared memory), and the rows' arithmetic would run one after the other
                __nv_bfloat162 xv[ROWS_PER_THREAD + HALO];
#pragma unroll
                for (int j = 0; j < ROWS_PER_THREAD + HALO; ++j)
                    xv[j] = *reinterpret_cast<const __nv_bfloat162 *>(xs + (r0 + j) * (KC * 2));
#pragma unroll
                for (int i = 0; i < ROWS_PER_THREAD; ++i) {
                    const float2 x0 = __bfloat1622float2(xv[i]), x1 = __bfloat1622float2(xv[i + 1]);
                    const float2 x2 = __bfloat1622float2(xv[i + 2]), x3 = __bfloat1622float2(xv[i + 3]);
                    float c0 = fmaf(wa.x, x0.x, ba), c1 = fmaf(wb.x, x0.y, bb);
                    c0 = fmaf(wa.y, x1.x, c0); c1 = fmaf(wb.y, x1.y, c1);
                    c0 = fmaf(wa.z, x2.x, c0); c1 = fmaf(wb.z, x2.y, c1);
                    c0 = fmaf(wa.w, x3.x, c0); c1 = fmaf(wb.w, x3.y, c1);
                    const __nv_bfloat162 o = __floats2bfloat162_rn(silu_tanh(c0), silu_tanh(c1));
                    const int r = r0 + i;
                    // 16-byte chunks of a row are XOR-swizzled with the row index, like the TMA box of an operand
                    *reinterpret_cast<__nv_bfloat162 *>(at + r * 128 + ((((cp >> 2) ^ (r & 7))) << 4) + (cp & 3) * 4) = o;
                }
            }
            fence_proxy_async_smem();  // the tile is read by the tensor core and by the TMA store
            // the store that read the tile of the NEXT block (AB - 1 blocks ago) is done before anyone writes that tile
            if (ct == 0) tma_store_wait_read<AB - 2>();
            bad = compute_sync_or(!ok || *abort_flag != 0);
            if (bad) break;
            if (ct == 0) {
                tma_store_3d(&tm_u, smem_u32(a_tile + ab * A_BYTES), kb * KC, t0, b);
                tma_store_commit();
                mbar_arrive(bar_a_full(ab));
                mbar_arrive(bar_x_empty(sx));
            }
        }
        if (!bad && warp < 6 && (warp & 3) * 32 < TM) {
            // epilogue: warps 2..5 read the tensor-memory lane quarter warp % 4 (those that hold steps of this tile)
            const int wq = warp & 3;
            if (wait_or_abort(bar_acc_full, 0, abort_flag)) {
                tc_fence_after();
                const int t = t0 + wq * 32 + lane;
                __nv_bfloat16 *row = xd + ((int64_t)b * L + t) * ldxd;
                for (int c0 = 0; c0 < n_mma; c0 += 32) {
                    const uint32_t taddr = tmem_base + c0 + ((uint32_t)(wq * 32) << 16);
                    uint32_t r[32];
                    if (n_mma - c0 >= 32) {
                        tmem_ld32(taddr, r);
                        tmem_ld_wait();
                    } else {
                        uint32_t h[16];
                        tmem_ld16(taddr, h);
                        tmem_ld_wait();   // the registers of a tensor-memory load are not to be touched before this
#pragma unroll
                        for (int j = 0; j < 16; ++j) { r[j] = h[j]; r[16 + j] = 0u; }
                    }
                    if (t < L) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            if (c0 + q * 8 < n_out) {   // n_out is a multiple of 8: whole 16-byte groups
                                uint32_t w[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[q * 8 + 2 * e]),
                                                                                     __uint_as_float(r[q * 8 + 2 * e + 1]));
                                    w[e] = *reinterpret_cast<const uint32_t *>(&h2);
                                }
                                *reinterpret_cast<uint4 *>(row + c0 + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        }
                    }
                }
            }
        }
        if (ct == 0) tma_store_wait_all<0>();  // the u tiles must outlive their TMA stores
    }

    // teardown: everybody meets, then the allocating warp frees tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

}  // namespace cx

hx_status read_status_convx(int *v, bool clear) {
    HX_CUDA(cudaMemcpyFromSymbol(v, cx::g_cx_status, sizeof(int)));
    if (clear && *v != 0) {
        const int zero = 0;
        HX_CUDA(cudaMemcpyToSymbol(cx::g_cx_status, &zero, sizeof(int)));
    }
    return HX_OK;
}

}  // namespace hx

namespace hx {
namespace cx {

template <int TM>
static hx_status launch(const void *x, int64_t x_batch_stride, int64_t x_row_stride, const float *conv_w, const float *conv_b,
                        const void *W_x, int64_t ldw, void *u, int64_t u_batch_stride, int64_t u_row_stride, void *x_dbl,
                        int64_t x_dbl_row_stride, int batch, int seq_len, int d_inner, int n_out, cudaStream_t st) {
    CUtensorMap mx, mw, mu;
    hx_status s;
    const uint64_t dims_x[3] = {(uint64_t)d_inner, (uint64_t)seq_len, (uint64_t)batch};
    const uint64_t str_x[2] = {(uint64_t)x_row_stride * 2, (uint64_t)x_batch_stride * 2};
    const uint32_t box_x[3] = {(uint32_t)KC, (uint32_t)Cfg<TM>::X_BOX_ROWS, 1};
    if ((s = encode_tensor_map(&mx, HX_BF16, 3, x, dims_x, str_x, box_x, false)) != HX_OK) return s;
    const int n_mma = (n_out + 15) / 16 * 16;   // W_x rows past n_out are out of range for TMA and read as zeros
    const uint64_t dims_w[2] = {(uint64_t)d_inner, (uint64_t)n_out};
    const uint64_t str_w[1] = {(uint64_t)ldw * 2};
    const uint32_t box_w[2] = {(uint32_t)KC, (uint32_t)n_mma};
    if ((s = encode_tensor_map(&mw, HX_BF16, 2, W_x, dims_w, str_w, box_w, true)) != HX_OK) return s;
    const uint64_t str_u[2] = {(uint64_t)u_row_stride * 2, (uint64_t)u_batch_stride * 2};
    const uint32_t box_u[3] = {(uint32_t)KC, (uint32_t)TM, 1};
    if ((s = encode_tensor_map(&mu, HX_BF16, 3, u, dims_x, str_u, box_u, true)) != HX_OK) return s;
    const int smem = smem_bytes<TM>(n_mma);
    static std::atomic<int> attr_set[64];  // largest size the attribute was set to, per device
    int dev = 0;
    HX_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && attr_set[dev].load(std::memory_order_acquire) < smem) {
        HX_CUDA(cudaFuncSetAttribute(conv_xproj_kernel<TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_set[dev].store(smem, std::memory_order_release);
    }
    uint32_t cols = 32;
    while ((int)cols < n_mma) cols *= 2;
    const int tiles_per_seq = (seq_len + TM - 1) / TM;
    conv_xproj_kernel<TM><<<batch * tiles_per_seq, THREADS, smem, st>>>(mx, mw, mu, conv_w, conv_b, static_cast<__nv_bfloat16 *>(x_dbl),
                                                                       x_dbl_row_stride, seq_len, d_inner, n_out, n_mma,
                                                                       tiles_per_seq, cols);
    return check_launch("conv_xproj_kernel");
}

}  // namespace cx
}  // namespace hx

extern "C" hx_status hx_conv1d_silu_xproj_fwd(const void *x, int64_t x_batch_stride, int64_t x_row_stride, const float *conv_w,
                                              const float *conv_b, const void *W_x, int64_t ldw, void *u, int64_t u_batch_stride,
                                              int64_t u_row_stride, void *x_dbl, int64_t x_dbl_row_stride, int32_t batch,
                                              int32_t seq_len, int32_t d_inner, int32_t d_conv, int32_t n_out, int32_t io_dtype,
                                              void *stream) {
    using namespace hx::cx;
    HX_REQUIRE(batch >= 0 && seq_len >= 0 && d_inner >= 1 && n_out >= 1, HX_ERR_INVALID_DIMENSION,
               "bad dimensions batch %d, seq_len %d, d_inner %d, n_out %d", batch, seq_len, d_inner, n_out);
    if (batch == 0 || seq_len == 0) return HX_OK;
    HX_REQUIRE(x && conv_w && W_x && u && x_dbl, HX_ERR_INVALID_INPUT, "a required operand is NULL");
    auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    // what the kernel is written for; a caller that gets this status runs hx_conv1d_silu_fwd and hx_gemm_bf16
    if (!(io_dtype == HX_BF16 && d_conv == 4 && d_inner % KC == 0 && n_out % 8 == 0 && n_out <= 256 && al16(conv_w) &&
          (!conv_b || al16(conv_b)) && al16(x_dbl) && (x_dbl_row_stride * 2) % 16 == 0 && x_dbl_row_stride >= n_out &&
          (int64_t)batch * ((seq_len + 63) / 64) <= 0x7fffffff))
        return hx::fail(HX_ERR_UNSUPPORTED_OPERATION,
                        "hx_conv1d_silu_xproj_fwd takes bf16, d_conv 4, d_inner a multiple of 64, n_out a multiple of 8 up to 256 "
                        "and 16-byte aligned operands");
    // 128-step tiles, or 64-step ones where the long tiles would leave SMs without a CTA (a CTA walks its channels
    // one block after the other, so a short grid is bound by that chain: 33.7 against 25.5 us at 4 x 2048 x 1536)
    const int64_t long_tiles = (int64_t)batch * ((seq_len + 127) / 128);
    cudaStream_t st = (cudaStream_t)stream;
    if (long_tiles < hx::sm_count())
        return launch<64>(x, x_batch_stride, x_row_stride, conv_w, conv_b, W_x, ldw, u, u_batch_stride, u_row_stride, x_dbl,
                          x_dbl_row_stride, batch, seq_len, d_inner, n_out, st);
    return launch<128>(x, x_batch_stride, x_row_stride, conv_w, conv_b, W_x, ldw, u, u_batch_stride, u_row_stride, x_dbl,
                       x_dbl_row_stride, batch, seq_len, d_inner, n_out, st);
}
