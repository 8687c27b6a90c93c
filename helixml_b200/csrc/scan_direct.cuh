// scan_direct_kernel: the fused selective scan with one lane per channel.
//
// Profiling the lane-split kernel (scan_tiled_kernel) showed where its time goes: shared-memory results
// return to registers at 128 bytes/clk/SM whatever the broadcast, so the fp32 B[t][n], C[t][n] operands every
// lane needs cost one wavefront per 32 floats delivered, and the point-wise results handed between lanes
// through shared-memory records cost as much again.  This kernel removes the records and lets one delivery
// of B/C serve more points:
//   * a lane owns CPL (1 or 2) adjacent channels and keeps all 16 states of each in registers (fp32,
//     packed as 8 x f32x2 per channel); the conv window lives in registers too;
//   * per time step the lane loads B[t][0..15] and C[t][0..15] once (8 x 128-bit broadcast loads) and uses
//     them for its CPL channels, so the delivery per point falls as 1/CPL;
//   * the point-wise math (conv, SiLU, softplus, decay, gate) runs in-line, packed f32x2 over the channel
//     pair when CPL == 2; with geometric A the 16 decays are powers of one exponential;
//   * no shuffles, no shared-memory traffic between lanes.
// The block's call can leave the dt projection to this kernel (dt = dt_low . W_dt^T, no dt tensor in memory): with one
// lane per channel the producer lane issues tcgen05.mma with the CTA's [128 channels x rank] W_dt tile as the M
// operand and the chunk's [16 steps x rank] dt_low rows as the N operand, so the accumulator's lane is the consumer
// lane that owns the channel and a consumer warp fetches its 16 steps of dt with one tcgen05.ld (FUSEDT == 2).
// A warp therefore covers 32*CPL channels; a CTA has 4 such warps plus the producer warp, which issues the
// TMA loads (unswizzled 128-byte-wide boxes: every warp-wide access is one contiguous row) and widens B/C to
// fp32 once per CTA.  y needs no staging: each step a warp writes one contiguous run of 32*CPL channels
// straight from registers.  Bounded waits, carry hand-over for split sequences and the status word are those
// of scan_tiled_kernel.
//
// Split sequences come in two forms.  MODE 0 chains the segments: segment s+1 starts from the state segment s
// hands over (carry + flag), so the segments of one chain run one after the other; that evens out the load when
// chains are plentiful.  MODES 1 and 2 are the look-back form for few chains (geometric A only), two launches in
// stream order with no flag between CTAs:
//   MODE 1, the aggregate pass, runs segments 0 .. S-2 at the same time, each from a zero state and backwards in
//           time: with w_t = exp2(A0 * sum_{tau > t} dt_tau) the end state is q[n] = sum_t (dt_t u_t w_t^(n+1)) B_t[n],
//           i.e. one multiply for the power (the input is folded into the chain of powers) and one FMA per state,
//           no C contraction, no gate, no output.  It writes q and sum(dt) per (segment, chain).
//   MODE 2, the output pass, runs all S segments at the same time: a segment first folds the aggregates of its
//           predecessors, h <- exp(A sum dt_j) h + q_j for j = 0 .. s-1 (the look-back), then scans its steps
//           with outputs like MODE 0.
#pragma once

// Tuning macros (python -m helixml_b200.build --define NAME=VALUE).
// Second argument of __launch_bounds__ for the one-pass / chained kernels and for the look-back passes (0 = none).
// With 1 the compiler schedules for the registers of a single resident CTA and uses about 100 instead of 70: the
// unfused one-pass kernel gets 10 % faster (455 -> 409 us at 49 152 chains, 3 to 4 CTAs still fit an SM); the
// look-back passes, which live on occupancy, are best left alone (a budget for 5 or 6 CTAs per SM spills and is
// 2-5 % slower).
#ifndef HX_SCAN_MINB_CHAINED
#define HX_SCAN_MINB_CHAINED 1
#endif
#ifndef HX_SCAN_UNROLL
#define HX_SCAN_UNROLL 8
#endif
// Whole 16-step chunks run fully unrolled and branch-free where dt arrives in registers (FUSEDT == 2, which needs it)
// and, with this macro at 1, in every one-channel-per-lane instantiation; two channels per lane always keep the step
// loop unrolled by HX_SCAN_UNROLL.  Measured: one channel per lane gains 1-2 % (the block's scan reading dt from memory
// 10.36 -> 10.13 ms per 24 blocks, configuration 2 in the look-back form 681 -> 654 us); two channels per lane lose
// 10-16 % (98 304 chains x 2048 steps 781 -> 894 us, 327 680 chains x 16 384 steps 19.3 -> 23.0 ms).
#ifndef HX_SCAN_FULL_UNROLL
#define HX_SCAN_FULL_UNROLL 1
#endif
#ifndef HX_SCAN_MINB_LOOKBACK
#define HX_SCAN_MINB_LOOKBACK 0
#endif

namespace hx {
namespace scan {

template <typename T, int CPL_, bool GEOM_, bool STD_, int STAGES_, int FUSEDT_ = 0, bool ZGATE_ = false,
          bool BLOCK_ = false, int MODE_ = 0>
struct DirectCfg {
    static constexpr int MODE = MODE_;                 // 0 chained segments, 1 aggregate pass, 2 output pass (see above)
    static constexpr bool BLOCK = BLOCK_;              // the Mamba block's call: no conv (u is given), gate and softplus
                                                       // present, all known at compile time
    static constexpr bool ZGATE = ZGATE_;              // z is known at compile time to hold silu(z) already
    // dt = dt_low . W_dt^T computed inside the kernel (bf16 only).  1: the producer warp runs mma.sync and writes an fp32
    // dt tile to shared memory.  2: one producer lane issues tcgen05.mma with the CTA's W_dt tile as the M = 128 operand
    // (one row per channel) and the chunk's dt_low rows as the N = 16 operand; the accumulator's lane IS the consumer
    // lane that owns the channel, so a consumer warp fetches its 16 steps of dt with one tcgen05.ld and no dt ever
    // touches shared memory (one lane per channel only).
    static constexpr int FUSEDT = FUSEDT_;
    static constexpr int TMEM_COLS = STAGES_ * 16 <= 32 ? 32 : 64;   // FUSEDT == 2: STAGES accumulators of TC columns
    static constexpr int RP = 64;                      // columns of the dt_low / W_dt tiles (dt_rank <= 64, zero filled)
    static constexpr int CPL = CPL_;
    static constexpr bool GEOM = GEOM_;
    static constexpr bool STD = STD_;
    static constexpr bool FAST = sizeof(T) == 2;
    static constexpr int ES = sizeof(T);
    static constexpr int TC = 16;                      // time steps per chunk
    static constexpr int STAGES = STAGES_;
    static constexpr int NWARP = 4;                    // consumer warps
    static constexpr int BOXC = 128 / ES;              // channels per 128-byte box
    static constexpr int WC = 32 * CPL;                // channels per warp
    static constexpr int WPB = BOXC / WC;              // warps per box (1 or 2)
    static constexpr int NB = NWARP / WPB;             // boxes per CTA
    static constexpr int DT = NB * BOXC;               // channels per CTA
    static constexpr int THREADS = (NWARP + 1) * 32;
    // second argument of __launch_bounds__ (0 = none): the register budget the compiler schedules for
    static constexpr int UNROLL = HX_SCAN_UNROLL;
    static constexpr bool FULL = FUSEDT_ == 2 || (HX_SCAN_FULL_UNROLL && CPL_ == 1);   // whole chunks fully unrolled
    static constexpr int REM_UNROLL = FULL ? 1 : HX_SCAN_UNROLL;                       // the loop they do not take
    static constexpr int MIN_CTAS = (MODE_ != 0 && !FUSEDT_) ? HX_SCAN_MINB_LOOKBACK : HX_SCAN_MINB_CHAINED;
    static constexpr int X_BYTES = (TC + 3) * 128;
    static constexpr int ROW_BYTES = TC * 128;
    static constexpr int DTROW = FUSEDT == 1 ? BOXC * 4 + 32 : 128;       // bytes per dt row (fp32 + pad when produced here:
                                                                          // the pad spreads the producer's stores over banks)
    static constexpr int DTT_BYTES = FUSEDT == 2 ? 0 : TC * DTROW;        // no dt rows at all when dt arrives in registers
    static constexpr int BOX_BYTES = X_BYTES + ROW_BYTES + DTT_BYTES;     // x, z, dt of one box
    static constexpr int BC_BYTES = (TC * 16 * ES + 127) / 128 * 128;
    static constexpr int BCF_BYTES = TC * 16 * 4;
    static constexpr int DTLOW_BYTES = FUSEDT ? TC * RP * 2 : 0;          // [TC][RP] bf16
    static constexpr int WDT_BYTES = FUSEDT ? DT * RP * 2 : 0;            // [DT][RP] bf16, once per CTA
    static constexpr int STAGE_RAW = NB * BOX_BYTES + 2 * BC_BYTES + 2 * BCF_BYTES + DTLOW_BYTES;
    static constexpr int STAGE_BYTES = FUSEDT ? (STAGE_RAW + 1023) / 1024 * 1024 : STAGE_RAW;  // swizzled tile first
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + WDT_BYTES + 128 + (FUSEDT ? 1024 : 128);
    static_assert(WC * ES <= 128, "a warp's channels must fit one 128-byte box");
    static_assert(3 * STAGES + 2 <= 12, "barrier area too small");
    static_assert(!FUSEDT || sizeof(T) == 2, "the fused dt projection takes bf16 operands");
    static_assert(FUSEDT != 2 || (CPL_ == 1 && DT == 128 && STAGES_ * TC <= TMEM_COLS),
                  "the tensor-memory form maps channel c of the CTA to accumulator lane c");
    static_assert(MODE == 0 || GEOM, "the look-back passes need geometric A");
};

template <typename T> __device__ __forceinline__ float2 ld_chan2(const char *p);  // two adjacent channels
template <> __device__ __forceinline__ float2 ld_chan2<float>(const char *p) { return *reinterpret_cast<const float2 *>(p); }
template <> __device__ __forceinline__ float2 ld_chan2<__nv_bfloat16>(const char *p) {
    const uint32_t v = *reinterpret_cast<const uint32_t *>(p);
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
template <typename T> __device__ __forceinline__ float ld_chan1(const char *p);
template <> __device__ __forceinline__ float ld_chan1<float>(const char *p) { return *reinterpret_cast<const float *>(p); }
template <> __device__ __forceinline__ float ld_chan1<__nv_bfloat16>(const char *p) {
    return __uint_as_float((uint32_t)(*reinterpret_cast<const uint16_t *>(p)) << 16);
}

template <typename T, typename Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::MIN_CTAS)
scan_direct_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_dt,
                   const __grid_constant__ CUtensorMap tm_z, const __grid_constant__ CUtensorMap tm_B,
                   const __grid_constant__ CUtensorMap tm_C, const __grid_constant__ CUtensorMap tm_dtlow,
                   const __grid_constant__ CUtensorMap tm_wdt, const TiledParams p, T *__restrict__ yg, const int64_t y_bs,
                   const int64_t y_rs) {
    constexpr int CPL = Cfg::CPL, TC = Cfg::TC, STAGES = Cfg::STAGES, NW = Cfg::NWARP, NB = Cfg::NB, ES = Cfg::ES;
    constexpr bool GEOM = Cfg::GEOM, FAST = Cfg::FAST, STD = Cfg::STD;
    constexpr int FUSEDT = Cfg::FUSEDT;
    constexpr bool BLOCK = Cfg::BLOCK;
    constexpr int MODE = Cfg::MODE;
    const bool has_conv = !BLOCK && (STD || p.K > 0), has_z = MODE != 1 && (STD || BLOCK || p.has_z),
               use_softplus = STD || BLOCK || p.dt_softplus;
    const bool z_gate = Cfg::ZGATE || p.z_gate;

    extern __shared__ __align__(16) char smem_raw[];
    // aligned by pointer arithmetic (keeps the shared address space): 1024 bytes when the swizzled W_dt tile is
    // present, 128 otherwise
    constexpr uint32_t ALIGN = FUSEDT ? 1024u : 128u;
    char *smem = smem_raw + ((ALIGN - (smem_u32(smem_raw) & (ALIGN - 1))) & (ALIGN - 1));
    char *wdt_tile = smem;  // [DT][64] bf16, 128-byte swizzle (row r: 16-byte chunk c sits at c ^ (r & 7))
    char *stage_base = smem + Cfg::WDT_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(stage_base + STAGES * Cfg::STAGE_BYTES);
    const uint32_t bar0 = smem_u32(bars);
    auto bar_full = [&](int s) { return bar0 + 8u * s; };
    auto bar_ready = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto bar_empty = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };
    const uint32_t bar_w = bar0 + 8u * (3 * STAGES);  // W_dt tile landed
    const uint32_t bar_tdone = bar0 + 8u * (3 * STAGES + 1);  // FUSEDT == 2: consumer warps are done with tensor memory
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 12);
    // stage layout: [dt_low tile (fused dt only, 1024-aligned for its swizzle)] [boxes] [B, C raw] [B, C fp32]
    constexpr int OFF_DTLOW = 0, OFF_BOX0 = Cfg::DTLOW_BYTES;
    constexpr int OFF_BC = OFF_BOX0 + NB * Cfg::BOX_BYTES, OFF_C = OFF_BC + Cfg::BC_BYTES, OFF_BF = OFF_C + Cfg::BC_BYTES,
                  OFF_CF = OFF_BF + Cfg::BCF_BYTES;
    constexpr int OFF_Z = Cfg::X_BYTES, OFF_DTT = Cfg::X_BYTES + Cfg::ROW_BYTES;  // inside a box: x, z, dt

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, b = blockIdx.y, seg = blockIdx.z + p.seg_base;
    const int d0 = tile * Cfg::DT;
    const int t_seg0 = seg * p.seg_len;
    const int t_seg1 = min(p.L, t_seg0 + p.seg_len);
    const int nchunks = (t_seg1 - t_seg0 + TC - 1) / TC;
    // boxes that hold at least one real channel (the others are neither loaded nor stored)
    const int live_boxes = min(NB, (p.D - d0 + Cfg::BOXC - 1) / Cfg::BOXC);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_ready(s), FUSEDT == 2 ? 2 : 1);  // the producer warp's arrival, and the MMA's commit
            mbar_init(bar_empty(s), NW);
        }
        mbar_init(bar_w, 1);
        mbar_init(bar_tdone, NW);
        mbar_fence_init();
    }
    uint32_t tmem_base = 0;
    if constexpr (FUSEDT == 2) {
        if (warp == NW) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                         "r"((uint32_t)Cfg::TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        tc::tc_fence_before();
    }
    __syncthreads();
    if constexpr (FUSEDT == 2) {
        tc::tc_fence_after();
        tmem_base = *tmem_slot;
    }

    if (warp == NW) {
        // ================================================================ producer warp
        if (lane == 0) {
            tma_prefetch_desc(&tm_x);
            tma_prefetch_desc(&tm_dt);
            tma_prefetch_desc(&tm_B);
            tma_prefetch_desc(&tm_C);
            if (has_z) tma_prefetch_desc(&tm_z);
        }
        // the aggregate pass reads neither z nor C
        const uint32_t stage_tx = live_boxes * ((TC + 3) * 128 + TC * 128 * ((has_z ? 1 : 0) + (FUSEDT ? 0 : 1))) +
                                  (MODE == 1 ? 1 : 2) * TC * 16 * ES + Cfg::DTLOW_BYTES;
        if constexpr (FUSEDT) {
            if (lane == 0) {
                tma_prefetch_desc(&tm_dtlow);
                tma_prefetch_desc(&tm_wdt);
                mbar_expect_tx(bar_w, Cfg::WDT_BYTES);
                tma_load_2d(smem_u32(wdt_tile), &tm_wdt, bar_w, 0, d0);  // rows past d_inner arrive as zeros
            }
        }
        auto issue = [&](int i) {
            const int s = i % STAGES;
            const int t0 = t_seg0 + (MODE == 1 ? nchunks - 1 - i : i) * TC;  // the aggregate pass walks backwards
            const uint32_t sb = smem_u32(stage_base + s * Cfg::STAGE_BYTES);
            mbar_expect_tx(bar_full(s), stage_tx);
            for (int bx = 0; bx < live_boxes; ++bx) {
                const uint32_t bb = sb + OFF_BOX0 + bx * Cfg::BOX_BYTES;
                const int dc = d0 + bx * Cfg::BOXC;
                tma_load_3d(bb, &tm_x, bar_full(s), dc, t0 - 3, b);
                if (has_z) tma_load_3d(bb + OFF_Z, &tm_z, bar_full(s), dc, t0, b);
                if constexpr (!FUSEDT) tma_load_3d(bb + OFF_DTT, &tm_dt, bar_full(s), dc, t0, b);
            }
            if constexpr (FUSEDT) tma_load_3d(sb + OFF_DTLOW, &tm_dtlow, bar_full(s), 0, t0, b);
            tma_load_3d(sb + OFF_BC, &tm_B, bar_full(s), 0, t0, b);
            if constexpr (MODE != 1) tma_load_3d(sb + OFF_C, &tm_C, bar_full(s), 0, t0, b);
        };
        int issued = 0;
        for (; issued < STAGES && issued < nchunks; ++issued)
            if (lane == 0) issue(issued);
        int fail_code = 0;
        if constexpr (FUSEDT) {
            const bool okw = mbar_wait(bar_w, 0);
            if (!__all_sync(0xffffffffu, okw)) fail_code = kWaitFull;
        }
        for (int i = 0; i <= nchunks && !fail_code; ++i) {
            if (i < nchunks) {
                const int s = i % STAGES;
                const bool ok = mbar_wait(bar_full(s), (i / STAGES) & 1);
                if (!__all_sync(0xffffffffu, ok)) { fail_code = kWaitFull; break; }
                char *st = stage_base + s * Cfg::STAGE_BYTES;
                if constexpr (FUSEDT == 2) {
                    // dt^T[DT channels][16 steps] = W_dt[DT][RP] . dt_low[16][RP]^T into tensor memory: lane = channel
                    if (lane == 0) {
                        tc::tc_fence_after();
                        const uint64_t da = tc::make_smem_desc(smem_u32(wdt_tile));
                        const uint64_t db = tc::make_smem_desc(smem_u32(st + OFF_DTLOW));
                        const uint32_t idesc = tc::idesc_bf16(128, TC);
                        const int ksteps = (p.dt_rank + 15) >> 4;
                        for (int k = 0; k < ksteps; ++k)
                            tc::umma_bf16(tmem_base + s * TC, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, k ? 1u : 0u);
                        tc::umma_commit(bar_ready(s));
                    }
                } else if constexpr (FUSEDT == 1) {
                    // dt[16 steps][DT channels] = dt_low[16][RP] . W_dt[DT][RP]^T on the tensor cores
                    // (mma.sync m16n8k16, bf16 in, fp32 out), written as the fp32 dt tile of every box
                    constexpr int RPB = Cfg::RP * 2;  // row bytes of both operand tiles
                    const int g = lane >> 2, tid = lane & 3;
                    const int ksteps = (p.dt_rank + 15) >> 4;
                    const char *dl = st + OFF_DTLOW + 2 * tid * 2;  // swizzled like the W_dt tile
                    uint32_t af[4][4];
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const int c0 = ((2 * kk) ^ g) << 4, c1 = ((2 * kk + 1) ^ g) << 4;  // (g + 8) & 7 == g
                        af[kk][0] = *reinterpret_cast<const uint32_t *>(dl + g * RPB + c0);
                        af[kk][1] = *reinterpret_cast<const uint32_t *>(dl + (g + 8) * RPB + c0);
                        af[kk][2] = *reinterpret_cast<const uint32_t *>(dl + g * RPB + c1);
                        af[kk][3] = *reinterpret_cast<const uint32_t *>(dl + (g + 8) * RPB + c1);
                    }
#pragma unroll 2
                    for (int nt = 0; nt < Cfg::DT / 8; ++nt) {
                        float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
                        // row nt*8+g of the swizzled tile: (row & 7) == g, so the eight rows a load touches
                        // land in eight different 16-byte chunks (no bank conflict)
                        const char *wr = wdt_tile + (nt * 8 + g) * RPB + 2 * tid * 2;
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            if (kk < ksteps) {
                                const uint32_t b0 = *reinterpret_cast<const uint32_t *>(wr + (((2 * kk) ^ g) << 4));
                                const uint32_t b1 = *reinterpret_cast<const uint32_t *>(wr + (((2 * kk + 1) ^ g) << 4));
                                asm volatile(
                                    "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
                                    "{%8, %9}, {%0, %1, %2, %3};"
                                    : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
                                    : "r"(af[kk][0]), "r"(af[kk][1]), "r"(af[kk][2]), "r"(af[kk][3]), "r"(b0), "r"(b1));
                            }
                        }
                        const int bx = (nt * 8) / Cfg::BOXC, col = (nt * 8) % Cfg::BOXC + 2 * tid;
                        char *dtt = st + OFF_BOX0 + bx * Cfg::BOX_BYTES + OFF_DTT + col * 4;
                        *reinterpret_cast<float2 *>(dtt + g * Cfg::DTROW) = make_float2(c0, c1);
                        *reinterpret_cast<float2 *>(dtt + (g + 8) * Cfg::DTROW) = make_float2(c2, c3);
                    }
                }
                // widen B and C of this chunk to fp32: TC*16 values per array, 8 per lane per round
                constexpr int ROUNDS = TC * 16 * 2 / (32 * 8);
#pragma unroll
                for (int r = 0; r < ROUNDS; ++r) {
                    const int e0 = (r * 32 + lane) * 8;
                    const int arr = e0 / (TC * 16), ea = e0 % (TC * 16);
                    if (MODE == 1 && arr) continue;  // C is not loaded in the aggregate pass
                    const char *src = st + (arr ? OFF_C : OFF_BC) + ea * ES;
                    float *dst = reinterpret_cast<float *>(st + (arr ? OFF_CF : OFF_BF)) + ea;
                    if constexpr (ES == 2) {
                        const uint4 raw = *reinterpret_cast<const uint4 *>(src);
                        *reinterpret_cast<float4 *>(dst) =
                            make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                        __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
                        *reinterpret_cast<float4 *>(dst + 4) =
                            make_float4(__uint_as_float(raw.z << 16), __uint_as_float(raw.z & 0xffff0000u),
                                        __uint_as_float(raw.w << 16), __uint_as_float(raw.w & 0xffff0000u));
                    } else {
                        *reinterpret_cast<float4 *>(dst) = *reinterpret_cast<const float4 *>(src);
                        *reinterpret_cast<float4 *>(dst + 4) = *reinterpret_cast<const float4 *>(src + 16);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_ready(s));
            }
            if (i >= 1 && issued < nchunks) {
                // refill the stage chunk i-1 used once every consumer warp has released it
                const int j = i - 1;
                int fc = 0;
                if (lane == 0) {
                    if (!mbar_wait(bar_empty(j % STAGES), (j / STAGES) & 1)) {
                        fc = kWaitEmpty;
                    } else {
                        issue(issued);
                    }
                }
                fc = __shfl_sync(0xffffffffu, fc, 0);
                if (fc) { fail_code = fc; break; }
                ++issued;
            }
        }
        if (lane == 0 && fail_code) {
            atomicOr(&g_wait_status, fail_code);
            // let loads already in flight land before the CTA's shared memory goes away
            for (int i = 0; i < issued; ++i) mbar_wait(bar_full(i % STAGES), (i / STAGES) & 1);
        }
        if constexpr (FUSEDT == 2) {
            // tensor memory goes back once the consumer warps have read their last chunk (a bounded wait: a consumer
            // that gave up never arrives)
            if (lane == 0) mbar_wait(bar_tdone, 0);
            __syncwarp();
            tc::tc_fence_after();
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS)
                         : "memory");
        }
        return;
    }

    // ==================================================================== consumer warps
    const int box = warp / Cfg::WPB;                                   // box this warp reads
    const int lane_byte = ((warp % Cfg::WPB) * Cfg::WC + lane * CPL) * ES;  // byte offset of the lane in a box row
    const int dch = d0 + box * Cfg::BOXC + (warp % Cfg::WPB) * Cfg::WC + lane * CPL;  // first channel of the lane

    float w_[CPL][4], cb_[CPL], db_[CPL], ds_[CPL], a0_[CPL];
    float a2l[GEOM ? 1 : CPL][16];
#pragma unroll
    for (int e = 0; e < CPL; ++e) {
        const int d = dch + e;
        const bool okc = d < p.D;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int src = j - (4 - p.K);
            w_[e][j] = (okc && p.K > 0 && src >= 0) ? p.conv_w[(int64_t)d * p.K + src] : 0.f;
        }
        cb_[e] = (okc && p.K > 0 && p.conv_b) ? p.conv_b[d] : 0.f;
        db_[e] = (okc && p.dt_bias) ? p.dt_bias[d] : 0.f;
        ds_[e] = (okc && p.Dskip) ? p.Dskip[d] : 0.f;
        a0_[e] = okc ? p.A[(int64_t)d * 16] * kLog2e : 0.f;
        if constexpr (!GEOM) {
#pragma unroll
            for (int n = 0; n < 16; ++n) a2l[e][n] = okc ? p.A[(int64_t)d * 16 + n] * kLog2e : 0.f;
        }
    }

    // both channels in range and the pair 4-/8-byte aligned in y: one vector store per step
    const bool pair_ok = CPL == 2 && dch + 1 < p.D && ((y_rs * ES) % (2 * ES) == 0) && ((y_bs * ES) % (2 * ES) == 0) &&
                         ((reinterpret_cast<uintptr_t>(yg) % (2 * ES)) == 0);
    float2 h[CPL][8];
#pragma unroll
    for (int e = 0; e < CPL; ++e)
#pragma unroll
        for (int j = 0; j < 8; ++j) h[e][j] = make_float2(0.f, 0.f);

    if constexpr (MODE == 1) {
        // ============================================================ aggregate pass (look-back form)
        // End state of this segment from a zero state, walking backwards: w = exp2(A0 * (sum of dt after t)) is the
        // decay from step t to the end of the segment, and q[n] += (dt_t u_t w^(n+1)) B_t[n].
        float sacc[CPL];
        float2 q[CPL][8];
#pragma unroll
        for (int e = 0; e < CPL; ++e) {
            sacc[e] = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) q[e][j] = make_float2(0.f, 0.f);
        }
        for (int i = 0; i < nchunks; ++i) {
            const int s = i % STAGES;
            const int c = nchunks - 1 - i;
            if (!mbar_wait(bar_ready(s), (i / STAGES) & 1)) {
                if (lane == 0) atomicOr(&g_wait_status, kWaitFull);
                return;
            }
            const char *sbox = stage_base + s * Cfg::STAGE_BYTES + OFF_BOX0 + box * Cfg::BOX_BYTES;
            const char *sx = sbox + lane_byte;  // row r = step r - 3 of the chunk
            const char *sd = sbox + OFF_DTT + (FUSEDT ? (lane_byte / ES) * 4 : lane_byte);
            constexpr int DROW = Cfg::DTROW;
            const float4 *sBf = reinterpret_cast<const float4 *>(stage_base + s * Cfg::STAGE_BYTES + OFF_BF);
            const int steps = min(TC, t_seg1 - (t_seg0 + c * TC));
            uint32_t dtreg[16];
            if constexpr (FUSEDT == 2) {
                // this lane's channel, the chunk's 16 steps: one row of the accumulator
                tc::tc_fence_after();
                tc::tmem_ld16(tmem_base + s * TC + ((uint32_t)(warp * 32) << 16), dtreg);
                tc::tmem_ld_wait();
            }
            // conv window for the walk backwards: x of the three steps that follow the row read next
            float xa[CPL], xb[CPL], xc3[CPL];
#pragma unroll
            for (int e = 0; e < CPL; ++e) {
                xa[e] = ld_chan1<T>(sx + (steps + 2) * 128 + e * ES);
                xb[e] = ld_chan1<T>(sx + (steps + 1) * 128 + e * ES);
                xc3[e] = ld_chan1<T>(sx + steps * 128 + e * ES);
            }
            auto back_step = [&](const int t, const float dt_reg) {
                float xn[CPL], dr[CPL];
#pragma unroll
                for (int e = 0; e < CPL; ++e) {
                    xn[e] = ld_chan1<T>(sx + t * 128 + e * ES);  // x three steps before step t
                    if constexpr (FUSEDT == 2) dr[e] = dt_reg;
                    else if constexpr (FUSEDT == 1) dr[e] = *reinterpret_cast<const float *>(sd + t * DROW + e * 4);
                    else dr[e] = ld_chan1<T>(sd + t * DROW + e * ES);
                }
                float4 Bv[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) Bv[k] = sBf[t * 4 + k];
#pragma unroll
                for (int e = 0; e < CPL; ++e) {
                    float u;
                    if (has_conv) {
                        float cv = cb_[e];
                        cv = fmaf(w_[e][0], xn[e], cv);
                        cv = fmaf(w_[e][1], xc3[e], cv);
                        cv = fmaf(w_[e][2], xb[e], cv);
                        cv = fmaf(w_[e][3], xa[e], cv);
                        u = silu_sel<FAST>(cv);
                    } else {
                        u = xa[e];
                    }
                    xa[e] = xb[e]; xb[e] = xc3[e]; xc3[e] = xn[e];
                    const float v = dr[e] + db_[e];
                    float dtv;
                    if (use_softplus) {
                        if constexpr (FAST) {
                            const float sp = kLn2 * lg2_approx(1.f + ex2_approx(v * kLog2e));
                            dtv = v > 20.f ? v : sp;
                        } else {
                            dtv = softplus_acc(v);
                        }
                    } else {
                        dtv = v;
                    }
                    const float xin = dtv * u;
                    float r;
                    if constexpr (FAST) r = ex2_approx(sacc[e] * a0_[e]);
                    else r = exp2f(sacc[e] * a0_[e]);
                    sacc[e] += dtv;
                    const float r2 = r * r, r4 = r2 * r2, r8 = r4 * r4;
                    float2 a[8];
                    a[0] = mul2(make_float2(r, r2), splat2(xin));
                    a[1] = mul2(a[0], splat2(r2));
                    a[2] = mul2(a[0], splat2(r4));
                    a[3] = mul2(a[1], splat2(r4));
#pragma unroll
                    for (int j = 0; j < 4; ++j) a[4 + j] = mul2(a[j], splat2(r8));
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        q[e][2 * k] = fma2(a[2 * k], make_float2(Bv[k].x, Bv[k].y), q[e][2 * k]);
                        q[e][2 * k + 1] = fma2(a[2 * k + 1], make_float2(Bv[k].z, Bv[k].w), q[e][2 * k + 1]);
                    }
                }
            };
            // whole chunks fully unrolled, the ragged one through the plain loop (see the output pass below)
            if (steps == TC && Cfg::FULL) {
#pragma unroll
                for (int t = TC - 1; t >= 0; --t) back_step(t, FUSEDT == 2 ? __uint_as_float(dtreg[t]) : 0.f);
            } else if constexpr (FUSEDT == 2) {
                float dtl[TC];
#pragma unroll
                for (int t = 0; t < TC; ++t) dtl[t] = __uint_as_float(dtreg[t]);
#pragma unroll 1
                for (int t = steps - 1; t >= 0; --t) back_step(t, dtl[t]);
            } else {
#pragma unroll(Cfg::REM_UNROLL)
                for (int tt = 0; tt < steps; ++tt) back_step(steps - 1 - tt, 0.f);
            }
            if constexpr (FUSEDT == 2) tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty(s));
        }
#pragma unroll
        for (int e = 0; e < CPL; ++e) {
            if (dch + e >= p.D) continue;
            const int64_t ci = ((int64_t)seg * p.B + b) * p.D + dch + e;
            float2 *dst = reinterpret_cast<float2 *>(p.carry + ci * 16);
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[j] = q[e][j];
            p.sdt[ci] = sacc[e];
        }
        if constexpr (FUSEDT == 2) {
            if (lane == 0) mbar_arrive(bar_tdone);
        }
        return;
    }

    if constexpr (MODE == 2) {
        // ============================================================ look-back: fold the predecessors' aggregates
        if (seg > 0) {
#pragma unroll
            for (int e = 0; e < CPL; ++e) {
                if (dch + e >= p.D) continue;
                const int64_t c0 = (int64_t)b * p.D + dch + e, cs = (int64_t)p.B * p.D;
                const float2 *q0 = reinterpret_cast<const float2 *>(p.carry + c0 * 16);
#pragma unroll
                for (int j = 0; j < 8; ++j) h[e][j] = q0[j];  // segment 0 starts from zero: its aggregate is its end state
                for (int js = 1; js < seg; ++js) {
                    const float sd = p.sdt[c0 + js * cs];
                    float r;
                    if constexpr (FAST) r = ex2_approx(sd * a0_[e]);
                    else r = exp2f(sd * a0_[e]);
                    float2 a[8];
                    a[0] = make_float2(r, r * r);
                    a[1] = mul2(a[0], splat2(a[0].y));
                    a[2] = mul2(a[0], splat2(a[1].y));
                    a[3] = mul2(a[1], splat2(a[1].y));
#pragma unroll
                    for (int j = 0; j < 4; ++j) a[4 + j] = mul2(a[j], splat2(a[3].y));
                    const float2 *qj = reinterpret_cast<const float2 *>(p.carry + (c0 + js * cs) * 16);
#pragma unroll
                    for (int j = 0; j < 8; ++j) h[e][j] = fma2(a[j], h[e][j], qj[j]);
                }
            }
        }
    }

    if (MODE == 0 && p.n_segments > 1 && seg > 0) {
        const int fidx = (((seg - 1) * p.B + b) * gridDim.x + tile) * 8 + warp;
        bool ok = false;
        const int poll_limit = g_carry_polls;
        for (int it = 0; it < poll_limit; ++it) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p.flags + fidx) : "memory");
            if (v == p.epoch) { ok = true; break; }
            __nanosleep(40);
        }
        if (!ok) {
            if (lane == 0) atomicOr(&g_wait_status, kWaitCarry);
        } else {
#pragma unroll
            for (int e = 0; e < CPL; ++e)
                if (dch + e < p.D) {
                    const float2 *src = reinterpret_cast<const float2 *>(p.carry + ((((int64_t)(seg - 1) * p.B + b) * p.D + dch + e) * 16));
#pragma unroll
                    for (int j = 0; j < 8; ++j) h[e][j] = src[j];
                }
        }
    }

    for (int i = 0; i < nchunks; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(bar_ready(s), (i / STAGES) & 1)) {
            if (lane == 0) atomicOr(&g_wait_status, kWaitFull);
            return;
        }
        const char *sbox = stage_base + s * Cfg::STAGE_BYTES + OFF_BOX0 + box * Cfg::BOX_BYTES;
        const char *sx = sbox + lane_byte;  // row 0 = 3 steps back
        const char *sz = sbox + OFF_Z + lane_byte;
        // dt: the caller's tile (io dtype) or the fp32 tile the producer computed
        const char *sd = sbox + OFF_DTT + (FUSEDT ? (lane_byte / ES) * 4 : lane_byte);
        constexpr int DROW = Cfg::DTROW;  // bytes per dt row
        const float4 *sBf = reinterpret_cast<const float4 *>(stage_base + s * Cfg::STAGE_BYTES + OFF_BF);
        const float4 *sCf = reinterpret_cast<const float4 *>(stage_base + s * Cfg::STAGE_BYTES + OFF_CF);
        const int steps = min(TC, t_seg1 - (t_seg0 + i * TC));
        T *yrow = yg + (int64_t)b * y_bs + (int64_t)(t_seg0 + i * TC) * y_rs + dch;  // this lane's first output
        uint32_t dtreg[16];
        if constexpr (FUSEDT == 2) {
            // this lane's channel, the chunk's 16 steps: one row of the accumulator
            tc::tc_fence_after();
            tc::tmem_ld16(tmem_base + s * TC + ((uint32_t)(warp * 32) << 16), dtreg);
            tc::tmem_ld_wait();
        }

        // conv window: the three steps before the chunk come from the halo rows
        float xw[CPL][3];
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            if constexpr (CPL == 2) {
                const float2 v = ld_chan2<T>(sx + k * 128);
                xw[0][k] = v.x;
                xw[1][k] = v.y;
            } else {
                xw[0][k] = ld_chan1<T>(sx + k * 128);
            }
        }

        auto fwd_step = [&](const int t, const float dt_reg) {
            float xc[CPL], dr[CPL], zr[CPL];
            if constexpr (CPL == 2) {
                const float2 vx = ld_chan2<T>(sx + (t + 3) * 128);
                float2 vd;
                if constexpr (FUSEDT == 1) vd = *reinterpret_cast<const float2 *>(sd + t * DROW);
                else vd = ld_chan2<T>(sd + t * DROW);
                xc[0] = vx.x; xc[1] = vx.y; dr[0] = vd.x; dr[1] = vd.y;
                if (has_z) {
                    const float2 vz = ld_chan2<T>(sz + t * 128);
                    zr[0] = vz.x; zr[1] = vz.y;
                }
            } else {
                xc[0] = ld_chan1<T>(sx + (t + 3) * 128);
                if constexpr (FUSEDT == 2) dr[0] = dt_reg;
                else if constexpr (FUSEDT == 1) dr[0] = *reinterpret_cast<const float *>(sd + t * DROW);
                else dr[0] = ld_chan1<T>(sd + t * DROW);
                if (has_z) zr[0] = ld_chan1<T>(sz + t * 128);
            }
            // B and C of this step, shared by the lane's channels
            float4 Bv[4], Cv[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                Bv[k] = sBf[t * 4 + k];
                Cv[k] = sCf[t * 4 + k];
            }
            float yout[CPL];
#pragma unroll
            for (int e = 0; e < CPL; ++e) {
                // ---- point-wise
                float u;
                if (has_conv) {
                    float c = cb_[e];
                    c = fmaf(w_[e][0], xw[e][0], c);
                    c = fmaf(w_[e][1], xw[e][1], c);
                    c = fmaf(w_[e][2], xw[e][2], c);
                    c = fmaf(w_[e][3], xc[e], c);
                    u = silu_sel<FAST>(c);
                } else {
                    u = xc[e];
                }
                xw[e][0] = xw[e][1]; xw[e][1] = xw[e][2]; xw[e][2] = xc[e];
                const float v = dr[e] + db_[e];
                float dtv;
                if (use_softplus) {
                    if constexpr (FAST) {
                        const float sp = kLn2 * lg2_approx(1.f + ex2_approx(v * kLog2e));
                        dtv = v > 20.f ? v : sp;
                    } else {
                        dtv = softplus_acc(v);
                    }
                } else {
                    dtv = v;
                }
                const float g = has_z ? (z_gate ? zr[e] : silu_sel<FAST>(zr[e])) : 1.f;
                const float xin = dtv * u;
                // ---- decays
                float2 a[8];
                if constexpr (GEOM) {
                    float r;
                    if constexpr (FAST) r = ex2_approx(dtv * a0_[e]);
                    else r = exp2f(dtv * a0_[e]);
                    const float r2 = r * r;
                    a[0] = make_float2(r, r2);
                    a[1] = mul2(a[0], splat2(r2));
                    const float r4 = a[1].y;
                    a[2] = mul2(a[0], splat2(r4));
                    a[3] = mul2(a[1], splat2(r4));
                    const float r8 = a[3].y;
#pragma unroll
                    for (int j = 0; j < 4; ++j) a[4 + j] = mul2(a[j], splat2(r8));
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if constexpr (FAST)
                            a[j] = make_float2(ex2_approx(dtv * a2l[GEOM ? 0 : e][2 * j]), ex2_approx(dtv * a2l[GEOM ? 0 : e][2 * j + 1]));
                        else
                            a[j] = make_float2(exp2f(dtv * a2l[GEOM ? 0 : e][2 * j]), exp2f(dtv * a2l[GEOM ? 0 : e][2 * j + 1]));
                    }
                }
                // ---- recurrence and output contraction, four independent accumulators
                const float2 x2 = splat2(xin);
                float2 acc[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    h[e][2 * k] = fma2(a[2 * k], h[e][2 * k], mul2(x2, make_float2(Bv[k].x, Bv[k].y)));
                    h[e][2 * k + 1] = fma2(a[2 * k + 1], h[e][2 * k + 1], mul2(x2, make_float2(Bv[k].z, Bv[k].w)));
                    acc[0] = fma2(make_float2(Cv[k].x, Cv[k].y), h[e][2 * k], acc[0]);
                    acc[1] = fma2(make_float2(Cv[k].z, Cv[k].w), h[e][2 * k + 1], acc[1]);
                }
                const float2 ys = add2(acc[0], acc[1]);
                yout[e] = (ys.x + ys.y + ds_[e] * u) * g;
            }
            // y goes straight from registers to HBM: the warp writes one contiguous run of 32*CPL channels
            T *yp = yrow + (int64_t)t * y_rs;
            if constexpr (CPL == 2) {
                if (pair_ok) {
                    if constexpr (ES == 2) {
                        const __nv_bfloat162 o = __floats2bfloat162_rn(yout[0], yout[1]);
                        *reinterpret_cast<uint32_t *>(yp) = *reinterpret_cast<const uint32_t *>(&o);
                    } else {
                        *reinterpret_cast<float2 *>(yp) = make_float2(yout[0], yout[1]);
                    }
                } else {
                    if (dch < p.D) st_f32(yp, yout[0]);
                    if (dch + 1 < p.D) st_f32(yp + 1, yout[1]);
                }
            } else {
                if (dch < p.D) st_f32(yp, yout[0]);
            }
        };
        // Whole chunks run fully unrolled with no test between the steps: a loop bound or a predicate per step keeps the
        // compiler from moving a step's loads and special-function results above the previous step's arithmetic, and
        // costs a sixth of the kernel.  The one ragged chunk of a segment takes the plain loop (with dt in registers,
        // FUSEDT == 2, through a local copy: there the step index has to be a compile-time constant).
        if (steps == TC && Cfg::FULL) {
#pragma unroll
            for (int t = 0; t < TC; ++t) fwd_step(t, FUSEDT == 2 ? __uint_as_float(dtreg[t]) : 0.f);
        } else if constexpr (FUSEDT == 2) {
            float dtl[TC];
#pragma unroll
            for (int t = 0; t < TC; ++t) dtl[t] = __uint_as_float(dtreg[t]);
#pragma unroll 1
            for (int t = 0; t < steps; ++t) fwd_step(t, dtl[t]);
        } else {
#pragma unroll(Cfg::REM_UNROLL)
            for (int t = 0; t < steps; ++t) fwd_step(t, 0.f);
        }
        if constexpr (FUSEDT == 2) tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty(s));
    }

    const bool last_seg = seg == p.n_segments - 1;
#pragma unroll
    for (int e = 0; e < CPL; ++e) {
        if (dch + e >= p.D) continue;
        float2 *dst = nullptr;
        if (last_seg && p.h_last) dst = reinterpret_cast<float2 *>(p.h_last + ((int64_t)b * p.D + dch + e) * 16);
        if (MODE == 0 && !last_seg) dst = reinterpret_cast<float2 *>(p.carry + (((int64_t)seg * p.B + b) * p.D + dch + e) * 16);
        if (dst) {
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[j] = h[e][j];
        }
    }
    if (MODE == 0 && !last_seg) {
        __threadfence();
        __syncwarp();
        if (lane == 0) {
            const int fidx = ((seg * p.B + b) * gridDim.x + tile) * 8 + warp;
            asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.flags + fidx), "r"(p.epoch) : "memory");
        }
    }
    if constexpr (FUSEDT == 2) {
        if (lane == 0) mbar_arrive(bar_tdone);
    }
}

}  // namespace scan
}  // namespace hx
