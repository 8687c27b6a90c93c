// Fused selective scan for sm_100a:
//   causal depthwise conv (<= 4 taps) + SiLU, softplus(dt), exp(dt*A) zero-order hold, the scan
//   with fp32 state in registers, the D skip term and the SiLU(z) gate, in one pass over HBM.
//
// Two kernels:
//   scan_simple_kernel  one thread per (batch, channel), any d_state <= 256, accurate libm-style
//                       math.  The parity baseline and the fallback for shapes the tiled kernel
//                       does not take.
//   scan_tiled_kernel   d_state == 16.  A CTA owns one batch row and a 128-byte-wide channel tile
//                       and walks the sequence in chunks.  A producer warp moves [chunk x tile]
//                       boxes of x/dt/z/B/C into shared memory with TMA (3-D tensor maps, 128-byte
//                       swizzle, zero fill outside the tensor gives the conv's causal padding) and
//                       stores finished y tiles back with TMA.  Consumer warps are independent:
//                       each owns 32/LPC channels, the 16 states of a channel are split over LPC
//                       adjacent lanes, and a warp alternates a point-wise phase (conv, SiLU,
//                       softplus, decay; packed f32x2 over channel pairs) with the recurrence phase
//                       (packed f32x2 FMAs over state pairs, partial dot products combined with warp
//                       shuffles).  When A[d][n] = (n+1) A[d][0] the decay exp(dt A[d][n]) is a power
//                       of one exponential, so a point costs 1 exp instead of 16.
//
// The reference has no selective scan to follow (its conv1d is the identity and selective_ssm
// ignores B and C, crates/nn/src/ssm.rs:467-483); the arithmetic is the one written in
// include/helix_b200.h above hx_scan_args.
#include <atomic>
#include <mutex>
#include <vector>

#include "hx_tma.cuh"
#include "hx_tcgen05.cuh"

namespace hx {
namespace scan {

// Per-device status word: a bounded wait that ran out ORs its code in here.
__device__ int g_wait_status = 0;
enum : int { kWaitFull = 1, kWaitEmpty = 2, kWaitOutFull = 4, kWaitOutEmpty = 8, kWaitCarry = 16 };
// Polls (40 ns apart) a segment spends on its predecessor's carry flag before it gives up, records kWaitCarry and
// carries on from a zero state.  The default is about 0.2 s; hx_debug_scan_orphan_segment lowers it for one launch.
constexpr int kCarryPollsDefault = 1 << 22;
__device__ int g_carry_polls = kCarryPollsDefault;

// ------------------------------------------------------------------------------------------
// simple kernel
// ------------------------------------------------------------------------------------------
struct SimpleParams {
    int B, L, D, N, K;
    int dt_softplus;
    int z_gate;  // z already holds silu(z)
    const void *x, *dt, *z, *Bm, *Cm;
    void *y;
    int64_t xb, xr, dtb, dtr, zb, zr, Bb, Br, Cb, Cr, yb, yr;
    const float *A, *Dskip, *conv_w, *conv_b, *dt_bias;
    float *h_last;
};

template <typename T, int NS>
__global__ void __launch_bounds__(128) scan_simple_kernel(SimpleParams p) {
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (d >= p.D) return;
    const T *x = static_cast<const T *>(p.x) + b * p.xb + d;
    const T *dt = static_cast<const T *>(p.dt) + b * p.dtb + d;
    const T *z = p.z ? static_cast<const T *>(p.z) + b * p.zb + d : nullptr;
    const T *Bm = static_cast<const T *>(p.Bm) + b * p.Bb;
    const T *Cm = static_cast<const T *>(p.Cm) + b * p.Cb;
    T *y = static_cast<T *>(p.y) + b * p.yb + d;
    float h[NS], a_row[NS];
#pragma unroll
    for (int n = 0; n < NS; ++n) {
        h[n] = 0.f;
        a_row[n] = n < p.N ? p.A[(int64_t)d * p.N + n] : 0.f;
    }
    float w[4] = {0.f, 0.f, 0.f, 0.f};
    if (p.conv_w)
        for (int j = 0; j < p.K; ++j) w[4 - p.K + j] = p.conv_w[(int64_t)d * p.K + j];
    const float cb = p.conv_b ? p.conv_b[d] : 0.f;
    const float bias = p.dt_bias ? p.dt_bias[d] : 0.f;
    const float dsk = p.Dskip ? p.Dskip[d] : 0.f;
    float x3 = 0.f, x2 = 0.f, x1 = 0.f;  // x[t-3], x[t-2], x[t-1]
    for (int t = 0; t < p.L; ++t) {
        const float x0 = ld_f32(x + t * p.xr);
        float u;
        if (p.conv_w) {
            // taps in ascending order, like the written definition
            float c = cb;
            c += w[0] * x3;
            c += w[1] * x2;
            c += w[2] * x1;
            c += w[3] * x0;
            u = silu_acc(c);
        } else {
            u = x0;
        }
        x3 = x2; x2 = x1; x1 = x0;
        const float v = ld_f32(dt + t * p.dtr) + bias;
        const float dtv = p.dt_softplus ? softplus_acc(v) : v;
        const float xin = dtv * u;
        float acc = 0.f;
#pragma unroll
        for (int n = 0; n < NS; ++n) {
            if (n < p.N) {
                const float bn = ld_f32(Bm + t * p.Br + n);
                const float cn = ld_f32(Cm + t * p.Cr + n);
                h[n] = expf(dtv * a_row[n]) * h[n] + xin * bn;
                acc += cn * h[n];
            }
        }
        acc += dsk * u;
        if (z) {
            const float zv = ld_f32(z + t * p.zr);
            acc *= p.z_gate ? zv : silu_acc(zv);
        }
        st_f32(y + t * p.yr, acc);
    }
    if (p.h_last) {
#pragma unroll
        for (int n = 0; n < NS; ++n)
            if (n < p.N) p.h_last[((int64_t)b * p.D + d) * p.N + n] = h[n];
    }
}

// ------------------------------------------------------------------------------------------
// tiled kernel
// ------------------------------------------------------------------------------------------
struct TiledParams {
    int B, L, D;
    int K;            // conv taps in use (0: no conv, x is u already)
    int has_z;
    int z_gate;       // z already holds silu(z)
    int dt_softplus;
    int n_segments;   // sequence segments (1 unless split)
    int seg_len;      // steps per segment, a multiple of the chunk length
    const float *A, *Dskip, *conv_w, *conv_b, *dt_bias;
    float *h_last;
    float *carry;     // [n_segments-1, B, D, 16] states handed from segment s to s+1
    int *flags;       // [n_segments-1, B, tiles, 8] one per consumer warp, set to `epoch` once its carry is written
    int epoch;
    int dt_rank;      // > 0: dt is produced in the kernel from dt_low and W_dt (direct kernel only)
    int seg_base;     // segment index of grid.z == 0 (0 except in hx_debug_scan_orphan_segment, which launches a
                      // segment without its predecessor)
    float *sdt;       // look-back form: [n_segments-1, B, D] sum of dt over each segment (its aggregate decay is
                      // exp(A * sdt)); `carry` then holds the segments' end states from a zero state
};

template <typename T, int LPC_, bool GEOM_, int TC_, int STAGES_, bool STD_>
struct TiledCfg {
    static constexpr int LPC = LPC_;
    static constexpr bool GEOM = GEOM_;
    static constexpr bool STD = STD_;  // conv (4 taps), softplus and gate all present: no runtime flag tests
    static constexpr bool FAST = sizeof(T) == 2;  // bf16 I/O uses the special-function approximations
    static constexpr int TC = TC_;                // time steps per chunk
    static constexpr int STAGES = STAGES_;
    static constexpr int ES = sizeof(T);
    static constexpr int DT = 128 / ES;           // channels per CTA tile: one 128-byte row
    static constexpr int CW = 32 / LPC;           // channels per consumer warp
    static constexpr int NW = DT / CW;            // consumer warps
    static constexpr int S = 16 / LPC;            // states per lane
    static constexpr int NCH = (CW * ES + 15) / 16;  // 16-byte chunks a warp's channels span
    static constexpr int PPR = CW / 2;            // channel pairs per row
    static constexpr int RPI = 32 / PPR;          // rows one warp-wide access covers
    static constexpr int TS = RPI * NCH;          // time steps per sub-chunk (8 for bf16, 16 for fp32)
    static constexpr int THREADS = (NW + 1) * 32;
    static constexpr bool POW4 = GEOM && LPC == 4;  // records carry r, r^2, r^3, r^4 as separate planes
    // shared memory carve-up (bytes)
    static constexpr int X_BYTES = ((TC + 3) * 128 + 1023) / 1024 * 1024;
    static constexpr int ROW_BYTES = TC * 128;
    static constexpr int BC_BYTES = (TC * 16 * ES + 127) / 128 * 128;  // one raw B or C tile
    static constexpr int BCF_BYTES = TC * 16 * 4;                       // one widened (fp32) B or C tile
    static constexpr int STAGE_BYTES = X_BYTES + 2 * ROW_BYTES + 2 * BC_BYTES + 2 * BCF_BYTES;
    static constexpr int OUT_BYTES = TC * 128;
    // per-warp records of one sub-chunk: RX {decay, x} and GS {gate, skip} as float2 per point, plus
    // (POW4) four planes of powers, each padded by 8 floats so that the planes fall in different banks
    static constexpr int PLANE_FLOATS = TS * CW + 8;
    static constexpr int REC_BYTES = 2 * TS * CW * 8 + (POW4 ? 4 * PLANE_FLOATS * 4 : 0);
    static constexpr int WARP_BYTES = (REC_BYTES + 127) / 128 * 128;
    static constexpr int BAR_BYTES = 128;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * OUT_BYTES + NW * WARP_BYTES + BAR_BYTES + 1024;
    static_assert(TC % TS == 0, "chunk must hold whole sub-chunks");
    static_assert(DT % CW == 0 && NW >= 1, "tile must hold whole warps");
    static_assert(3 * STAGES + 4 <= BAR_BYTES / 8, "barrier area too small");
};

// byte offset of (row, channel) inside a 128-byte-wide tile written by TMA with the 128-byte
// swizzle: the 16-byte chunk index is XORed with (row mod 8).
template <int ES> __device__ __forceinline__ int swz(int row, int ch) {
    const int byte = ch * ES;
    return row * 128 + ((((byte >> 4) ^ (row & 7)) << 4) | (byte & 15));
}

template <typename T> __device__ __forceinline__ float2 ld_pair(const char *tile, int off);
template <> __device__ __forceinline__ float2 ld_pair<float>(const char *tile, int off) {
    return *reinterpret_cast<const float2 *>(tile + off);
}
template <> __device__ __forceinline__ float2 ld_pair<__nv_bfloat16>(const char *tile, int off) {
    const uint32_t v = *reinterpret_cast<const uint32_t *>(tile + off);
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}

template <bool FAST> __device__ __forceinline__ float silu_sel(float x) {
    if constexpr (FAST) return silu_tanh(x);  // bf16 I/O: one special-function result, error below the output rounding
    else return silu_acc(x);
}

template <typename T, typename Cfg>
__global__ void __launch_bounds__(Cfg::THREADS)
scan_tiled_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_dt,
                  const __grid_constant__ CUtensorMap tm_z, const __grid_constant__ CUtensorMap tm_B,
                  const __grid_constant__ CUtensorMap tm_C, const __grid_constant__ CUtensorMap tm_y,
                  const TiledParams p) {
    constexpr int LPC = Cfg::LPC, S = Cfg::S, CW = Cfg::CW, NW = Cfg::NW, TC = Cfg::TC, TS = Cfg::TS;
    constexpr int ES = Cfg::ES, DT = Cfg::DT, STAGES = Cfg::STAGES, NCH = Cfg::NCH, PPR = Cfg::PPR;
    constexpr bool GEOM = Cfg::GEOM, FAST = Cfg::FAST, POW4 = Cfg::POW4, STD = Cfg::STD;
    const bool has_conv = STD || p.K > 0, has_z = STD || p.has_z, use_softplus = STD || p.dt_softplus;

    extern __shared__ __align__(16) char smem_raw[];
    // 1024-byte alignment by pointer arithmetic (an integer round trip would turn every access into a
    // generic load)
    char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    char *stage_base = smem;
    char *out_base = stage_base + STAGES * Cfg::STAGE_BYTES;
    char *warp_base = out_base + 2 * Cfg::OUT_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(warp_base + NW * Cfg::WARP_BYTES);
    // barriers: full[STAGES] (TMA landed), ready[STAGES] (B/C widened), empty[STAGES], out_full[2], out_empty[2]
    const uint32_t bar0 = smem_u32(bars);
    auto bar_full = [&](int s) { return bar0 + 8u * s; };
    auto bar_ready = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto bar_empty = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };
    auto bar_out_full = [&](int b) { return bar0 + 8u * (3 * STAGES + b); };
    auto bar_out_empty = [&](int b) { return bar0 + 8u * (3 * STAGES + 2 + b); };
    // offsets inside a stage
    constexpr int OFF_DT = Cfg::X_BYTES, OFF_Z = OFF_DT + Cfg::ROW_BYTES, OFF_B = OFF_Z + Cfg::ROW_BYTES,
                  OFF_C = OFF_B + Cfg::BC_BYTES, OFF_BF = OFF_C + Cfg::BC_BYTES, OFF_CF = OFF_BF + Cfg::BCF_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, b = blockIdx.y, seg = blockIdx.z + p.seg_base;
    const int d0 = tile * DT;
    const int t_seg0 = seg * p.seg_len;
    const int t_seg1 = min(p.L, t_seg0 + p.seg_len);
    const int nchunks = (t_seg1 - t_seg0 + TC - 1) / TC;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_ready(s), 1);
            mbar_init(bar_empty(s), NW);
        }
        for (int k = 0; k < 2; ++k) {
            mbar_init(bar_out_full(k), NW);
            mbar_init(bar_out_empty(k), 1);
        }
        mbar_fence_init();
    }
    __syncthreads();

    const uint32_t stage_tx = (TC + 3) * 128 + TC * 128 * (has_z ? 2 : 1) + 2 * TC * 16 * ES;

    if (warp == NW) {
        // ================================================================ producer warp
        // lane 0 drives TMA (loads, stores) and the barriers; all 32 lanes widen each stage's B and C
        // tiles to fp32 once for the whole CTA, one chunk ahead of the consumers.
        if (lane == 0) {
            tma_prefetch_desc(&tm_x);
            tma_prefetch_desc(&tm_dt);
            tma_prefetch_desc(&tm_B);
            tma_prefetch_desc(&tm_C);
            tma_prefetch_desc(&tm_y);
            if (has_z) tma_prefetch_desc(&tm_z);
        }
        auto issue = [&](int i) {
            const int s = i % STAGES;
            const int t0 = t_seg0 + i * TC;
            const uint32_t sb = smem_u32(stage_base + s * Cfg::STAGE_BYTES);
            mbar_expect_tx(bar_full(s), stage_tx);
            tma_load_3d(sb, &tm_x, bar_full(s), d0, t0 - 3, b);
            tma_load_3d(sb + OFF_DT, &tm_dt, bar_full(s), d0, t0, b);
            if (has_z) tma_load_3d(sb + OFF_Z, &tm_z, bar_full(s), d0, t0, b);
            tma_load_3d(sb + OFF_B, &tm_B, bar_full(s), 0, t0, b);
            tma_load_3d(sb + OFF_C, &tm_C, bar_full(s), 0, t0, b);
        };
        int issued = 0;
        if (lane == 0)
            for (; issued < STAGES && issued < nchunks; ++issued) issue(issued);
        int fail_code = 0;
        // step i: widen chunk i (if any), then retire chunk i-1 (store its y tile, refill its stage)
        for (int i = 0; i <= nchunks; ++i) {
            if (i < nchunks) {
                const int s = i % STAGES;
                const bool ok = mbar_wait(bar_full(s), (i / STAGES) & 1);
                if (!__all_sync(0xffffffffu, ok)) { fail_code = kWaitFull; break; }
                char *st = stage_base + s * Cfg::STAGE_BYTES;
                // TC*16 elements per array; lane handles 8 consecutive elements per round
                constexpr int ROUNDS = TC * 16 * 2 / (32 * 8);
#pragma unroll
                for (int r = 0; r < ROUNDS; ++r) {
                    const int e0 = (r * 32 + lane) * 8;  // over both arrays
                    const int arr = e0 / (TC * 16), ea = e0 % (TC * 16);
                    const int row = ea / 16, n0 = ea % 16;
                    const char *src = st + (arr ? OFF_C : OFF_B) + (row * 16 + n0) * ES;
                    float vals[8];
                    if constexpr (ES == 2) {
                        const uint4 raw = *reinterpret_cast<const uint4 *>(src);
                        const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            vals[2 * k] = __uint_as_float(wds[k] << 16);
                            vals[2 * k + 1] = __uint_as_float(wds[k] & 0xffff0000u);
                        }
                    } else {
                        const float4 f0 = *reinterpret_cast<const float4 *>(src);
                        const float4 f1 = *reinterpret_cast<const float4 *>(src + 16);
                        vals[0] = f0.x; vals[1] = f0.y; vals[2] = f0.z; vals[3] = f0.w;
                        vals[4] = f1.x; vals[5] = f1.y; vals[6] = f1.z; vals[7] = f1.w;
                    }
                    // lane q of a channel finds its S states (n = q + LPC*j) contiguous at [row][q*S + j]
                    float *dst = reinterpret_cast<float *>(st + (arr ? OFF_CF : OFF_BF)) + row * 16;
#pragma unroll
                    for (int qq = 0; qq < LPC; ++qq) {
                        // elements n0+qq, n0+qq+LPC, ... land at j = (n0+qq)/LPC + m
                        constexpr int PER = 8 / LPC;
                        float *d2 = dst + qq * S + n0 / LPC;
                        if constexpr (PER == 8) {
                            *reinterpret_cast<float4 *>(d2) = make_float4(vals[0], vals[1], vals[2], vals[3]);
                            *reinterpret_cast<float4 *>(d2 + 4) = make_float4(vals[4], vals[5], vals[6], vals[7]);
                        } else if constexpr (PER == 4) {
                            *reinterpret_cast<float4 *>(d2) = make_float4(vals[qq], vals[qq + 2], vals[qq + 4], vals[qq + 6]);
                        } else {
                            *reinterpret_cast<float2 *>(d2) = make_float2(vals[qq], vals[qq + 4]);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_ready(s));
            }
            if (i >= 1) {
                const int j = i - 1, ob = j & 1;
                int fc = 0;
                if (lane == 0) {
                    if (!mbar_wait(bar_out_full(ob), (j >> 1) & 1)) {
                        fc = kWaitOutFull;
                    } else {
                        tma_store_3d(&tm_y, smem_u32(out_base + ob * Cfg::OUT_BYTES), d0, t_seg0 + j * TC, b);
                        tma_store_commit();
                        if (issued < nchunks) {
                            // chunk j has been consumed (its out tile is complete), so its stage is free
                            if (!mbar_wait(bar_empty(j % STAGES), (j / STAGES) & 1)) {
                                fc = kWaitEmpty;
                            } else {
                                issue(issued);
                                ++issued;
                            }
                        }
                        tma_store_wait_read<1>();
                        if (j >= 1) mbar_arrive(bar_out_empty((j - 1) & 1));
                    }
                }
                fc = __shfl_sync(0xffffffffu, fc, 0);
                if (fc) { fail_code = fc; break; }
            }
        }
        if (lane == 0) {
            tma_store_wait_all<0>();
            if (fail_code) {
                atomicOr(&g_wait_status, fail_code);
                // let loads already in flight land before the CTA's shared memory goes away
                for (int i = 0; i < issued; ++i) mbar_wait(bar_full(i % STAGES), (i / STAGES) & 1);
            }
        }
        return;
    }

    // ==================================================================== consumer warps
    char *wsm = warp_base + warp * Cfg::WARP_BYTES;
    float2 *recRX = reinterpret_cast<float2 *>(wsm);                  // [TS][CW] {decay (r or dt), x}
    float2 *recGS = recRX + TS * CW;                                   // [TS][CW] {gate, skip}
    float *recP = reinterpret_cast<float *>(recGS + TS * CW);          // POW4: 4 planes [TS][CW] (+8 pad)

    // ---- point-wise phase: this lane's channel pair
    const int pj = lane % PPR, rs = lane / PPR;
    const int pch = warp * CW + 2 * pj;  // tile-local channel of the pair
    float2 cw[4], cbias, dbias, dskip, a0l2;
    {
        float w_[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float cb_[2] = {0.f, 0.f}, db_[2] = {0.f, 0.f}, ds_[2] = {0.f, 0.f}, a0_[2] = {0.f, 0.f};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int d = d0 + pch + e;
            if (d < p.D) {
                if (p.K > 0) {
                    for (int j = 0; j < p.K; ++j) w_[e][4 - p.K + j] = p.conv_w[(int64_t)d * p.K + j];
                    if (p.conv_b) cb_[e] = p.conv_b[d];
                }
                if (p.dt_bias) db_[e] = p.dt_bias[d];
                if (p.Dskip) ds_[e] = p.Dskip[d];
                a0_[e] = p.A[(int64_t)d * 16] * kLog2e;
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) cw[j] = make_float2(w_[0][j], w_[1][j]);
        cbias = make_float2(cb_[0], cb_[1]);
        dbias = make_float2(db_[0], db_[1]);
        dskip = make_float2(ds_[0], ds_[1]);
        a0l2 = make_float2(a0_[0], a0_[1]);
    }

    // ---- recurrence phase: this lane's channel and state slice.  State j of the lane is
    //      n = q + LPC * j.
    const int c = lane / LPC, q = lane % LPC;
    const int dch = d0 + warp * CW + c;
    float a2l[S];  // A * log2(e) for the general (non-geometric) decay
    if constexpr (!GEOM) {
#pragma unroll
        for (int j = 0; j < S; ++j) a2l[j] = dch < p.D ? p.A[(int64_t)dch * 16 + q + LPC * j] * kLog2e : 0.f;
    }
    float2 h[S / 2];
#pragma unroll
    for (int j = 0; j < S / 2; ++j) h[j] = make_float2(0.f, 0.f);

    // carry-in for a split sequence: wait (bounded) for the previous segment's final state
    if (p.n_segments > 1 && seg > 0) {
        // the same warp index of the previous segment's CTA owns the same channels
        const int fidx = (((seg - 1) * p.B + b) * gridDim.x + tile) * 8 + warp;
        bool ok = false;
        const int poll_limit = g_carry_polls;
        for (int it = 0; it < poll_limit; ++it) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p.flags + fidx) : "memory");
            if (v == p.epoch) { ok = true; break; }
            __nanosleep(200);
        }
        if (!ok) {
            if (lane == 0) atomicOr(&g_wait_status, kWaitCarry);
        } else if (dch < p.D) {
            const float *src = p.carry + ((((int64_t)(seg - 1) * p.B + b) * p.D + dch) * 16);
#pragma unroll
            for (int j = 0; j < S / 2; ++j) h[j] = make_float2(src[q + LPC * (2 * j)], src[q + LPC * (2 * j + 1)]);
        }
    }

    // byte offsets of this lane's loads inside a sub-chunk, swizzle included.  A sub-chunk starts at a
    // row that is a multiple of 8, so the swizzle phase depends on the lane and the pass only.
    int xoff[NCH][4], doff[NCH];
#pragma unroll
    for (int pass = 0; pass < NCH; ++pass) {
        const int row = rs * NCH + pass;
#pragma unroll
        for (int j = 0; j < 4; ++j) xoff[pass][j] = swz<ES>(row + j, pch);
        doff[pass] = swz<ES>(row, pch);
    }
    // out-tile offsets of the rows this lane finalises (row = grp*LPC + q inside a sub-chunk)
    int yoff[TS / LPC];
#pragma unroll
    for (int grp = 0; grp < TS / LPC; ++grp) yoff[grp] = swz<ES>(grp * LPC + q, warp * CW + c);

    for (int i = 0; i < nchunks; ++i) {
        const int s = i % STAGES, ob = i & 1;
        if (!mbar_wait(bar_ready(s), (i / STAGES) & 1)) {
            if (lane == 0) atomicOr(&g_wait_status, kWaitFull);
            return;
        }
        const char *sx = stage_base + s * Cfg::STAGE_BYTES;
        const float *sBf = reinterpret_cast<const float *>(sx + OFF_BF);
        const float *sCf = reinterpret_cast<const float *>(sx + OFF_CF);
        char *so = out_base + ob * Cfg::OUT_BYTES;
        const int t_chunk0 = t_seg0 + i * TC;

#pragma unroll 1
        for (int sub = 0; sub < TC / TS; ++sub) {
            const int tl0 = sub * TS;  // chunk-local first step of this sub-chunk
            if (t_chunk0 + tl0 >= t_seg1) break;
            const char *sxs = sx + tl0 * 128;       // x tile rows of this sub-chunk (row 0 = 3 steps back)
            const char *sds = sxs + OFF_DT, *szs = sxs + OFF_Z;
            const bool tail = t_chunk0 + tl0 + TS > t_seg1;  // some rows lie past the end of the sequence
            // ------------------------------------------------------------ point-wise phase
#pragma unroll
            for (int pass = 0; pass < NCH; ++pass) {
                const int row = rs * NCH + pass;  // 0..TS-1
                float2 u;
                {
                    const float2 x0 = ld_pair<T>(sxs, xoff[pass][3]);
                    if (has_conv) {
                        float2 acc = cbias;
                        acc = fma2(cw[0], ld_pair<T>(sxs, xoff[pass][0]), acc);
                        acc = fma2(cw[1], ld_pair<T>(sxs, xoff[pass][1]), acc);
                        acc = fma2(cw[2], ld_pair<T>(sxs, xoff[pass][2]), acc);
                        acc = fma2(cw[3], x0, acc);
                        if constexpr (FAST) {
                            const float2 t = mul2(acc, splat2(-kLog2e));
                            const float2 den = add2(make_float2(ex2_approx(t.x), ex2_approx(t.y)), splat2(1.f));
                            u = mul2(acc, make_float2(rcp_approx(den.x), rcp_approx(den.y)));
                        } else {
                            u = make_float2(silu_acc(acc.x), silu_acc(acc.y));
                        }
                    } else {
                        u = x0;
                    }
                }
                const float2 v = add2(ld_pair<T>(sds, doff[pass]), dbias);
                float2 dtv;
                if (use_softplus) {
                    if constexpr (FAST) {
                        const float2 vl = mul2(v, splat2(kLog2e));
                        const float2 w = add2(make_float2(ex2_approx(vl.x), ex2_approx(vl.y)), splat2(1.f));
                        const float2 sp = mul2(make_float2(lg2_approx(w.x), lg2_approx(w.y)), splat2(kLn2));
                        dtv.x = v.x > 20.f ? v.x : sp.x;
                        dtv.y = v.y > 20.f ? v.y : sp.y;
                    } else {
                        dtv = make_float2(softplus_acc(v.x), softplus_acc(v.y));
                    }
                } else {
                    dtv = v;
                }
                float2 g = make_float2(1.f, 1.f);
                if (has_z) {
                    const float2 zz = ld_pair<T>(szs, doff[pass]);
                    if (p.z_gate) {
                        g = zz;
                    } else if constexpr (FAST) {
                        const float2 t = mul2(zz, splat2(-kLog2e));
                        const float2 den = add2(make_float2(ex2_approx(t.x), ex2_approx(t.y)), splat2(1.f));
                        g = mul2(zz, make_float2(rcp_approx(den.x), rcp_approx(den.y)));
                    } else {
                        g = make_float2(silu_acc(zz.x), silu_acc(zz.y));
                    }
                }
                float2 xin = mul2(dtv, u);
                const float2 sk = mul2(mul2(dskip, u), g);
                float2 r1;  // GEOM: exp(dt*A[d][0]);  general: dt itself
                if constexpr (GEOM) {
                    const float2 e = mul2(dtv, a0l2);
                    if constexpr (FAST) r1 = make_float2(ex2_approx(e.x), ex2_approx(e.y));
                    else r1 = make_float2(exp2f(e.x), exp2f(e.y));
                } else {
                    r1 = dtv;
                }
                if (tail && (t_chunk0 + tl0 + row) >= t_seg1) {  // steps past the end leave the state untouched
                    xin = make_float2(0.f, 0.f);
                    r1 = GEOM ? make_float2(1.f, 1.f) : make_float2(0.f, 0.f);
                }
                const int ri = row * CW + 2 * pj;  // records of the pair are adjacent: one 16-byte store each
                *reinterpret_cast<float4 *>(recGS + ri) = make_float4(g.x, sk.x, g.y, sk.y);
                if constexpr (POW4) {
                    const float2 r2 = mul2(r1, r1), r3 = mul2(r2, r1), r4 = mul2(r2, r2);
                    *reinterpret_cast<float4 *>(recRX + ri) = make_float4(r4.x, xin.x, r4.y, xin.y);
                    *reinterpret_cast<float2 *>(recP + 0 * Cfg::PLANE_FLOATS + ri) = r1;
                    *reinterpret_cast<float2 *>(recP + 1 * Cfg::PLANE_FLOATS + ri) = r2;
                    *reinterpret_cast<float2 *>(recP + 2 * Cfg::PLANE_FLOATS + ri) = r3;
                    *reinterpret_cast<float2 *>(recP + 3 * Cfg::PLANE_FLOATS + ri) = r4;
                } else {
                    *reinterpret_cast<float4 *>(recRX + ri) = make_float4(r1.x, xin.x, r1.y, xin.y);
                }
            }
            __syncwarp();
            if (sub == 0 && i >= 2) {
                // the out tile is about to be overwritten: its previous TMA store must have read it
                if (!mbar_wait(bar_out_empty(ob), ((i >> 1) - 1) & 1)) {
                    if (lane == 0) atomicOr(&g_wait_status, kWaitOutEmpty);
                    return;
                }
            }
            // ------------------------------------------------------------ recurrence phase
#pragma unroll
            for (int grp = 0; grp < TS / LPC; ++grp) {
                float part[LPC];
#pragma unroll
                for (int k = 0; k < LPC; ++k) {
                    const int row = grp * LPC + k;
                    const int ri = row * CW + c;
                    float2 a[S / 2];
                    const float2 rx = recRX[ri];
                    const float xin = rx.y;
                    if constexpr (GEOM && LPC == 4) {  // r^(q+1), r^(q+5), r^(q+9), r^(q+13)
                        const float base = recP[q * Cfg::PLANE_FLOATS + ri];
                        const float r8 = rx.x * rx.x;
                        a[0] = make_float2(base, base * rx.x);
                        a[1] = mul2(a[0], splat2(r8));
                    } else if constexpr (GEOM && LPC == 2) {  // r^(q+1+2j)
                        const float r2 = rx.x * rx.x;
                        const float r4 = r2 * r2;
                        const float r8 = r4 * r4;
                        const float base = q ? r2 : rx.x;
                        a[0] = make_float2(base, base * r2);
                        a[1] = mul2(a[0], splat2(r4));
                        a[2] = mul2(a[0], splat2(r8));
                        a[3] = mul2(a[1], splat2(r8));
                    } else if constexpr (GEOM) {  // LPC == 1: r^1 .. r^16
                        const float r2 = rx.x * rx.x;
                        a[0] = make_float2(rx.x, r2);
                        a[1] = mul2(a[0], splat2(r2));
                        const float r4 = a[1].y;
                        a[2] = mul2(a[0], splat2(r4));
                        a[3] = mul2(a[1], splat2(r4));
                        const float r8 = a[3].y;
#pragma unroll
                        for (int j = 0; j < 4; ++j) a[4 + j] = mul2(a[j], splat2(r8));
                    } else {
#pragma unroll
                        for (int j = 0; j < S / 2; ++j) {
                            if constexpr (FAST)
                                a[j] = make_float2(ex2_approx(rx.x * a2l[2 * j]), ex2_approx(rx.x * a2l[2 * j + 1]));
                            else
                                a[j] = make_float2(exp2f(rx.x * a2l[2 * j]), exp2f(rx.x * a2l[2 * j + 1]));
                        }
                    }
                    const float4 *Bq = reinterpret_cast<const float4 *>(sBf + (tl0 + row) * 16 + q * S);
                    const float4 *Cq = reinterpret_cast<const float4 *>(sCf + (tl0 + row) * 16 + q * S);
                    const float2 x2 = splat2(xin);
                    float2 yacc0 = make_float2(0.f, 0.f), yacc1 = make_float2(0.f, 0.f);  // two chains for ILP
#pragma unroll
                    for (int j4 = 0; j4 < S / 4; ++j4) {
                        const float4 bv = Bq[j4], cv = Cq[j4];
                        h[2 * j4] = fma2(a[2 * j4], h[2 * j4], mul2(x2, make_float2(bv.x, bv.y)));
                        h[2 * j4 + 1] = fma2(a[2 * j4 + 1], h[2 * j4 + 1], mul2(x2, make_float2(bv.z, bv.w)));
                        yacc0 = fma2(make_float2(cv.x, cv.y), h[2 * j4], yacc0);
                        yacc1 = fma2(make_float2(cv.z, cv.w), h[2 * j4 + 1], yacc1);
                    }
                    const float2 yacc = add2(yacc0, yacc1);
                    part[k] = yacc.x + yacc.y;
                }
                // combine the LPC partial sums of each channel so that lane q ends up with step q
                float ysum;
                if constexpr (LPC == 4) {
                    const bool hi = q & 2, lo = q & 1;
                    const float s0 = hi ? part[0] : part[2], s1 = hi ? part[1] : part[3];
                    float k0 = hi ? part[2] : part[0], k1 = hi ? part[3] : part[1];
                    k0 += __shfl_xor_sync(0xffffffffu, s0, 2);
                    k1 += __shfl_xor_sync(0xffffffffu, s1, 2);
                    const float sd = lo ? k0 : k1;
                    ysum = (lo ? k1 : k0) + __shfl_xor_sync(0xffffffffu, sd, 1);
                } else if constexpr (LPC == 2) {
                    const float sd = q ? part[0] : part[1];
                    ysum = (q ? part[1] : part[0]) + __shfl_xor_sync(0xffffffffu, sd, 1);
                } else {
                    ysum = part[0];
                }
                const int row = grp * LPC + q;
                const float2 gs = recGS[row * CW + c];
                const float yv = fmaf(ysum, gs.x, gs.y);
                st_f32(reinterpret_cast<T *>(so + tl0 * 128 + yoff[grp]), yv);
            }
            __syncwarp();
        }
        // hand the stage back and publish the out tile
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(bar_empty(s));
            mbar_arrive(bar_out_full(ob));
        }
    }

    // final state: to h_last (last segment) or to the carry buffer (split sequence)
    const bool last_seg = seg == p.n_segments - 1;
    if (last_seg && p.h_last && dch < p.D) {
        float *dst = p.h_last + ((int64_t)b * p.D + dch) * 16;
#pragma unroll
        for (int j = 0; j < S / 2; ++j) {
            dst[q + LPC * (2 * j)] = h[j].x;
            dst[q + LPC * (2 * j + 1)] = h[j].y;
        }
    }
    if (!last_seg) {
        if (dch < p.D) {
            float *dst = p.carry + (((int64_t)seg * p.B + b) * p.D + dch) * 16;
#pragma unroll
            for (int j = 0; j < S / 2; ++j) {
                dst[q + LPC * (2 * j)] = h[j].x;
                dst[q + LPC * (2 * j + 1)] = h[j].y;
            }
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) {
            const int fidx = ((seg * p.B + b) * gridDim.x + tile) * 8 + warp;
            asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.flags + fidx), "r"(p.epoch) : "memory");
        }
    }
}

}  // namespace scan
}  // namespace hx

#include "scan_direct.cuh"

namespace hx {
namespace scan {

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
static hx_status validate_dims(const hx_scan_args *a) {
    HX_REQUIRE(a != nullptr, HX_ERR_INVALID_INPUT, "hx_selective_scan_fwd: args is NULL");
    HX_REQUIRE(a->batch >= 0 && a->seq_len >= 0 && a->d_inner >= 0, HX_ERR_INVALID_DIMENSION,
               "negative dimension (batch %d, seq_len %d, d_inner %d)", a->batch, a->seq_len, a->d_inner);
    HX_REQUIRE(a->d_state >= 1 && a->d_state <= 256, HX_ERR_INVALID_DIMENSION, "d_state %d outside [1, 256]",
               a->d_state);
    HX_REQUIRE(a->io_dtype == HX_F32 || a->io_dtype == HX_BF16, HX_ERR_DTYPE_MISMATCH,
               "io_dtype %d is neither HX_F32 nor HX_BF16", a->io_dtype);
    return HX_OK;
}

static hx_status validate(const hx_scan_args *a) {
    hx_status s = validate_dims(a);
    if (s != HX_OK) return s;
    if (a->batch == 0 || a->seq_len == 0 || a->d_inner == 0) return HX_OK;
    HX_REQUIRE(a->x && (a->dt || a->W_dt) && a->Bm && a->Cm && a->y && a->A, HX_ERR_INVALID_INPUT,
               "x, dt (or W_dt), Bm, Cm, y and A must not be NULL");
    if (a->W_dt) {
        HX_REQUIRE(a->dt_low != nullptr, HX_ERR_INVALID_INPUT, "W_dt given without dt_low");
        HX_REQUIRE(a->dt_rank >= 8 && a->dt_rank <= 64 && a->dt_rank % 8 == 0, HX_ERR_INVALID_DIMENSION,
                   "fused dt projection needs dt_rank in [8, 64] and a multiple of 8 (got %d)", a->dt_rank);
        HX_REQUIRE(a->io_dtype == HX_BF16, HX_ERR_UNSUPPORTED_OPERATION, "the fused dt projection takes bf16 operands");
        HX_REQUIRE(a->dt_low_row_stride >= a->dt_rank, HX_ERR_SHAPE_MISMATCH, "dt_low row stride smaller than dt_rank");
    }
    if (a->conv_w)
        HX_REQUIRE(a->d_conv >= 1 && a->d_conv <= 4, HX_ERR_INVALID_DIMENSION, "d_conv %d outside [1, 4]", a->d_conv);
    HX_REQUIRE(a->conv_w || !a->conv_b, HX_ERR_INVALID_INPUT, "conv_b given without conv_w");
    const int64_t D = a->d_inner, N = a->d_state;
    HX_REQUIRE(a->x_row_stride >= D && (a->W_dt || a->dt_row_stride >= D) && a->y_row_stride >= D && (!a->z || a->z_row_stride >= D),
               HX_ERR_SHAPE_MISMATCH, "a row stride is smaller than d_inner %d", a->d_inner);
    HX_REQUIRE(a->B_row_stride >= N && a->C_row_stride >= N, HX_ERR_SHAPE_MISMATCH,
               "B/C row stride is smaller than d_state %d", a->d_state);
    return HX_OK;
}

static hx_status launch_simple(const hx_scan_args *a, cudaStream_t st) {
    HX_REQUIRE(a->W_dt == nullptr, HX_ERR_UNSUPPORTED_OPERATION, "the simple scan kernel has no fused dt projection");
    SimpleParams p;
    p.B = a->batch; p.L = a->seq_len; p.D = a->d_inner; p.N = a->d_state; p.K = a->conv_w ? a->d_conv : 0;
    p.dt_softplus = a->dt_softplus;
    p.z_gate = a->z_is_gate != 0;
    p.x = a->x; p.dt = a->dt; p.z = a->z; p.Bm = a->Bm; p.Cm = a->Cm; p.y = a->y;
    p.xb = a->x_batch_stride; p.xr = a->x_row_stride; p.dtb = a->dt_batch_stride; p.dtr = a->dt_row_stride;
    p.zb = a->z_batch_stride; p.zr = a->z_row_stride; p.Bb = a->B_batch_stride; p.Br = a->B_row_stride;
    p.Cb = a->C_batch_stride; p.Cr = a->C_row_stride; p.yb = a->y_batch_stride; p.yr = a->y_row_stride;
    p.A = a->A; p.Dskip = a->Dskip; p.conv_w = a->conv_w; p.conv_b = a->conv_b; p.dt_bias = a->dt_bias;
    p.h_last = a->h_last;
    dim3 grid((a->d_inner + 127) / 128, a->batch), block(128);
    const bool bf = a->io_dtype == HX_BF16;
    if (a->d_state <= 16) {
        if (bf) scan_simple_kernel<__nv_bfloat16, 16><<<grid, block, 0, st>>>(p);
        else scan_simple_kernel<float, 16><<<grid, block, 0, st>>>(p);
    } else if (a->d_state <= 64) {
        if (bf) scan_simple_kernel<__nv_bfloat16, 64><<<grid, block, 0, st>>>(p);
        else scan_simple_kernel<float, 64><<<grid, block, 0, st>>>(p);
    } else {
        if (bf) scan_simple_kernel<__nv_bfloat16, 256><<<grid, block, 0, st>>>(p);
        else scan_simple_kernel<float, 256><<<grid, block, 0, st>>>(p);
    }
    return check_launch("scan_simple_kernel");
}

// Number of sequence segments and their length for the split variant.
static void seg_plan(const hx_scan_args *a, int chunk, int *n_seg, int *seg_len) {
    int want = a->seq_splits > 0 ? a->seq_splits : 4;
    int len = (a->seq_len + want - 1) / want;
    len = (len + chunk - 1) / chunk * chunk;
    if (len < chunk) len = chunk;
    *seg_len = len;
    *n_seg = (a->seq_len + len - 1) / len;
}

constexpr int kChunkBf16 = 32, kChunkF32 = 32;
constexpr int kPlanChunk = 32;  // segment lengths are multiples of this

static int tiles_of(const hx_scan_args *a) {
    const int DT = a->io_dtype == HX_BF16 ? 64 : 32;
    return (a->d_inner + DT - 1) / DT;
}

// Workspace of a split scan, one layout for every form: the per-segment states (chained form: the carries;
// look-back form: the aggregates), the chained form's flags, the look-back form's sums of dt.
struct WsLayout {
    size_t carry, flags, sdt, total;  // byte offsets from the 256-aligned base; total includes the alignment slack
    size_t flag_bytes;
};
static WsLayout ws_layout(const hx_scan_args *a, int n_seg) {
    WsLayout l{0, 0, 0, 0, 0};
    if (n_seg <= 1) return l;
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    const size_t chains = (size_t)(n_seg - 1) * a->batch * a->d_inner;
    l.flag_bytes = (size_t)(n_seg - 1) * a->batch * tiles_of(a) * 8 * sizeof(int);
    l.carry = 0;
    l.flags = up(chains * 16 * sizeof(float));
    l.sdt = l.flags + up(l.flag_bytes);
    l.total = l.sdt + up(chains * sizeof(float)) + 256;
    return l;
}
static size_t workspace_bytes(const hx_scan_args *a, int n_seg) { return ws_layout(a, n_seg).total; }

template <typename T, int LPC, bool GEOM, int TC, int STAGES, bool STD>
static hx_status launch_tiled_inst(const hx_scan_args *a, const TiledParams &p, const CUtensorMap *maps, dim3 grid,
                                   cudaStream_t st) {
    using Cfg = TiledCfg<T, LPC, GEOM, TC, STAGES, STD>;
    auto kern = scan_tiled_kernel<T, Cfg>;
    static std::atomic<bool> attr_set[64];  // zero-initialised; setting the attribute twice is harmless
    int dev = 0;
    HX_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
        HX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_set[dev].store(true, std::memory_order_release);
    }
    kern<<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], p);
    return check_launch("scan_tiled_kernel");
}

static int choose_lpc(const hx_scan_args *a) {
    if (a->lanes_per_channel == 1 || a->lanes_per_channel == 2 || a->lanes_per_channel == 4)
        return a->lanes_per_channel;
    // One lane per channel needs ~4 consumer warps per warp scheduler (4 schedulers per SM) to keep the pipes
    // busy.  Below that, two lanes per channel double the warps at a small cost per point (measured at
    // 24 576 chains: 0.68 ms with 2 lanes, 0.87 ms with 1 or 4); four lanes pay twice the exchange cost and only
    // win when even two lanes leave most schedulers without a warp.
    const double chains = (double)a->batch * a->d_inner;
    if (chains / 32.0 >= 16.0 * sm_count()) return 1;
    if (chains / 16.0 >= 4.0 * sm_count()) return 2;
    return 4;
}

static hx_status launch_tiled(const hx_scan_args *a, bool split, cudaStream_t st) {
    HX_REQUIRE(a->W_dt == nullptr, HX_ERR_UNSUPPORTED_OPERATION, "the lane-split scan kernel has no fused dt projection");
    HX_REQUIRE(a->d_state == 16, HX_ERR_UNSUPPORTED_OPERATION, "the tiled scan needs d_state == 16 (got %d)", a->d_state);
    const bool bf = a->io_dtype == HX_BF16;
    // `reserved` picks another (chunk, stages) pair for the bf16 / geometric / standard path (tuning knob)
    const bool stdp0 = a->conv_w != nullptr && a->z != nullptr && a->dt_softplus != 0;
    // only 1 and 2 name a tuning variant; anything else (the direct kernel's selector among them) is the default
    const int tune = (bf && a->a_geometric && stdp0 && (a->reserved == 1 || a->reserved == 2)) ? a->reserved : 0;
    const int ES = bf ? 2 : 4, DT = 128 / ES, TC = tune >= 1 ? 16 : (bf ? kChunkBf16 : kChunkF32);
    const int tiles = (a->d_inner + DT - 1) / DT;
    int n_seg = 1, seg_len = (a->seq_len + TC - 1) / TC * TC;
    // segments are planned on 32-step chunks whatever the kernel's own chunk (16 or 32), so that the size query
    // and every launcher agree on the plan
    if (split) seg_plan(a, kPlanChunk, &n_seg, &seg_len);

    TiledParams p;
    p.B = a->batch; p.L = a->seq_len; p.D = a->d_inner;
    p.K = a->conv_w ? a->d_conv : 0;
    p.has_z = a->z != nullptr;
    p.z_gate = a->z_is_gate != 0;
    p.dt_softplus = a->dt_softplus;
    p.n_segments = n_seg; p.seg_len = seg_len;
    p.A = a->A; p.Dskip = a->Dskip; p.conv_w = a->conv_w; p.conv_b = a->conv_b; p.dt_bias = a->dt_bias;
    p.h_last = a->h_last;
    p.carry = nullptr; p.flags = nullptr; p.epoch = 1; p.dt_rank = 0; p.sdt = nullptr; p.seg_base = 0;
    if (n_seg > 1) {
        const WsLayout wl = ws_layout(a, n_seg);
        HX_REQUIRE(a->workspace && a->workspace_bytes >= wl.total, HX_ERR_INVALID_INPUT,
                   "the sequence-split scan needs a workspace of %zu bytes (got %zu)", wl.total, a->workspace_bytes);
        char *ws = reinterpret_cast<char *>((reinterpret_cast<uintptr_t>(a->workspace) + 255) & ~uintptr_t(255));
        p.carry = reinterpret_cast<float *>(ws + wl.carry);
        p.flags = reinterpret_cast<int *>(ws + wl.flags);
        // flags are compared against a per-launch epoch, so they are cleared on every call
        HX_CUDA(cudaMemsetAsync(p.flags, 0, wl.flag_bytes, st));
    }

    // tensor maps: x/dt/z/y are [B, L, D] with D innermost; B/C are [B, L, 16]
    CUtensorMap maps[6];
    const uint64_t dims_d[3] = {(uint64_t)a->d_inner, (uint64_t)a->seq_len, (uint64_t)a->batch};
    const uint64_t dims_n[3] = {16, (uint64_t)a->seq_len, (uint64_t)a->batch};
    auto strides = [&](int64_t row, int64_t batch, uint64_t *out) {
        out[0] = (uint64_t)row * ES;
        out[1] = (uint64_t)batch * ES;
    };
    uint64_t sb[2];
    const uint32_t box_x[3] = {(uint32_t)DT, (uint32_t)TC + 3, 1}, box_r[3] = {(uint32_t)DT, (uint32_t)TC, 1},
                   box_n[3] = {16, (uint32_t)TC, 1};
    hx_status s;
    strides(a->x_row_stride, a->x_batch_stride, sb);
    if ((s = encode_tensor_map(&maps[0], a->io_dtype, 3, a->x, dims_d, sb, box_x, true)) != HX_OK) return s;
    strides(a->dt_row_stride, a->dt_batch_stride, sb);
    if ((s = encode_tensor_map(&maps[1], a->io_dtype, 3, a->dt, dims_d, sb, box_r, true)) != HX_OK) return s;
    if (a->z) {
        strides(a->z_row_stride, a->z_batch_stride, sb);
        if ((s = encode_tensor_map(&maps[2], a->io_dtype, 3, a->z, dims_d, sb, box_r, true)) != HX_OK) return s;
    } else {
        maps[2] = maps[1];
    }
    strides(a->B_row_stride, a->B_batch_stride, sb);
    if ((s = encode_tensor_map(&maps[3], a->io_dtype, 3, a->Bm, dims_n, sb, box_n, false)) != HX_OK) return s;
    strides(a->C_row_stride, a->C_batch_stride, sb);
    if ((s = encode_tensor_map(&maps[4], a->io_dtype, 3, a->Cm, dims_n, sb, box_n, false)) != HX_OK) return s;
    strides(a->y_row_stride, a->y_batch_stride, sb);
    if ((s = encode_tensor_map(&maps[5], a->io_dtype, 3, a->y, dims_d, sb, box_r, true)) != HX_OK) return s;

    HX_REQUIRE(a->batch <= 65535 && n_seg <= 65535, HX_ERR_INVALID_DIMENSION, "batch %d or segments %d exceed the grid limit",
               a->batch, n_seg);
    dim3 grid(tiles, a->batch, n_seg);
    const int lpc = choose_lpc(a);
    const bool geom = a->a_geometric != 0;
    // the standard path (4-tap conv, softplus, gate) has its flags fixed at compile time
    const bool stdp = a->conv_w != nullptr && a->z != nullptr && a->dt_softplus != 0;
#define HX_TILED_CASE(T, LPC, GEOM, TCv, ST)                                                    \
    do {                                                                                        \
        if (stdp) return launch_tiled_inst<T, LPC, GEOM, TCv, ST, true>(a, p, maps, grid, st);  \
        return launch_tiled_inst<T, LPC, GEOM, TCv, ST, false>(a, p, maps, grid, st);           \
    } while (0)
    if (tune == 1) {
        if (lpc == 1) return launch_tiled_inst<__nv_bfloat16, 1, true, 16, 3, true>(a, p, maps, grid, st);
        if (lpc == 2) return launch_tiled_inst<__nv_bfloat16, 2, true, 16, 3, true>(a, p, maps, grid, st);
        return launch_tiled_inst<__nv_bfloat16, 4, true, 16, 3, true>(a, p, maps, grid, st);
    }
    if (tune == 2) {
        if (lpc == 1) return launch_tiled_inst<__nv_bfloat16, 1, true, 16, 4, true>(a, p, maps, grid, st);
        if (lpc == 2) return launch_tiled_inst<__nv_bfloat16, 2, true, 16, 4, true>(a, p, maps, grid, st);
        return launch_tiled_inst<__nv_bfloat16, 4, true, 16, 4, true>(a, p, maps, grid, st);
    }
    if (bf) {
        if (geom) {
            if (lpc == 1) HX_TILED_CASE(__nv_bfloat16, 1, true, kChunkBf16, 2);
            if (lpc == 2) HX_TILED_CASE(__nv_bfloat16, 2, true, kChunkBf16, 2);
            HX_TILED_CASE(__nv_bfloat16, 4, true, kChunkBf16, 2);
        } else {
            if (lpc == 1) HX_TILED_CASE(__nv_bfloat16, 1, false, kChunkBf16, 2);
            if (lpc == 2) HX_TILED_CASE(__nv_bfloat16, 2, false, kChunkBf16, 2);
            HX_TILED_CASE(__nv_bfloat16, 4, false, kChunkBf16, 2);
        }
    } else {
        if (geom) {
            if (lpc == 1) HX_TILED_CASE(float, 1, true, kChunkF32, 2);
            if (lpc == 2) HX_TILED_CASE(float, 2, true, kChunkF32, 2);
            HX_TILED_CASE(float, 4, true, kChunkF32, 2);
        } else {
            if (lpc == 1) HX_TILED_CASE(float, 1, false, kChunkF32, 2);
            if (lpc == 2) HX_TILED_CASE(float, 2, false, kChunkF32, 2);
            HX_TILED_CASE(float, 4, false, kChunkF32, 2);
        }
    }
#undef HX_TILED_CASE
    return HX_OK;
}


template <typename T, int CPL, bool GEOM, bool STD, int STAGES = 2, int FUSEDT = 0, bool ZGATE = false, bool BLOCK = false,
          int MODE = 0>
static hx_status launch_direct_inst(const TiledParams &p, const CUtensorMap *maps, dim3 grid, cudaStream_t st, void *y,
                                    int64_t y_bs, int64_t y_rs) {
    using Cfg = DirectCfg<T, CPL, GEOM, STD, STAGES, FUSEDT, ZGATE, BLOCK, MODE>;
    auto kern = scan_direct_kernel<T, Cfg>;
    static std::atomic<bool> attr_set[64];  // zero-initialised; setting the attribute twice is harmless
    int dev = 0;
    HX_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
        HX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_set[dev].store(true, std::memory_order_release);
    }
    kern<<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[6], maps[7], p,
                                                      static_cast<T *>(y), y_bs, y_rs);
    return check_launch("scan_direct_kernel");
}

// The two launches of the look-back form: the aggregate pass over segments 0 .. S-2, then the output pass over
// all S segments (stream order is the only dependency between them).
template <typename T, bool STD, int FUSEDT, bool BLOCK>
static hx_status launch_lookback_pair(const TiledParams &p, const CUtensorMap *maps, dim3 grid, cudaStream_t st, void *y,
                                      int64_t y_bs, int64_t y_rs) {
    dim3 g1(grid.x, grid.y, grid.z - 1);
    hx_status s = launch_direct_inst<T, 1, true, STD, 2, FUSEDT, false, BLOCK, 1>(p, maps, g1, st, y, y_bs, y_rs);
    if (s != HX_OK) return s;
    return launch_direct_inst<T, 1, true, STD, 2, FUSEDT, false, BLOCK, 2>(p, maps, grid, st, y, y_bs, y_rs);
}

// 1: the fused dt projection of the block's one-lane-per-channel scan runs as tcgen05.mma into tensor memory; 0: as
// mma.sync in the producer warp, through a shared-memory tile.
#ifndef HX_SCAN_FUSEDT_TC
#define HX_SCAN_FUSEDT_TC 1
#endif
// ring stages of that form: with two, the chain load -> MMA -> commit of the next chunk does not always fit under the
// 16 steps of the current one (10.90 against 10.74 ms over the 24 blocks of the byte LM)
// chained segments: split until the grid is about this many waves of CTA slots (measured at 49 152 chains with the
// dt projection inside, per 24 blocks: 3 waves = 4 segments 10.98 ms, 6 = 8 segments 10.7-10.8, 12 = 16 segments 11.08)
#ifndef HX_SCAN_CHAIN_WAVES
#define HX_SCAN_CHAIN_WAVES 6.0
#endif
#ifndef HX_SCAN_FUSEDT_STAGES
#define HX_SCAN_FUSEDT_STAGES 3
#endif
#ifndef HX_SCAN_CPL2_MIN_WARPS
#define HX_SCAN_CPL2_MIN_WARPS 8.0
#endif
// channels per lane for the direct kernel: 2 when that still leaves about two warps per scheduler
static int choose_cpl(const hx_scan_args *a) {
    if (a->io_dtype != HX_BF16) return 1;
    if (a->reserved % 10 == 1 || a->reserved % 10 == 2) return a->reserved % 10;
    const double chains = (double)a->batch * a->d_inner;
    return chains / 64.0 >= HX_SCAN_CPL2_MIN_WARPS * sm_count() ? 2 : 1;
}

// What the look-back form supports: geometric A, and where the dt projection is fused the block's configuration.
static bool lookback_ok(const hx_scan_args *a) {
    if (a->d_state != 16 || !a->a_geometric || a->z_is_gate) return false;
    if (a->W_dt) return a->conv_w == nullptr && a->z != nullptr && a->dt_softplus != 0;
    return true;
}

// hx_debug_scan_orphan_segment: first segment the calling thread's next chained launch starts (0 = all of them)
static thread_local int t_orphan_from = 0;

// form: 0 = one pass (segments, if any, chained through carries), 1 = look-back (aggregate pass + output pass)
static hx_status launch_direct(const hx_scan_args *a, bool split, cudaStream_t st, int form = 0) {
    HX_REQUIRE(a->d_state == 16, HX_ERR_UNSUPPORTED_OPERATION, "the direct scan needs d_state == 16 (got %d)", a->d_state);
    const bool bf = a->io_dtype == HX_BF16;
    const int ES = bf ? 2 : 4, BOXC = 128 / ES, TC = 16;
    if (form == 1)
        HX_REQUIRE(lookback_ok(a), HX_ERR_UNSUPPORTED_OPERATION,
                   "the look-back scan needs a_geometric = 1 (and, with a fused dt projection, the block's configuration)");
    const int cpl = form == 1 ? 1 : choose_cpl(a);
    const int DT = bf ? (cpl == 2 ? 256 : 128) : 128;  // channels per CTA (4 consumer warps)
    const int tiles = (a->d_inner + DT - 1) / DT;
    int n_seg = 1, seg_len = (a->seq_len + TC - 1) / TC * TC;
    if (split) seg_plan(a, kPlanChunk, &n_seg, &seg_len);
    if (n_seg <= 1) form = 0;

    TiledParams p;
    p.B = a->batch; p.L = a->seq_len; p.D = a->d_inner;
    p.K = a->conv_w ? a->d_conv : 0;
    p.has_z = a->z != nullptr;
    p.z_gate = a->z_is_gate != 0;
    p.dt_softplus = a->dt_softplus;
    p.n_segments = n_seg; p.seg_len = seg_len;
    p.A = a->A; p.Dskip = a->Dskip; p.conv_w = a->conv_w; p.conv_b = a->conv_b; p.dt_bias = a->dt_bias;
    p.h_last = a->h_last;
    p.carry = nullptr; p.flags = nullptr; p.epoch = 1; p.sdt = nullptr;
    p.dt_rank = a->W_dt ? a->dt_rank : 0;
    p.seg_base = t_orphan_from;
    if (n_seg > 1) {
        const WsLayout wl = ws_layout(a, n_seg);
        HX_REQUIRE(a->workspace && a->workspace_bytes >= wl.total, HX_ERR_INVALID_INPUT,
                   "the sequence-split scan needs a workspace of %zu bytes (got %zu)", wl.total, a->workspace_bytes);
        char *ws = reinterpret_cast<char *>((reinterpret_cast<uintptr_t>(a->workspace) + 255) & ~uintptr_t(255));
        p.carry = reinterpret_cast<float *>(ws + wl.carry);
        p.flags = reinterpret_cast<int *>(ws + wl.flags);
        p.sdt = reinterpret_cast<float *>(ws + wl.sdt);
        // chained form: the flags are compared against a per-launch epoch, so they are cleared on every call.
        // The look-back form has no flags: every aggregate is written by the first launch before the second reads it.
        if (form == 0) HX_CUDA(cudaMemsetAsync(p.flags, 0, wl.flag_bytes, st));
    }

    CUtensorMap maps[8];
    const uint64_t dims_d[3] = {(uint64_t)a->d_inner, (uint64_t)a->seq_len, (uint64_t)a->batch};
    const uint64_t dims_n[3] = {16, (uint64_t)a->seq_len, (uint64_t)a->batch};
    auto strides = [&](int64_t row, int64_t batch, uint64_t *out) {
        out[0] = (uint64_t)row * ES;
        out[1] = (uint64_t)batch * ES;
    };
    uint64_t sb[2];
    const uint32_t box_x[3] = {(uint32_t)BOXC, (uint32_t)TC + 3, 1}, box_r[3] = {(uint32_t)BOXC, (uint32_t)TC, 1},
                   box_n[3] = {16, (uint32_t)TC, 1};
    hx_status s;
    strides(a->x_row_stride, a->x_batch_stride, sb);
    if ((s = encode_tensor_map(&maps[0], a->io_dtype, 3, a->x, dims_d, sb, box_x, false)) != HX_OK) return s;
    const bool fused_dt = a->W_dt != nullptr;
    if (fused_dt) {
        // dt_low [B, L, R] -> boxes of [16 steps x 64 columns] (columns past R are zero-filled);
        // W_dt [D, R] -> one [DT channels x 64] tile per CTA
        const uint64_t dims_l[3] = {(uint64_t)a->dt_rank, (uint64_t)a->seq_len, (uint64_t)a->batch};
        const uint32_t box_l[3] = {64, (uint32_t)TC, 1};
        strides(a->dt_low_row_stride, a->dt_low_batch_stride, sb);
        if ((s = encode_tensor_map(&maps[6], HX_BF16, 3, a->dt_low, dims_l, sb, box_l, true)) != HX_OK) return s;
        const uint64_t dims_w[2] = {(uint64_t)a->dt_rank, (uint64_t)a->d_inner};
        const uint64_t str_w[1] = {(uint64_t)a->dt_rank * 2};
        const uint32_t box_w[2] = {64, (uint32_t)DT};
        if ((s = encode_tensor_map(&maps[7], HX_BF16, 2, a->W_dt, dims_w, str_w, box_w, true)) != HX_OK) return s;
        maps[1] = maps[0];
    } else {
        strides(a->dt_row_stride, a->dt_batch_stride, sb);
        if ((s = encode_tensor_map(&maps[1], a->io_dtype, 3, a->dt, dims_d, sb, box_r, false)) != HX_OK) return s;
        maps[6] = maps[0];
        maps[7] = maps[0];
    }
    if (a->z) {
        strides(a->z_row_stride, a->z_batch_stride, sb);
        if ((s = encode_tensor_map(&maps[2], a->io_dtype, 3, a->z, dims_d, sb, box_r, false)) != HX_OK) return s;
    } else {
        maps[2] = maps[1];
    }
    strides(a->B_row_stride, a->B_batch_stride, sb);
    if ((s = encode_tensor_map(&maps[3], a->io_dtype, 3, a->Bm, dims_n, sb, box_n, false)) != HX_OK) return s;
    strides(a->C_row_stride, a->C_batch_stride, sb);
    if ((s = encode_tensor_map(&maps[4], a->io_dtype, 3, a->Cm, dims_n, sb, box_n, false)) != HX_OK) return s;
    maps[5] = maps[0];  // y is stored straight from registers: no tensor map, no TMA alignment rule for it

    HX_REQUIRE(a->batch <= 65535 && n_seg <= 65535, HX_ERR_INVALID_DIMENSION, "batch %d or segments %d exceed the grid limit",
               a->batch, n_seg);
    dim3 grid(tiles, a->batch, n_seg - p.seg_base);
    const bool geom = a->a_geometric != 0;
    const bool stdp = a->conv_w != nullptr && a->z != nullptr && a->dt_softplus != 0;
    // the block's own call: u already convolved, gate and softplus present, geometric A
    const bool blockp = bf && geom && !p.z_gate && a->conv_w == nullptr && a->z != nullptr && a->dt_softplus != 0;
    void *yv = a->y;
    const int64_t ybs = a->y_batch_stride, yrs = a->y_row_stride;
    if (form == 1) {
        if (fused_dt) {
            if (HX_SCAN_FUSEDT_TC) return launch_lookback_pair<__nv_bfloat16, false, 2, true>(p, maps, grid, st, yv, ybs, yrs);
            return launch_lookback_pair<__nv_bfloat16, false, 1, true>(p, maps, grid, st, yv, ybs, yrs);
        }
        if (blockp) return launch_lookback_pair<__nv_bfloat16, false, 0, true>(p, maps, grid, st, yv, ybs, yrs);
        if (bf && stdp) return launch_lookback_pair<__nv_bfloat16, true, 0, false>(p, maps, grid, st, yv, ybs, yrs);
        if (bf) return launch_lookback_pair<__nv_bfloat16, false, 0, false>(p, maps, grid, st, yv, ybs, yrs);
        return launch_lookback_pair<float, false, 0, false>(p, maps, grid, st, yv, ybs, yrs);
    }
#define HX_DIRECT_CASE(T, CPL)                                                                                         \
    do {                                                                                                               \
        if (geom && stdp) return launch_direct_inst<T, CPL, true, true>(p, maps, grid, st, yv, ybs, yrs);              \
        if (geom) return launch_direct_inst<T, CPL, true, false>(p, maps, grid, st, yv, ybs, yrs);                     \
        if (stdp) return launch_direct_inst<T, CPL, false, true>(p, maps, grid, st, yv, ybs, yrs);                     \
        return launch_direct_inst<T, CPL, false, false>(p, maps, grid, st, yv, ybs, yrs);                              \
    } while (0)
    if (fused_dt) {
        HX_REQUIRE(stdp || (a->z != nullptr && a->dt_softplus != 0), HX_ERR_UNSUPPORTED_OPERATION,
                   "the fused dt projection is built for the block's configuration (gate and softplus present)");
        // the block hands u (already convolved): conv flags are read at run time, so STD is false here
        // the gate flag is a compile-time constant on this path (the block's), so the activation code is gone when
        // in_proj has already applied it
        if (p.z_gate) {
            if (cpl == 2) {
                if (geom) return launch_direct_inst<__nv_bfloat16, 2, true, false, 2, 1, true>(p, maps, grid, st, yv, ybs, yrs);
                return launch_direct_inst<__nv_bfloat16, 2, false, false, 2, 1, true>(p, maps, grid, st, yv, ybs, yrs);
            }
            if (geom) return launch_direct_inst<__nv_bfloat16, 1, true, false, 2, 1, true>(p, maps, grid, st, yv, ybs, yrs);
            return launch_direct_inst<__nv_bfloat16, 1, false, false, 2, 1, true>(p, maps, grid, st, yv, ybs, yrs);
        }
        // the block's own call: every flag is a compile-time constant, which saves the per-point flag tests and the
        // registers of the unused conv window
        if (blockp) {
            if (cpl == 2) return launch_direct_inst<__nv_bfloat16, 2, true, false, 2, 1, false, true>(p, maps, grid, st, yv, ybs, yrs);
            // one lane per channel: the projection runs as tcgen05.mma into tensor memory, lane = channel
            if (HX_SCAN_FUSEDT_TC)
                return launch_direct_inst<__nv_bfloat16, 1, true, false, HX_SCAN_FUSEDT_STAGES, 2, false, true>(p, maps, grid, st, yv, ybs, yrs);
            return launch_direct_inst<__nv_bfloat16, 1, true, false, 2, 1, false, true>(p, maps, grid, st, yv, ybs, yrs);
        }
        if (cpl == 2) {
            if (geom) return launch_direct_inst<__nv_bfloat16, 2, true, false, 2, 1>(p, maps, grid, st, yv, ybs, yrs);
            return launch_direct_inst<__nv_bfloat16, 2, false, false, 2, 1>(p, maps, grid, st, yv, ybs, yrs);
        }
        if (geom) return launch_direct_inst<__nv_bfloat16, 1, true, false, 2, 1>(p, maps, grid, st, yv, ybs, yrs);
        return launch_direct_inst<__nv_bfloat16, 1, false, false, 2, 1>(p, maps, grid, st, yv, ybs, yrs);
    }
    if (bf && geom && stdp && a->reserved / 10 == 1) {  // tuning: three stages instead of two
        if (cpl == 2) return launch_direct_inst<__nv_bfloat16, 2, true, true, 3>(p, maps, grid, st, yv, ybs, yrs);
        return launch_direct_inst<__nv_bfloat16, 1, true, true, 3>(p, maps, grid, st, yv, ybs, yrs);
    }
    if (blockp) {
        // the block's configuration with dt read from memory: compile-time flags as in the fused form
        if (cpl == 2) return launch_direct_inst<__nv_bfloat16, 2, true, false, 2, 0, false, true>(p, maps, grid, st, yv, ybs, yrs);
        return launch_direct_inst<__nv_bfloat16, 1, true, false, 2, 0, false, true>(p, maps, grid, st, yv, ybs, yrs);
    }
    if (bf) {
        if (cpl == 2) HX_DIRECT_CASE(__nv_bfloat16, 2);
        HX_DIRECT_CASE(__nv_bfloat16, 1);
    }
    HX_DIRECT_CASE(float, 1);
#undef HX_DIRECT_CASE
    return HX_OK;
}

// ---- kernel choice of HX_SCAN_AUTO (d_state == 16), shared with the Mamba block's planning
// Chains are (batch, channel) pairs; a one-lane-per-channel warp holds 32 of them.  With at least 8 such warps per
// SM the direct kernel runs them one pass, chained segments evening out the load.  Below that the machine is short
// of independent work: with geometric A and a split the look-back form runs the segments of a chain at the same
// time; otherwise the lane-split kernel spreads a chain's states over 2 or 4 lanes.
int auto_channels_per_lane(const hx_scan_args *a) { return choose_cpl(a); }

ScanKind auto_kind(const hx_scan_args *a) {
    const double warps_per_sm = (double)a->batch * a->d_inner / 32.0 / sm_count();
    if (warps_per_sm >= 8.0) return ScanKind::Direct;
    if (a->seq_splits > 1 && lookback_ok(a)) return ScanKind::LookBack;
    if (a->W_dt != nullptr) return ScanKind::Direct;  // the fused dt projection exists only there
    return ScanKind::Tiled;
}

}  // namespace scan

hx_status read_status_scan(int *v, bool clear) {
    HX_CUDA(cudaMemcpyFromSymbol(v, scan::g_wait_status, sizeof(int)));
    if (clear && *v != 0) {
        const int zero = 0;
        HX_CUDA(cudaMemcpyToSymbol(scan::g_wait_status, &zero, sizeof(int)));
    }
    return HX_OK;
}

}  // namespace hx

extern "C" {

hx_status hx_selective_scan_fwd(const hx_scan_args *a, void *stream) {
    hx_status s = hx::scan::validate(a);
    if (s != HX_OK) return s;
    if (a->batch == 0 || a->seq_len == 0 || a->d_inner == 0) return HX_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const bool split = a->seq_splits > 1;  // the tiled and direct kernels can both hand carries between segments
    switch (a->variant) {
        case HX_SCAN_SIMPLE: return hx::scan::launch_simple(a, st);
        case HX_SCAN_TILED: return hx::scan::launch_tiled(a, split, st);
        case HX_SCAN_SEQSPLIT: return hx::scan::launch_tiled(a, true, st);
        case HX_SCAN_DIRECT: return hx::scan::launch_direct(a, split, st);
        case HX_SCAN_LOOKBACK: return hx::scan::launch_direct(a, true, st, 1);
        case HX_SCAN_AUTO: {
            if (a->d_state == 16) {
                switch (hx::scan::auto_kind(a)) {
                    case hx::scan::ScanKind::Direct: s = hx::scan::launch_direct(a, split, st); break;
                    case hx::scan::ScanKind::LookBack: s = hx::scan::launch_direct(a, true, st, 1); break;
                    default: s = hx::scan::launch_tiled(a, split, st); break;
                }
                // an operand that does not meet the TMA alignment rules goes to the simple kernel
                if (s != HX_ERR_UNSUPPORTED_OPERATION) return s;
            }
            return hx::scan::launch_simple(a, st);
        }
        default: return hx::fail(HX_ERR_INVALID_INPUT, "unknown scan variant %d", a->variant);
    }
}

int32_t hx_selective_scan_suggest_splits(const hx_scan_args *a) {
    if (!a || a->d_state != 16 || a->batch <= 0 || a->seq_len <= 0 || a->d_inner <= 0) return 1;
    const double chains = (double)a->batch * a->d_inner;
    const double warps_per_sm = chains / 32.0 / hx::sm_count();
    const bool direct = warps_per_sm >= 8.0;
    if (!direct && a->a_geometric && !a->z_is_gate) {
        // few chains, geometric A: the look-back form runs the segments of a chain at the same time.  Its aggregate
        // pass covers all segments but the last, so split until that pass alone has about 8 one-lane-per-channel
        // warps per SM (measured: below that it is short of warps, beyond it the extra work of shorter segments
        // buys nothing), keeping segments of at least 64 steps
        int splits = 1;
        while (splits < 16 && (splits - 1) * warps_per_sm < 8.0 && a->seq_len / (2 * splits) >= 64) splits *= 2;
        return splits;
    }
    // chained segments: CTAs of the kernel AUTO would pick, against the CTA slots of the device (about 3 per SM)
    const int tile = direct ? 128 : (a->io_dtype == HX_BF16 ? 64 : 32);
    const double ctas = (double)a->batch * ((a->d_inner + tile - 1) / tile);
    const double slots = 3.0 * hx::sm_count();
    if (ctas >= 8.0 * slots) return 1;
    int want = (int)(HX_SCAN_CHAIN_WAVES * slots / ctas + 0.999);
    int splits = 1;
    while (splits < want && splits < 16) splits *= 2;
    while (splits > 1 && a->seq_len / splits < 128) splits /= 2;  // keep segments long enough to amortise the hand-over
    return splits;
}

hx_status hx_selective_scan_workspace_bytes(const hx_scan_args *a, size_t *bytes) {
    HX_REQUIRE(a && bytes, HX_ERR_INVALID_INPUT, "hx_selective_scan_workspace_bytes: NULL argument");
    *bytes = 0;
    if (a->variant != HX_SCAN_SEQSPLIT && a->variant != HX_SCAN_LOOKBACK && a->seq_splits <= 1) return HX_OK;
    if (a->variant == HX_SCAN_SIMPLE) return HX_OK;
    int n_seg, seg_len;
    hx::scan::seg_plan(a, hx::scan::kPlanChunk, &n_seg, &seg_len);
    *bytes = hx::scan::workspace_bytes(a, n_seg);
    return HX_OK;
}

// ---- host-buffer form: x, dt, z, Bm, Cm are read from (pinned) host memory and y is written to host
// memory; parameters (A, Dskip, conv_w, conv_b, dt_bias) and h_last stay device pointers.  The device
// staging area is the caller's: dense [B, L, D] / [B, L, N] copies of the five inputs and of y.
static size_t host_stage_bytes(const hx_scan_args *a, size_t *off /* x, dt, z, B, C, y, ws */) {
    const size_t es = hx::dtype_size(a->io_dtype);
    const size_t big = ((size_t)a->batch * a->seq_len * a->d_inner * es + 255) / 256 * 256;
    const size_t small = ((size_t)a->batch * a->seq_len * a->d_state * es + 255) / 256 * 256;
    size_t o = 0;
    off[0] = o; o += big;
    off[1] = o; o += big;
    off[2] = o; o += a->z ? big : 0;
    off[3] = o; o += small;
    off[4] = o; o += small;
    off[5] = o; o += big;
    off[6] = o;
    size_t inner = 0;
    hx_selective_scan_workspace_bytes(a, &inner);  // 0 unless the call splits the sequence
    return o + inner + 256;
}

hx_status hx_selective_scan_host_workspace_bytes(const hx_scan_args *a, size_t *bytes) {
    HX_REQUIRE(a && bytes, HX_ERR_INVALID_INPUT, "hx_selective_scan_host_workspace_bytes: NULL argument");
    hx_status s = hx::scan::validate_dims(a);
    if (s != HX_OK) return s;
    size_t off[7];
    *bytes = host_stage_bytes(a, off);
    return HX_OK;
}

hx_status hx_selective_scan_host(const hx_scan_args *a, void *dev_workspace, size_t dev_workspace_bytes, void *stream) {
    HX_REQUIRE(a != nullptr, HX_ERR_INVALID_INPUT, "hx_selective_scan_host: args is NULL");
    hx_status s = hx::scan::validate(a);
    if (s != HX_OK) return s;
    if (a->batch == 0 || a->seq_len == 0 || a->d_inner == 0) return HX_OK;
    HX_REQUIRE(a->W_dt == nullptr && a->dt != nullptr, HX_ERR_UNSUPPORTED_OPERATION,
               "hx_selective_scan_host takes dt as a host tensor; the fused dt projection is a device-side form");
    size_t off[7];
    const size_t need = host_stage_bytes(a, off);
    HX_REQUIRE(dev_workspace && dev_workspace_bytes >= need, HX_ERR_INVALID_INPUT,
               "hx_selective_scan_host needs a device workspace of %zu bytes (got %zu)", need, dev_workspace_bytes);
    char *ws = reinterpret_cast<char *>((reinterpret_cast<uintptr_t>(dev_workspace) + 255) & ~uintptr_t(255));
    cudaStream_t st = (cudaStream_t)stream;
    const size_t es = hx::dtype_size(a->io_dtype);
    const size_t D = a->d_inner, N = a->d_state, L = a->seq_len;
    // strided host views are gathered by 2-D copies (one per batch row), dense ones by a single copy
    auto h2d = [&](void *dst, const void *src, int64_t bstride, int64_t rstride, size_t width) -> hx_status {
        for (int b = 0; b < a->batch; ++b) {
            const char *sp = static_cast<const char *>(src) + (size_t)b * bstride * es;
            char *dp = static_cast<char *>(dst) + (size_t)b * L * width * es;
            HX_CUDA(cudaMemcpy2DAsync(dp, width * es, sp, (size_t)rstride * es, width * es, L, cudaMemcpyHostToDevice, st));
        }
        return HX_OK;
    };
    hx_scan_args d = *a;
    d.x = ws + off[0]; d.dt = ws + off[1]; d.z = a->z ? ws + off[2] : nullptr;
    d.Bm = ws + off[3]; d.Cm = ws + off[4]; d.y = ws + off[5];
    d.x_row_stride = d.dt_row_stride = d.z_row_stride = d.y_row_stride = (int64_t)D;
    d.x_batch_stride = d.dt_batch_stride = d.z_batch_stride = d.y_batch_stride = (int64_t)(L * D);
    d.B_row_stride = d.C_row_stride = (int64_t)N;
    d.B_batch_stride = d.C_batch_stride = (int64_t)(L * N);
    d.workspace = ws + off[6];
    d.workspace_bytes = dev_workspace_bytes - (size_t)((ws + off[6]) - static_cast<char *>(dev_workspace));
    if ((s = h2d(const_cast<void *>(d.x), a->x, a->x_batch_stride, a->x_row_stride, D)) != HX_OK) return s;
    if ((s = h2d(const_cast<void *>(d.dt), a->dt, a->dt_batch_stride, a->dt_row_stride, D)) != HX_OK) return s;
    if (a->z && (s = h2d(const_cast<void *>(d.z), a->z, a->z_batch_stride, a->z_row_stride, D)) != HX_OK) return s;
    if ((s = h2d(const_cast<void *>(d.Bm), a->Bm, a->B_batch_stride, a->B_row_stride, N)) != HX_OK) return s;
    if ((s = h2d(const_cast<void *>(d.Cm), a->Cm, a->C_batch_stride, a->C_row_stride, N)) != HX_OK) return s;
    if ((s = hx_selective_scan_fwd(&d, stream)) != HX_OK) return s;
    for (int b = 0; b < a->batch; ++b) {
        char *hp = static_cast<char *>(a->y) + (size_t)b * a->y_batch_stride * es;
        const char *dp = static_cast<const char *>(d.y) + (size_t)b * L * D * es;
        HX_CUDA(cudaMemcpy2DAsync(hp, (size_t)a->y_row_stride * es, dp, D * es, D * es, L, cudaMemcpyDeviceToHost, st));
    }
    return HX_OK;
}

// ---- allocation-free entry point -----------------------------------------------------------------
// Scratch for hx_selective_scan_fwd_noalloc: a fixed array in the library's device image, so the call
// never enters the CUDA allocator.  Every device that loads the library holds it until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[HX_SCAN_NOALLOC_SCRATCH_BYTES];

namespace {
std::mutex g_noalloc_mu;
void *g_noalloc_ptr[64] = {nullptr};  // device address of g_noalloc_scratch, per device ordinal
}  // namespace

hx_status hx_selective_scan_fwd_noalloc(const hx_scan_args *a, void *stream) {
    hx_status s = hx::scan::validate(a);
    if (s != HX_OK) return s;
    if (a->batch == 0 || a->seq_len == 0 || a->d_inner == 0) return HX_OK;
    hx_scan_args b = *a;
    b.variant = HX_SCAN_SEQSPLIT;
    size_t need = 0;
    if ((s = hx_selective_scan_workspace_bytes(&b, &need)) != HX_OK) return s;
    HX_REQUIRE(need <= (size_t)HX_SCAN_NOALLOC_SCRATCH_BYTES, HX_ERR_INVALID_INPUT,
               "hx_selective_scan_fwd_noalloc: this problem needs %zu bytes of carry scratch, the built-in array holds "
               "%zu; use fewer seq_splits, a smaller batch * d_inner, or hx_selective_scan_fwd with your own workspace",
               need, (size_t)HX_SCAN_NOALLOC_SCRATCH_BYTES);
    int dev = 0;
    HX_CUDA(cudaGetDevice(&dev));
    HX_REQUIRE(dev >= 0 && dev < 64, HX_ERR_BACKEND, "device ordinal %d out of range", dev);
    void *ptr = nullptr;
    {
        // One-time set-up per device, with that device current: the array's name is only a host-side
        // stand-in, the kernel needs the address cudaGetSymbolAddress returns for THIS device.
        std::lock_guard<std::mutex> lock(g_noalloc_mu);
        if (g_noalloc_ptr[dev] == nullptr) {
            void *p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || p == nullptr) {
                cudaGetLastError();
                return hx::fail(HX_ERR_BACKEND, "cudaGetSymbolAddress(g_noalloc_scratch) failed on device %d: %s", dev,
                                cudaGetErrorString(e));
            }
            g_noalloc_ptr[dev] = p;
        }
        ptr = g_noalloc_ptr[dev];
    }
    b.workspace = ptr;
    b.workspace_bytes = (size_t)HX_SCAN_NOALLOC_SCRATCH_BYTES;
    // launch_tiled clears the carry flags with a memset on `stream` before the kernel, so nothing is
    // inherited from the previous call; the carry states themselves are always written before they are read.
    return hx::scan::launch_tiled(&b, true, (cudaStream_t)stream);
}

hx_status hx_debug_scan_orphan_segment(const hx_scan_args *a, int32_t polls, void *stream) {
    hx_status s = hx::scan::validate(a);
    if (s != HX_OK) return s;
    HX_REQUIRE(polls >= 1 && polls <= hx::scan::kCarryPollsDefault, HX_ERR_INVALID_INPUT, "polls %d outside [1, 2^22]", polls);
    HX_REQUIRE(a->d_state == 16 && a->seq_splits == 2 && a->seq_len > 2 * hx::scan::kPlanChunk, HX_ERR_INVALID_INPUT,
               "hx_debug_scan_orphan_segment: d_state 16, seq_splits 2 and more than 64 steps");
    cudaStream_t st = (cudaStream_t)stream;
    HX_CUDA(cudaMemcpyToSymbolAsync(hx::scan::g_carry_polls, &polls, sizeof(int), 0, cudaMemcpyHostToDevice, st));
    hx::scan::t_orphan_from = 1;  // segment 1 alone: nobody publishes the flag it waits for
    s = hx::scan::launch_direct(a, true, st);
    hx::scan::t_orphan_from = 0;
    const int def = hx::scan::kCarryPollsDefault;
    cudaMemcpyToSymbolAsync(hx::scan::g_carry_polls, &def, sizeof(int), 0, cudaMemcpyHostToDevice, st);
    return s;
}

hx_status hx_scan_check_geometric(const float *A, int32_t d_inner, int32_t d_state, int32_t *is_geometric) {
    HX_REQUIRE(A && is_geometric, HX_ERR_INVALID_INPUT, "hx_scan_check_geometric: NULL argument");
    HX_REQUIRE(d_inner >= 0 && d_state >= 1, HX_ERR_INVALID_DIMENSION, "bad dimensions %d x %d", d_inner, d_state);
    std::vector<float> h((size_t)d_inner * d_state);
    if (!h.empty()) HX_CUDA(cudaMemcpy(h.data(), A, h.size() * sizeof(float), cudaMemcpyDeviceToHost));
    int ok = 1;
    for (int d = 0; d < d_inner && ok; ++d) {
        const float a0 = h[(size_t)d * d_state];
        if (!(a0 <= 0.f)) ok = 0;  // decays only; also rejects NaN
        for (int n = 1; n < d_state && ok; ++n) {
            const float want = (float)(n + 1) * a0, got = h[(size_t)d * d_state + n];
            if (fabsf(got - want) > 1e-6f * fabsf(want)) ok = 0;
        }
    }
    *is_geometric = ok;
    return HX_OK;
}

}  // extern "C"
