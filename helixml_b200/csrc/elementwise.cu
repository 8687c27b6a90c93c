// Memory-bound helpers around the scan: causal depthwise conv + SiLU, RMSNorm (+ residual add),
// byte-embedding gather, SiLU.  All are single-pass, 128-bit vectorised where the layout allows.
#include "hx_common.cuh"

namespace hx {
namespace ew {

template <typename T> struct Vec;  // 16-byte vector of T
template <> struct Vec<float> {
    static constexpr int N = 4;
    float v[4];
    __device__ __forceinline__ void load(const float *p) {
        const float4 f = *reinterpret_cast<const float4 *>(p);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    }
    __device__ __forceinline__ void store(float *p) const {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    float v[8];
    __device__ __forceinline__ void load(const __nv_bfloat16 *p) {
        const uint4 r = *reinterpret_cast<const uint4 *>(p);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            v[2 * k] = __uint_as_float(w[k] << 16);
            v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
        }
    }
    __device__ __forceinline__ void store(__nv_bfloat16 *p) const {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
            w[k] = *reinterpret_cast<const uint32_t *>(&h);
        }
        *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// ---------------------------------------------------------------- conv1d + SiLU
// Thread = one 16-byte channel group x TB consecutive time steps (sliding window over the taps).
// FASTM (bf16 I/O): SiLU through ex2/rcp on the special-function unit; fp32 I/O keeps the accurate form.
template <typename T, bool VEC, int TB, bool FASTM = (sizeof(T) == 2)>
__global__ void __launch_bounds__(64)
conv_silu_kernel(const T *__restrict__ x, int64_t xb, int64_t xr, const float *__restrict__ cw, const float *__restrict__ cb,
                 T *__restrict__ u, int64_t ub, int64_t ur, int L, int D, int K) {
    constexpr int VN = VEC ? Vec<T>::N : 1;
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    const int d = g * VN;
    if (d >= D) return;
    const int t0 = blockIdx.y * TB;
    const int b = blockIdx.z;
    float w[VN][4], bias[VN];
#pragma unroll
    for (int e = 0; e < VN; ++e) {
        if (K == 4 && (reinterpret_cast<uintptr_t>(cw) & 15) == 0) {
            const float4 f = *reinterpret_cast<const float4 *>(cw + (int64_t)(d + e) * 4);
            w[e][0] = f.x; w[e][1] = f.y; w[e][2] = f.z; w[e][3] = f.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // tap j of the 4-wide window is tap j-(4-K) of the K given ones
                const int src = j - (4 - K);
                w[e][j] = src >= 0 ? cw[(int64_t)(d + e) * K + src] : 0.f;
            }
        }
        bias[e] = cb ? cb[d + e] : 0.f;
    }
    const T *xp = x + b * xb + d;
    T *up = u + b * ub + d;
    float win[3][VN];  // x[t-3], x[t-2], x[t-1]
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        const int t = t0 - 3 + j;
        if (t >= 0) {
            if constexpr (VEC) {
                Vec<T> v;
                v.load(xp + t * xr);
#pragma unroll
                for (int e = 0; e < VN; ++e) win[j][e] = v.v[e];
            } else {
                win[j][0] = ld_f32(xp + t * xr);
            }
        } else {
#pragma unroll
            for (int e = 0; e < VN; ++e) win[j][e] = 0.f;
        }
    }
#pragma unroll 4
    for (int k = 0; k < TB; ++k) {
        const int t = t0 + k;
        if (t >= L) break;
        float cur[VN], out[VN];
        if constexpr (VEC) {
            Vec<T> v;
            v.load(xp + t * xr);
#pragma unroll
            for (int e = 0; e < VN; ++e) cur[e] = v.v[e];
        } else {
            cur[0] = ld_f32(xp + t * xr);
        }
#pragma unroll
        for (int e = 0; e < VN; ++e) {
            float c = bias[e];
            c += w[e][0] * win[0][e];
            c += w[e][1] * win[1][e];
            c += w[e][2] * win[2][e];
            c += w[e][3] * cur[e];
            out[e] = FASTM ? silu_fast(c) : silu_acc(c);
            win[0][e] = win[1][e];
            win[1][e] = win[2][e];
            win[2][e] = cur[e];
        }
        if constexpr (VEC) {
            Vec<T> v;
#pragma unroll
            for (int e = 0; e < VN; ++e) v.v[e] = out[e];
            v.store(up + t * ur);
        } else {
            st_f32(up + t * ur, out[0]);
        }
    }
}

// Lean bf16 variant: a thread owns CH (2 or 4) adjacent channels and a strip of TB time steps; a warp reads
// 32*CH contiguous channels per row.  Rows are fetched eight at a time before any arithmetic, so every thread
// keeps eight loads in flight, and the strips are short enough (TB = 32) that the grid has several thousand
// CTAs to spread over the SMs.  The window of the three previous rows lives in registers.
template <int CH> struct PackBf16;
template <> struct PackBf16<2> { using T = uint32_t; };
template <> struct PackBf16<4> { using T = uint2; };

template <int CH>
__device__ __forceinline__ void unpack_bf16(const typename PackBf16<CH>::T &v, float *f) {
    const uint32_t *p = reinterpret_cast<const uint32_t *>(&v);
#pragma unroll
    for (int i = 0; i < CH / 2; ++i) {
        f[2 * i] = __uint_as_float(p[i] << 16);
        f[2 * i + 1] = __uint_as_float(p[i] & 0xffff0000u);
    }
}

template <int CH, int TB>
__global__ void __launch_bounds__(128)
conv_silu_strip_kernel(const __nv_bfloat16 *__restrict__ x, int64_t xb, int64_t xr, const float *__restrict__ cw,
                       const float *__restrict__ cb, __nv_bfloat16 *__restrict__ u, int64_t ub, int64_t ur, int L, int D, int K) {
    using V = typename PackBf16<CH>::T;
    const int d = (blockIdx.x * blockDim.x + threadIdx.x) * CH;
    if (d >= D) return;
    const int t0 = blockIdx.y * TB;
    const int b = blockIdx.z;
    const int n = min(TB, L - t0);
    // the strips are short, so the per-thread set-up counts: with four taps a channel's weights are one 16-byte load
    float w[4][CH], bias[CH];
#pragma unroll
    for (int e = 0; e < CH; ++e) {
        if (K == 4 && (reinterpret_cast<uintptr_t>(cw) & 15) == 0) {  // a 4-byte-aligned slice takes the scalar loads
            const float4 q = __ldg(reinterpret_cast<const float4 *>(cw) + d + e);
            w[0][e] = q.x; w[1][e] = q.y; w[2][e] = q.z; w[3][e] = q.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // tap j of the 4-wide window is tap j-(4-K) of the K given ones
                const int src = j - (4 - K);
                w[j][e] = src >= 0 ? cw[(int64_t)(d + e) * K + src] : 0.f;
            }
        }
    }
    // no branch around a load here: a conditional load would have to land before the row loads below could be
    // issued, and with strips this short one more round trip to memory costs a quarter of the kernel's time
    const float *cbp = cb ? cb : cw;
#pragma unroll
    for (int e = 0; e < CH; ++e) {
        const float v = cbp[d + e];
        bias[e] = cb ? v : 0.f;
    }
    const __nv_bfloat16 *xp = x + b * xb + d + (int64_t)t0 * xr;
    __nv_bfloat16 *up = u + b * ub + d + (int64_t)t0 * ur;
    auto ld = [&](int k) { return *reinterpret_cast<const V *>(xp + (int64_t)k * xr); };
    float w0[CH], w1[CH], w2[CH];  // x[t-3], x[t-2], x[t-1]; rows before the sequence start read row t0 and are zeroed
    unpack_bf16<CH>(ld(t0 >= 3 ? -3 : 0), w0);
    unpack_bf16<CH>(ld(t0 >= 2 ? -2 : 0), w1);
    unpack_bf16<CH>(ld(t0 >= 1 ? -1 : 0), w2);
#pragma unroll
    for (int e = 0; e < CH; ++e) {
        w0[e] = t0 >= 3 ? w0[e] : 0.f;
        w1[e] = t0 >= 2 ? w1[e] : 0.f;
        w2[e] = t0 >= 1 ? w2[e] : 0.f;
    }
    auto step = [&](const V &v, int k) {
        float cur[CH];
        unpack_bf16<CH>(v, cur);
        V o;
        uint32_t *op = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
        for (int e = 0; e < CH; e += 2) {
            float c0 = fmaf(w[0][e], w0[e], bias[e]), c1 = fmaf(w[0][e + 1], w0[e + 1], bias[e + 1]);
            c0 = fmaf(w[1][e], w1[e], c0); c1 = fmaf(w[1][e + 1], w1[e + 1], c1);
            c0 = fmaf(w[2][e], w2[e], c0); c1 = fmaf(w[2][e + 1], w2[e + 1], c1);
            c0 = fmaf(w[3][e], cur[e], c0); c1 = fmaf(w[3][e + 1], cur[e + 1], c1);
            const __nv_bfloat162 ob = __floats2bfloat162_rn(silu_tanh(c0), silu_tanh(c1));
            op[e / 2] = *reinterpret_cast<const uint32_t *>(&ob);
        }
        *reinterpret_cast<V *>(up + (int64_t)k * ur) = o;
#pragma unroll
        for (int e = 0; e < CH; ++e) { w0[e] = w1[e]; w1[e] = w2[e]; w2[e] = cur[e]; }
    };
    int k0 = 0;
    for (; k0 + 8 <= n; k0 += 8) {
        V v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = ld(k0 + e);
#pragma unroll
        for (int e = 0; e < 8; ++e) step(v[e], k0 + e);
    }
    for (; k0 < n; ++k0) step(ld(k0), k0);
}

// ---------------------------------------------------------------- RMSNorm (+ residual add)
// One warp per row.  residual (fp32) is updated in place with x when both are given.
template <typename TX, typename TY>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const TX *x, float *residual, const float *w, TY *y, int64_t rows, int d, float eps) {
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const TX *xr = x ? x + row * d : nullptr;
    float *rr = residual ? residual + row * d : nullptr;
    float ss = 0.f;
    for (int j = lane; j < d; j += 32) {
        float v = xr ? ld_f32(xr + j) : 0.f;
        if (rr) {
            v += rr[j];
            if (xr) rr[j] = v;
        }
        ss += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int j = lane; j < d; j += 32) {
        const float v = rr ? rr[j] : ld_f32(xr + j);
        st_f32(y + row * d + j, v * inv * w[j]);
    }
}

// Vector path: d is a multiple of 8 and at most 8*32*NV; every lane keeps its NV groups of 8 values in
// registers between the two passes, so each operand crosses HBM once.
template <typename TX, typename TY, int NV, bool HAS_X>
__global__ void __launch_bounds__(256)
rmsnorm_vec_kernel(const TX *x, float *residual, const float *w, TY *y, int64_t rows, int d, float eps) {
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int groups = d / 8;
    float v[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int g = lane + 32 * i;
        if (g < groups) {
            const int64_t off = row * d + g * 8;
            if constexpr (HAS_X) {
                if constexpr (sizeof(TX) == 2) {
                    Vec<__nv_bfloat16> t;
                    t.load(reinterpret_cast<const __nv_bfloat16 *>(x) + off);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[i][e] = t.v[e];
                } else {
                    Vec<float> t0, t1;
                    t0.load(reinterpret_cast<const float *>(x) + off);
                    t1.load(reinterpret_cast<const float *>(x) + off + 4);
#pragma unroll
                    for (int e = 0; e < 4; ++e) { v[i][e] = t0.v[e]; v[i][4 + e] = t1.v[e]; }
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[i][e] = 0.f;
            }
            if (residual) {
                Vec<float> r0, r1;
                r0.load(residual + off);
                r1.load(residual + off + 4);
#pragma unroll
                for (int e = 0; e < 4; ++e) { v[i][e] += r0.v[e]; v[i][4 + e] += r1.v[e]; }
                if constexpr (HAS_X) {  // nothing was added when x is NULL: the stream is read, not rewritten
#pragma unroll
                    for (int e = 0; e < 4; ++e) { r0.v[e] = v[i][e]; r1.v[e] = v[i][4 + e]; }
                    r0.store(residual + off);
                    r1.store(residual + off + 4);
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int g = lane + 32 * i;
        if (g < groups) {
            const int64_t off = row * d + g * 8;
            Vec<float> w0, w1;
            w0.load(w + g * 8);
            w1.load(w + g * 8 + 4);
            if constexpr (sizeof(TY) == 2) {
                Vec<__nv_bfloat16> o;
#pragma unroll
                for (int e = 0; e < 4; ++e) { o.v[e] = v[i][e] * inv * w0.v[e]; o.v[4 + e] = v[i][4 + e] * inv * w1.v[e]; }
                o.store(reinterpret_cast<__nv_bfloat16 *>(y) + off);
            } else {
                Vec<float> o0, o1;
#pragma unroll
                for (int e = 0; e < 4; ++e) { o0.v[e] = v[i][e] * inv * w0.v[e]; o1.v[e] = v[i][4 + e] * inv * w1.v[e]; }
                o0.store(reinterpret_cast<float *>(y) + off);
                o1.store(reinterpret_cast<float *>(y) + off + 4);
            }
        }
    }
}

// ---------------------------------------------------------------- embedding gather
template <typename TE, typename TO>
__global__ void __launch_bounds__(256)
embedding_kernel(const uint8_t *tok, const TE *emb, TO *out, int64_t n, int d) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * d) return;
    const int64_t r = i / d;
    const int j = (int)(i - r * d);
    st_f32(out + i, ld_f32(emb + (int64_t)tok[r] * d + j));
}

// bf16 table, rows of a multiple of 8 elements: a thread moves 8 elements (one 16-byte load of the table row,
// 16 or 32 bytes stored) and reads its token once
template <typename TO>
__global__ void __launch_bounds__(256)
embedding_vec_kernel(const uint8_t *__restrict__ tok, const __nv_bfloat16 *__restrict__ emb, TO *__restrict__ out, int64_t n, int d) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // group of 8 elements
    const int gpr = d >> 3;
    if (i >= n * gpr) return;
    const int64_t r = i / gpr;
    const int j = (int)(i - r * gpr) << 3;
    const uint4 v = *reinterpret_cast<const uint4 *>(emb + (int64_t)tok[r] * d + j);
    TO *o = out + r * d + j;
    if constexpr (sizeof(TO) == 2) {
        *reinterpret_cast<uint4 *>(o) = v;
    } else {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        float f[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            f[2 * e] = __uint_as_float(w[e] << 16);
            f[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
        }
        *reinterpret_cast<float4 *>(o) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4 *>(o + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) silu_kernel(const T *x, T *y, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) st_f32(y + i, silu_acc(ld_f32(x + i)));
}

template <typename T>
__global__ void __launch_bounds__(256) residual_add_kernel(float *resid, const T *x, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) resid[i] += ld_f32(x + i);
}

}  // namespace ew

hx_status residual_add(float *resid, const void *x, int x_dtype, int64_t n, cudaStream_t st) {
    if (n <= 0) return HX_OK;
    dim3 grid((unsigned)((n + 255) / 256)), block(256);
    if (x_dtype == HX_BF16) ew::residual_add_kernel<<<grid, block, 0, st>>>(resid, static_cast<const __nv_bfloat16 *>(x), n);
    else ew::residual_add_kernel<<<grid, block, 0, st>>>(resid, static_cast<const float *>(x), n);
    return check_launch("residual_add_kernel");
}

}  // namespace hx

extern "C" {

hx_status hx_conv1d_silu_fwd(const void *x, int64_t xb, int64_t xr, const float *conv_w, const float *conv_b, void *u,
                             int64_t ub, int64_t ur, int32_t batch, int32_t seq_len, int32_t d_inner, int32_t d_conv,
                             int32_t io_dtype, void *stream) {
    using namespace hx::ew;
    HX_REQUIRE(batch >= 0 && seq_len >= 0 && d_inner >= 0, HX_ERR_INVALID_DIMENSION, "negative dimension");
    HX_REQUIRE(d_conv >= 1 && d_conv <= 4, HX_ERR_INVALID_DIMENSION, "d_conv %d outside [1, 4]", d_conv);
    HX_REQUIRE(io_dtype == HX_F32 || io_dtype == HX_BF16, HX_ERR_DTYPE_MISMATCH, "io_dtype %d unsupported", io_dtype);
    if (batch == 0 || seq_len == 0 || d_inner == 0) return HX_OK;
    HX_REQUIRE(x && u && conv_w, HX_ERR_INVALID_INPUT, "x, u and conv_w must not be NULL");
    HX_REQUIRE(xr >= d_inner && ur >= d_inner, HX_ERR_SHAPE_MISMATCH, "row stride smaller than d_inner");
    HX_REQUIRE(batch <= 65535, HX_ERR_INVALID_DIMENSION, "batch %d exceeds the grid limit", batch);
    cudaStream_t st = (cudaStream_t)stream;
    constexpr int TB = 32;
    const int es = io_dtype == HX_BF16 ? 2 : 4, vn = 16 / es;
    const bool vec = d_inner % vn == 0 && xr % vn == 0 && ur % vn == 0 && xb % vn == 0 && ub % vn == 0 &&
                     (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(u) & 15) == 0;
    const int groups = vec ? d_inner / vn : d_inner;
    dim3 grid((groups + 63) / 64, (seq_len + TB - 1) / TB, batch), block(64);
    if (io_dtype == HX_BF16) {
        auto fits = [&](int ch) {
            return d_inner % ch == 0 && xr % ch == 0 && ur % ch == 0 && xb % ch == 0 && ub % ch == 0 &&
                   (reinterpret_cast<uintptr_t>(x) % (2 * ch)) == 0 && (reinterpret_cast<uintptr_t>(u) % (2 * ch)) == 0;
        };
        constexpr int TBS = 32;
        auto xp = static_cast<const __nv_bfloat16 *>(x);
        auto up = static_cast<__nv_bfloat16 *>(u);
        if (fits(4)) {
            dim3 g2((d_inner / 4 + 127) / 128, (seq_len + TBS - 1) / TBS, batch);
            conv_silu_strip_kernel<4, TBS><<<g2, 128, 0, st>>>(xp, xb, xr, conv_w, conv_b, up, ub, ur, seq_len, d_inner, d_conv);
            return hx::check_launch("conv_silu_strip_kernel");
        }
        if (fits(2)) {
            dim3 g2((d_inner / 2 + 127) / 128, (seq_len + TBS - 1) / TBS, batch);
            conv_silu_strip_kernel<2, TBS><<<g2, 128, 0, st>>>(xp, xb, xr, conv_w, conv_b, up, ub, ur, seq_len, d_inner, d_conv);
            return hx::check_launch("conv_silu_strip_kernel");
        }
    }
    if (io_dtype == HX_BF16) {
        auto xp = static_cast<const __nv_bfloat16 *>(x);
        auto up = static_cast<__nv_bfloat16 *>(u);
        if (vec) conv_silu_kernel<__nv_bfloat16, true, TB><<<grid, block, 0, st>>>(xp, xb, xr, conv_w, conv_b, up, ub, ur, seq_len, d_inner, d_conv);
        else conv_silu_kernel<__nv_bfloat16, false, TB><<<grid, block, 0, st>>>(xp, xb, xr, conv_w, conv_b, up, ub, ur, seq_len, d_inner, d_conv);
    } else {
        auto xp = static_cast<const float *>(x);
        auto up = static_cast<float *>(u);
        if (vec) conv_silu_kernel<float, true, TB><<<grid, block, 0, st>>>(xp, xb, xr, conv_w, conv_b, up, ub, ur, seq_len, d_inner, d_conv);
        else conv_silu_kernel<float, false, TB><<<grid, block, 0, st>>>(xp, xb, xr, conv_w, conv_b, up, ub, ur, seq_len, d_inner, d_conv);
    }
    return hx::check_launch("conv_silu_kernel");
}

hx_status hx_rmsnorm_fwd(const void *x, int32_t x_dtype, float *residual, const float *w, void *y, int32_t y_dtype,
                         int64_t rows, int32_t d, float eps, void *stream) {
    using namespace hx::ew;
    HX_REQUIRE(rows >= 0 && d >= 1, HX_ERR_INVALID_DIMENSION, "bad dimensions rows %lld, d %d", (long long)rows, d);
    if (rows == 0) return HX_OK;
    HX_REQUIRE((x || residual) && w && y, HX_ERR_INVALID_INPUT, "x or residual, w and y must not be NULL");
    HX_REQUIRE((x_dtype == HX_F32 || x_dtype == HX_BF16) && (y_dtype == HX_F32 || y_dtype == HX_BF16),
               HX_ERR_DTYPE_MISMATCH, "dtype unsupported");
    cudaStream_t st = (cudaStream_t)stream;
    const int wpb = 8;
    dim3 grid((unsigned)((rows + wpb - 1) / wpb)), block(wpb * 32);
    const bool xb = x_dtype == HX_BF16, yb = y_dtype == HX_BF16;
    auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (d % 8 == 0 && d <= 8 * 32 * 4 && al16(x) && al16(residual) && al16(w) && al16(y)) {
        // every lane holds up to 4 groups of 8 values (d <= 1024)
#define HX_NORM_VEC(TX, TY)                                                                                      \
        do {                                                                                                     \
            if (x) rmsnorm_vec_kernel<TX, TY, 4, true><<<grid, block, 0, st>>>(static_cast<const TX *>(x), residual, w,  \
                                                                               static_cast<TY *>(y), rows, d, eps);  \
            else rmsnorm_vec_kernel<TX, TY, 4, false><<<grid, block, 0, st>>>(static_cast<const TX *>(x), residual, w,   \
                                                                              static_cast<TY *>(y), rows, d, eps);  \
        } while (0)
        if (xb && yb) HX_NORM_VEC(__nv_bfloat16, __nv_bfloat16);
        else if (xb) HX_NORM_VEC(__nv_bfloat16, float);
        else if (yb) HX_NORM_VEC(float, __nv_bfloat16);
        else HX_NORM_VEC(float, float);
#undef HX_NORM_VEC
        return hx::check_launch("rmsnorm_vec_kernel");
    }
    if (xb && yb) rmsnorm_kernel<<<grid, block, 0, st>>>(static_cast<const __nv_bfloat16 *>(x), residual, w, static_cast<__nv_bfloat16 *>(y), rows, d, eps);
    else if (xb) rmsnorm_kernel<<<grid, block, 0, st>>>(static_cast<const __nv_bfloat16 *>(x), residual, w, static_cast<float *>(y), rows, d, eps);
    else if (yb) rmsnorm_kernel<<<grid, block, 0, st>>>(static_cast<const float *>(x), residual, w, static_cast<__nv_bfloat16 *>(y), rows, d, eps);
    else rmsnorm_kernel<<<grid, block, 0, st>>>(static_cast<const float *>(x), residual, w, static_cast<float *>(y), rows, d, eps);
    return hx::check_launch("rmsnorm_kernel");
}

hx_status hx_embedding_fwd(const uint8_t *tokens, const void *emb, int32_t emb_dtype, void *out, int32_t out_dtype,
                           int64_t n_tokens, int32_t d_model, void *stream) {
    using namespace hx::ew;
    HX_REQUIRE(n_tokens >= 0 && d_model >= 1, HX_ERR_INVALID_DIMENSION, "bad dimensions");
    if (n_tokens == 0) return HX_OK;
    HX_REQUIRE(tokens && emb && out, HX_ERR_INVALID_INPUT, "tokens, emb and out must not be NULL");
    HX_REQUIRE((emb_dtype == HX_F32 || emb_dtype == HX_BF16) && (out_dtype == HX_F32 || out_dtype == HX_BF16),
               HX_ERR_DTYPE_MISMATCH, "dtype unsupported");
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t total = n_tokens * d_model;
    dim3 grid((unsigned)((total + 255) / 256)), block(256);
    const bool eb = emb_dtype == HX_BF16, ob = out_dtype == HX_BF16;
    if (eb && d_model % 8 == 0 && (reinterpret_cast<uintptr_t>(emb) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        const int64_t groups = n_tokens * (d_model / 8);
        dim3 g8((unsigned)((groups + 255) / 256));
        if (ob) embedding_vec_kernel<<<g8, block, 0, st>>>(tokens, static_cast<const __nv_bfloat16 *>(emb), static_cast<__nv_bfloat16 *>(out), n_tokens, d_model);
        else embedding_vec_kernel<<<g8, block, 0, st>>>(tokens, static_cast<const __nv_bfloat16 *>(emb), static_cast<float *>(out), n_tokens, d_model);
        return hx::check_launch("embedding_vec_kernel");
    }
    if (eb && ob) embedding_kernel<<<grid, block, 0, st>>>(tokens, static_cast<const __nv_bfloat16 *>(emb), static_cast<__nv_bfloat16 *>(out), n_tokens, d_model);
    else if (eb) embedding_kernel<<<grid, block, 0, st>>>(tokens, static_cast<const __nv_bfloat16 *>(emb), static_cast<float *>(out), n_tokens, d_model);
    else if (ob) embedding_kernel<<<grid, block, 0, st>>>(tokens, static_cast<const float *>(emb), static_cast<__nv_bfloat16 *>(out), n_tokens, d_model);
    else embedding_kernel<<<grid, block, 0, st>>>(tokens, static_cast<const float *>(emb), static_cast<float *>(out), n_tokens, d_model);
    return hx::check_launch("embedding_kernel");
}

hx_status hx_silu_fwd(const void *x, void *y, int64_t n, int32_t io_dtype, void *stream) {
    using namespace hx::ew;
    HX_REQUIRE(n >= 0, HX_ERR_INVALID_DIMENSION, "negative size");
    if (n == 0) return HX_OK;
    HX_REQUIRE(x && y, HX_ERR_INVALID_INPUT, "x and y must not be NULL");
    HX_REQUIRE(io_dtype == HX_F32 || io_dtype == HX_BF16, HX_ERR_DTYPE_MISMATCH, "io_dtype %d unsupported", io_dtype);
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid((unsigned)((n + 255) / 256)), block(256);
    if (io_dtype == HX_BF16) silu_kernel<<<grid, block, 0, st>>>(static_cast<const __nv_bfloat16 *>(x), static_cast<__nv_bfloat16 *>(y), n);
    else silu_kernel<<<grid, block, 0, st>>>(static_cast<const float *>(x), static_cast<float *>(y), n);
    return hx::check_launch("silu_kernel");
}

}  // extern "C"
