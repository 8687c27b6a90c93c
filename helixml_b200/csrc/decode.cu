// Single-token decode step of the Mamba block: the recurrent form of the prefill path.  Prefill leaves, per
// layer, the scan's final state h [B, E, N] (fp32) and the last three conv inputs [B, 3, E]; one step then costs
// three small GEMMs and two element-wise kernels:
//   xz = x W_in^T -> conv_step (window in, u out, window shifted) -> [dt_low | B | C] = u W_x^T ->
//   ssm_step (dt projection + bias + softplus, h <- exp(dt A) h + dt B u, y = C.h + D u, y *= silu(z)) -> y W_out^T
// The step is bound by reading the weights once (a few MB per block) and by launch latency, so the kernels are
// plain one-thread-per-channel code with libm-accurate math; callers capture the whole step in a CUDA graph.
#include <cstring>

#include "hx_common.cuh"

namespace hx {
namespace decode {

// Conv window layout: state[b][j][d], j = 0..2 holding x[t-3], x[t-2], x[t-1] in the io dtype.
template <typename T>
__global__ void __launch_bounds__(256)
conv_step_kernel(const T *__restrict__ x, int64_t x_stride, T *__restrict__ state, const float *__restrict__ cw,
                 const float *__restrict__ cb, T *__restrict__ u, int B, int E, int K) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)B * E) return;
    const int b = (int)(i / E), d = (int)(i % E);
    T *st = state + (int64_t)b * 3 * E + d;
    const float x0 = ld_f32(st), x1 = ld_f32(st + E), x2 = ld_f32(st + 2 * E);
    const float xc = ld_f32(x + (int64_t)b * x_stride + d);
    float w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {  // tap j of the 4-wide window is tap j-(4-K) of the K given ones
        const int src = j - (4 - K);
        w[j] = src >= 0 ? cw[(int64_t)d * K + src] : 0.f;
    }
    float c = cb ? cb[d] : 0.f;
    c += w[0] * x0;
    c += w[1] * x1;
    c += w[2] * x2;
    c += w[3] * xc;
    st_f32(u + (int64_t)b * E + d, silu_acc(c));
    st_f32(st, x1);
    st_f32(st + E, x2);
    st_f32(st + 2 * E, xc);
}

// One thread per (batch row, channel): dt projection (dot product of length R), softplus, the N state updates,
// the output contraction, skip and gate.  dbc row = [dt_low (R) | B (N) | C (N)].
template <typename T>
__global__ void __launch_bounds__(128)
ssm_step_kernel(const T *__restrict__ u, const T *__restrict__ z, int64_t z_stride, const T *__restrict__ dbc, int W,
                const T *__restrict__ W_dt, const float *__restrict__ b_dt, const float *__restrict__ A,
                const float *__restrict__ Dskip, float *__restrict__ h, T *__restrict__ y, int B, int E, int N, int R) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)B * E) return;
    const int b = (int)(i / E), d = (int)(i % E);
    const T *row = dbc + (int64_t)b * W;
    float v = b_dt ? b_dt[d] : 0.f;
    const T *wr = W_dt + (int64_t)d * R;
    for (int r = 0; r < R; ++r) v = fmaf(ld_f32(row + r), ld_f32(wr + r), v);
    const float dt = softplus_acc(v);
    const float uu = ld_f32(u + (int64_t)b * E + d);
    const float xin = dt * uu;
    float *hp = h + ((int64_t)b * E + d) * N;
    const float *ap = A + (int64_t)d * N;
    float acc = 0.f;
    for (int n = 0; n < N; ++n) {
        const float hn = expf(dt * ap[n]) * hp[n] + xin * ld_f32(row + R + n);
        hp[n] = hn;
        acc = fmaf(ld_f32(row + R + N + n), hn, acc);
    }
    float out = acc + (Dskip ? Dskip[d] : 0.f) * uu;
    if (z) out *= silu_acc(ld_f32(z + (int64_t)b * z_stride + d));
    st_f32(y + (int64_t)b * E + d, out);
}

// The same for the serving shape (bf16, d_state 16, dt_rank a multiple of 8, d_inner a multiple of the block): a
// block covers 128 channels of one batch row, the row's [dt_low | B | C] goes through shared memory once, every
// per-thread operand (W_dt row, the 16 states, the A row) is fetched with 16-byte loads issued together, and the
// 16 decays come from ex2.approx.  Everything a thread needs is in flight before the first dependent operation.
__global__ void __launch_bounds__(128)
ssm_step16_kernel(const __nv_bfloat16 *__restrict__ u, const __nv_bfloat16 *__restrict__ z, int64_t z_stride,
                  const __nv_bfloat16 *__restrict__ dbc, int W, const __nv_bfloat16 *__restrict__ W_dt,
                  const float *__restrict__ b_dt, const float *__restrict__ A, const float *__restrict__ Dskip,
                  float *__restrict__ h, __nv_bfloat16 *__restrict__ y, int E, int R) {
    __shared__ float srow[64 + 32];  // dt_low (R <= 64), B, C as fp32
    const int b = blockIdx.y, d = blockIdx.x * 128 + threadIdx.x;
    const __nv_bfloat16 *row = dbc + (int64_t)b * W;
    for (int j = threadIdx.x; j < R + 32; j += 128) srow[j < R ? j : 64 + (j - R)] = __bfloat162float(row[j]);
    // per-thread operands, all independent loads
    const uint4 *wr = reinterpret_cast<const uint4 *>(W_dt + (int64_t)d * R);
    uint4 wv[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) wv[q] = q * 8 < R ? wr[q] : make_uint4(0u, 0u, 0u, 0u);
    float4 *hp = reinterpret_cast<float4 *>(h + ((int64_t)b * E + d) * 16);
    const float4 *ap = reinterpret_cast<const float4 *>(A + (int64_t)d * 16);
    float4 hv[4], av[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) { hv[q] = hp[q]; av[q] = ap[q]; }
    const float uu = __bfloat162float(u[(int64_t)b * E + d]);
    const float zz = z ? __bfloat162float(z[(int64_t)b * z_stride + d]) : 0.f;
    float v = b_dt ? b_dt[d] : 0.f;
    const float dsk = Dskip ? Dskip[d] : 0.f;
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        if (q * 8 < R) {
            const uint32_t wq[4] = {wv[q].x, wv[q].y, wv[q].z, wv[q].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                v = fmaf(srow[q * 8 + 2 * e], __uint_as_float(wq[e] << 16), v);
                v = fmaf(srow[q * 8 + 2 * e + 1], __uint_as_float(wq[e] & 0xffff0000u), v);
            }
        }
    }
    const float dt = softplus_acc(v);
    const float xin = dt * uu, dl = dt * kLog2e;
    float acc = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        float hq[4] = {hv[q].x, hv[q].y, hv[q].z, hv[q].w};
        const float aq[4] = {av[q].x, av[q].y, av[q].z, av[q].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int n = q * 4 + e;
            hq[e] = fmaf(ex2_approx(dl * aq[e]), hq[e], xin * srow[64 + n]);
            acc = fmaf(srow[64 + 16 + n], hq[e], acc);
        }
        hp[q] = make_float4(hq[0], hq[1], hq[2], hq[3]);
    }
    float out = acc + dsk * uu;
    if (z) out *= silu_acc(zz);
    y[(int64_t)b * E + d] = __float2bfloat16_rn(out);
}

// After a prefill: the last three conv inputs of every sequence (zeros where the sequence is shorter).
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_kernel(const T *__restrict__ x, int64_t xb, int64_t xr, T *__restrict__ state, int B, int L, int E) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)B * 3 * E) return;
    const int d = (int)(i % E), j = (int)((i / E) % 3), b = (int)(i / (3 * (int64_t)E));
    const int t = L - 3 + j;
    st_f32(state + i, t >= 0 ? ld_f32(x + (int64_t)b * xb + (int64_t)t * xr + d) : 0.f);
}

// in_proj of a decode step with its neighbours folded in (bf16 weights, d_model a multiple of 32, batch <= 64):
//   A = rmsnorm(residual) * norm_w is formed on the fly from the fp32 residual stream (the row scale 1/rms is
//   applied to the accumulators at the end, the sum of squares is gathered while the row is read);
//   columns n < E get the conv step (window in, u out, window shifted), columns n >= E are z.
// Work split as in gemm_skinny_kernel: 8 output columns per CTA, 16 warps share K in blocks of 32, mma.sync with
// the k-permuted 8-element operand loads, partial tiles summed through shared memory.
constexpr int kStepWarps = 16;

template <int MT>
__global__ void __launch_bounds__(kStepWarps * 32)
inproj_step_kernel(const float *__restrict__ resid, const float *__restrict__ norm_w, float eps,
                   const __nv_bfloat16 *__restrict__ W, __nv_bfloat16 *__restrict__ conv_state,
                   const float *__restrict__ cw, const float *__restrict__ cb, __nv_bfloat16 *__restrict__ u,
                   __nv_bfloat16 *__restrict__ z, int M, int K, int E, int Kc) {
    __shared__ float partial[kStepWarps * MT * 128];
    __shared__ float ssq_part[kStepWarps][MT * 16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tid = lane & 3;
    const int n0 = blockIdx.x * 8;
    const int n = n0 + g;  // the W row this lane loads (2E is a multiple of 8)
    const __nv_bfloat16 *wrow = W + (int64_t)n * K + tid * 8;
    float acc[MT][4], ssq[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        ssq[mt][0] = ssq[mt][1] = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;
    }
    for (int k0 = warp * 32; k0 < K; k0 += kStepWarps * 32) {
        const uint4 b = *reinterpret_cast<const uint4 *>(wrow + k0);
        const float4 w0 = *reinterpret_cast<const float4 *>(norm_w + k0 + tid * 8);
        const float4 w1 = *reinterpret_cast<const float4 *>(norm_w + k0 + tid * 8 + 4);
        uint4 a[MT][2];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = mt * 16 + h * 8 + g;
                float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f), x1 = x0;
                if (r < M) {
                    const float *xr = resid + (int64_t)r * K + k0 + tid * 8;
                    x0 = *reinterpret_cast<const float4 *>(xr);
                    x1 = *reinterpret_cast<const float4 *>(xr + 4);
                }
                ssq[mt][h] += x0.x * x0.x + x0.y * x0.y + x0.z * x0.z + x0.w * x0.w + x1.x * x1.x + x1.y * x1.y +
                              x1.z * x1.z + x1.w * x1.w;
                const __nv_bfloat162 p0 = __floats2bfloat162_rn(x0.x * w0.x, x0.y * w0.y);
                const __nv_bfloat162 p1 = __floats2bfloat162_rn(x0.z * w0.z, x0.w * w0.w);
                const __nv_bfloat162 p2 = __floats2bfloat162_rn(x1.x * w1.x, x1.y * w1.y);
                const __nv_bfloat162 p3 = __floats2bfloat162_rn(x1.z * w1.z, x1.w * w1.w);
                a[mt][h] = make_uint4(*reinterpret_cast<const uint32_t *>(&p0), *reinterpret_cast<const uint32_t *>(&p1),
                                      *reinterpret_cast<const uint32_t *>(&p2), *reinterpret_cast<const uint32_t *>(&p3));
            }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                         "{%0, %1, %2, %3};"
                         : "+f"(acc[mt][0]), "+f"(acc[mt][1]), "+f"(acc[mt][2]), "+f"(acc[mt][3])
                         : "r"(a[mt][0].x), "r"(a[mt][1].x), "r"(a[mt][0].y), "r"(a[mt][1].y), "r"(b.x), "r"(b.y));
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                         "{%0, %1, %2, %3};"
                         : "+f"(acc[mt][0]), "+f"(acc[mt][1]), "+f"(acc[mt][2]), "+f"(acc[mt][3])
                         : "r"(a[mt][0].z), "r"(a[mt][1].z), "r"(a[mt][0].w), "r"(a[mt][1].w), "r"(b.z), "r"(b.w));
        }
    }
    // sums of squares: the four lanes of a row group hold different k, then the warps hold different k-blocks
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float v = ssq[mt][h];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if (tid == 0) ssq_part[warp][mt * 16 + h * 8 + g] = v;
        }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
        *reinterpret_cast<float4 *>(&partial[((warp * MT + mt) * 32 + lane) * 4]) =
            make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]);
    __syncthreads();
    const int t = threadIdx.x;
    if (t >= MT * 128) return;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kStepWarps; ++w) v += partial[w * MT * 128 + t];
    const int mt = t >> 7, ln = (t & 127) >> 2, i = t & 3;
    const int r = mt * 16 + (i >> 1) * 8 + (ln >> 2);
    const int c = n0 + 2 * (ln & 3) + (i & 1);
    if (r >= M) return;
    float ss = 0.f;
#pragma unroll
    for (int w = 0; w < kStepWarps; ++w) ss += ssq_part[w][r];
    v *= 1.0f / sqrtf(ss / (float)K + eps);
    if (c >= E) {
        z[(int64_t)r * E + (c - E)] = __float2bfloat16_rn(v);
        return;
    }
    // conv step on the bf16-rounded in_proj output, as the unfused path sees it
    const float xc = __bfloat162float(__float2bfloat16_rn(v));
    __nv_bfloat16 *st = conv_state + (int64_t)r * 3 * E + c;
    const float x0 = __bfloat162float(st[0]), x1 = __bfloat162float(st[E]), x2 = __bfloat162float(st[2 * E]);
    float wt[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int src = j - (4 - Kc);
        wt[j] = src >= 0 ? cw[(int64_t)c * Kc + src] : 0.f;
    }
    float cv = cb ? cb[c] : 0.f;
    cv += wt[0] * x0;
    cv += wt[1] * x1;
    cv += wt[2] * x2;
    cv += wt[3] * xc;
    u[(int64_t)r * E + c] = __float2bfloat16_rn(silu_acc(cv));
    st[0] = __float2bfloat16_rn(x1);
    st[E] = __float2bfloat16_rn(x2);
    st[2 * E] = __float2bfloat16_rn(xc);
}

struct StepLayout {
    size_t xz, u, dbc, y, total;
    int64_t W;
};

static StepLayout plan(const hx_mamba_step_args *a) {
    const size_t es = dtype_size(a->io_dtype);
    const size_t Bn = (size_t)a->batch, E = (size_t)a->d_inner;
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    StepLayout l;
    l.W = a->dt_rank + 2 * a->d_state;
    size_t off = 0;
    l.xz = off; off += up(Bn * 2 * E * es);
    l.u = off; off += up(Bn * E * es);
    l.dbc = off; off += up(Bn * l.W * es);
    l.y = off; off += up(Bn * E * es);
    l.total = off + 256;
    return l;
}

static hx_status validate(const hx_mamba_step_args *a) {
    HX_REQUIRE(a != nullptr, HX_ERR_INVALID_INPUT, "args is NULL");
    HX_REQUIRE(a->io_dtype == HX_F32 || a->io_dtype == HX_BF16, HX_ERR_DTYPE_MISMATCH, "io_dtype %d unsupported", a->io_dtype);
    HX_REQUIRE(a->batch >= 0 && a->d_model >= 1 && a->d_inner >= 1 && a->dt_rank >= 1, HX_ERR_INVALID_DIMENSION,
               "bad dimensions (batch %d, d_model %d, d_inner %d, dt_rank %d)", a->batch, a->d_model, a->d_inner, a->dt_rank);
    HX_REQUIRE(a->d_state >= 1 && a->d_state <= 256, HX_ERR_INVALID_DIMENSION, "d_state %d outside [1, 256]", a->d_state);
    HX_REQUIRE(a->d_conv >= 1 && a->d_conv <= 4, HX_ERR_INVALID_DIMENSION, "d_conv %d outside [1, 4]", a->d_conv);
    return HX_OK;
}

}  // namespace decode
}  // namespace hx

extern "C" {

hx_status hx_conv_state_from_prefill(const void *x, int64_t xb, int64_t xr, void *conv_state, int32_t batch,
                                     int32_t seq_len, int32_t d_inner, int32_t io_dtype, void *stream) {
    using namespace hx::decode;
    HX_REQUIRE(batch >= 0 && seq_len >= 0 && d_inner >= 0, HX_ERR_INVALID_DIMENSION, "negative dimension");
    HX_REQUIRE(io_dtype == HX_F32 || io_dtype == HX_BF16, HX_ERR_DTYPE_MISMATCH, "io_dtype %d unsupported", io_dtype);
    if (batch == 0 || d_inner == 0) return HX_OK;
    HX_REQUIRE(x && conv_state, HX_ERR_INVALID_INPUT, "x and conv_state must not be NULL");
    const int64_t n = (int64_t)batch * 3 * d_inner;
    dim3 grid((unsigned)((n + 255) / 256)), block(256);
    cudaStream_t st = (cudaStream_t)stream;
    if (io_dtype == HX_BF16)
        conv_state_kernel<<<grid, block, 0, st>>>(static_cast<const __nv_bfloat16 *>(x), xb, xr,
                                                  static_cast<__nv_bfloat16 *>(conv_state), batch, seq_len, d_inner);
    else
        conv_state_kernel<<<grid, block, 0, st>>>(static_cast<const float *>(x), xb, xr, static_cast<float *>(conv_state),
                                                  batch, seq_len, d_inner);
    return hx::check_launch("conv_state_kernel");
}

hx_status hx_mamba_step_workspace_bytes(const hx_mamba_step_args *a, size_t *bytes) {
    HX_REQUIRE(bytes != nullptr, HX_ERR_INVALID_INPUT, "bytes is NULL");
    hx_status s = hx::decode::validate(a);
    if (s != HX_OK) return s;
    *bytes = hx::decode::plan(a).total;
    return HX_OK;
}

hx_status hx_mamba_block_step(const hx_mamba_step_args *a, void *stream) {
    using namespace hx::decode;
    hx_status s = validate(a);
    if (s != HX_OK) return s;
    if (a->batch == 0) return HX_OK;
    const bool res = a->residual != nullptr;
    HX_REQUIRE(!res || a->norm_w, HX_ERR_INVALID_INPUT, "the residual form needs norm_w");
    HX_REQUIRE((res || (a->x && a->out)) && a->W_in && a->W_x && a->W_dt && a->W_out && a->conv_w && a->b_dt && a->A &&
                   a->Dskip && a->h && a->conv_state,
               HX_ERR_INVALID_INPUT, "a required step operand is NULL");
    const StepLayout l = plan(a);
    HX_REQUIRE(a->workspace && a->workspace_bytes >= l.total, HX_ERR_INVALID_INPUT,
               "hx_mamba_block_step needs a workspace of %zu bytes (got %zu)", l.total, a->workspace_bytes);
    char *ws = reinterpret_cast<char *>((reinterpret_cast<uintptr_t>(a->workspace) + 255) & ~uintptr_t(255));
    const int Bn = a->batch, E = a->d_inner, M = a->d_model, N = a->d_state, R = a->dt_rank, W = (int)l.W;
    void *xz = ws + l.xz, *u = ws + l.u, *dbc = ws + l.dbc, *y = ws + l.y;
    const bool bf = a->io_dtype == HX_BF16;
    cudaStream_t st = (cudaStream_t)stream;

    auto gemm = [&](const void *A, int64_t lda, const void *Wt, int64_t ldw, void *C, int64_t ldc, int m, int n,
                    int k) -> hx_status {
        if (bf && k % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 &&
            (reinterpret_cast<uintptr_t>(Wt) & 15) == 0)
            return hx_gemm_bf16(A, lda, Wt, ldw, nullptr, C, ldc, HX_BF16, m, n, k, 0, stream);
        return hx_gemm_simt(A, lda, Wt, ldw, nullptr, C, ldc, a->io_dtype, a->io_dtype, m, n, k, 0, stream);
    };

    const int64_t pts = (int64_t)Bn * E;
    // residual form on the tensor-core path: norm + in_proj + conv step in one kernel, u and z dense [B, E]
    const bool fused = res && bf && M % 32 == 0 && Bn <= 64 && (2 * E) % 8 == 0 &&
                       (reinterpret_cast<uintptr_t>(a->W_in) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->residual) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(a->norm_w) & 15) == 0;
    const void *x_in = a->x;
    const __nv_bfloat16 *z_bf = static_cast<const __nv_bfloat16 *>(xz) + E;
    int64_t z_stride = 2 * E;
    if (fused) {
        auto zp = static_cast<__nv_bfloat16 *>(xz);  // the xz area holds z [B, E] here
        const dim3 grid((unsigned)(2 * E / 8)), block(kStepWarps * 32);
#define HX_INPROJ_STEP(MT)                                                                                          \
        inproj_step_kernel<MT><<<grid, block, 0, st>>>(a->residual, a->norm_w, a->norm_eps,                         \
                                                       static_cast<const __nv_bfloat16 *>(a->W_in),                 \
                                                       static_cast<__nv_bfloat16 *>(a->conv_state), a->conv_w,      \
                                                       a->conv_b, static_cast<__nv_bfloat16 *>(u), zp, Bn, M, E, a->d_conv)
        if (Bn <= 16) HX_INPROJ_STEP(1);
        else if (Bn <= 32) HX_INPROJ_STEP(2);
        else HX_INPROJ_STEP(4);
#undef HX_INPROJ_STEP
        if ((s = hx::check_launch("inproj_step_kernel")) != HX_OK) return s;
        z_bf = zp;
        z_stride = E;
    } else if (res) {
        // generic residual form: x = rmsnorm(residual) * norm_w into the y area (free until the state step)
        HX_REQUIRE(a->out != nullptr, HX_ERR_INVALID_INPUT, "this path needs `out` as scratch for the residual update");
        if ((s = hx_rmsnorm_fwd(nullptr, a->io_dtype, a->residual, a->norm_w, y, a->io_dtype, Bn, M, a->norm_eps, stream)) != HX_OK)
            return s;
        x_in = y;
    }
    if (!fused && (s = gemm(x_in, M, a->W_in, M, xz, 2 * E, Bn, 2 * E, M)) != HX_OK) return s;
    if (fused) {
        // u and the window are done
    } else if (bf)
        conv_step_kernel<<<(unsigned)((pts + 255) / 256), 256, 0, st>>>(
            static_cast<const __nv_bfloat16 *>(xz), (int64_t)2 * E, static_cast<__nv_bfloat16 *>(a->conv_state), a->conv_w,
            a->conv_b, static_cast<__nv_bfloat16 *>(u), Bn, E, a->d_conv);
    else
        conv_step_kernel<<<(unsigned)((pts + 255) / 256), 256, 0, st>>>(
            static_cast<const float *>(xz), (int64_t)2 * E, static_cast<float *>(a->conv_state), a->conv_w, a->conv_b,
            static_cast<float *>(u), Bn, E, a->d_conv);
    if (!fused && (s = hx::check_launch("conv_step_kernel")) != HX_OK) return s;
    if ((s = gemm(u, E, a->W_x, E, dbc, W, Bn, W, E)) != HX_OK) return s;
    const bool step16 = bf && N == 16 && R % 8 == 0 && R <= 64 && E % 128 == 0 && Bn <= 65535 &&
                        (reinterpret_cast<uintptr_t>(a->W_dt) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->h) & 15) == 0 &&
                        (reinterpret_cast<uintptr_t>(a->A) & 15) == 0;
    if (step16)
        ssm_step16_kernel<<<dim3(E / 128, Bn), 128, 0, st>>>(
            static_cast<const __nv_bfloat16 *>(u), z_bf, z_stride, static_cast<const __nv_bfloat16 *>(dbc), W,
            static_cast<const __nv_bfloat16 *>(a->W_dt), a->b_dt, a->A, a->Dskip, a->h, static_cast<__nv_bfloat16 *>(y), E, R);
    else if (bf)
        ssm_step_kernel<<<(unsigned)((pts + 127) / 128), 128, 0, st>>>(
            static_cast<const __nv_bfloat16 *>(u), z_bf, z_stride,
            static_cast<const __nv_bfloat16 *>(dbc), W, static_cast<const __nv_bfloat16 *>(a->W_dt), a->b_dt, a->A, a->Dskip,
            a->h, static_cast<__nv_bfloat16 *>(y), Bn, E, N, R);
    else
        ssm_step_kernel<<<(unsigned)((pts + 127) / 128), 128, 0, st>>>(
            static_cast<const float *>(u), static_cast<const float *>(xz) + E, (int64_t)2 * E, static_cast<const float *>(dbc),
            W, static_cast<const float *>(a->W_dt), a->b_dt, a->A, a->Dskip, a->h, static_cast<float *>(y), Bn, E, N, R);
    if ((s = hx::check_launch("ssm_step_kernel")) != HX_OK) return s;
    if (!res) return gemm(y, E, a->W_out, E, a->out, M, Bn, M, E);
    const bool tc_out = bf && E % 8 == 0 && (reinterpret_cast<uintptr_t>(a->W_out) & 15) == 0;
    if (tc_out) return hx_gemm_bf16_acc(y, E, a->W_out, E, a->residual, M, Bn, M, E, stream);
    HX_REQUIRE(a->out != nullptr, HX_ERR_INVALID_INPUT, "this path needs `out` as scratch for the residual update");
    if ((s = gemm(y, E, a->W_out, E, a->out, M, Bn, M, E)) != HX_OK) return s;
    return hx::residual_add(a->residual, a->out, a->io_dtype, (int64_t)Bn * M, st);
}

}  // extern "C"
