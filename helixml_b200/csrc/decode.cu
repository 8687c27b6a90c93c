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
    HX_REQUIRE(a->x && a->out && a->W_in && a->W_x && a->W_dt && a->W_out && a->conv_w && a->b_dt && a->A && a->Dskip &&
                   a->h && a->conv_state,
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

    if ((s = gemm(a->x, M, a->W_in, M, xz, 2 * E, Bn, 2 * E, M)) != HX_OK) return s;
    const int64_t pts = (int64_t)Bn * E;
    if (bf)
        conv_step_kernel<<<(unsigned)((pts + 255) / 256), 256, 0, st>>>(
            static_cast<const __nv_bfloat16 *>(xz), (int64_t)2 * E, static_cast<__nv_bfloat16 *>(a->conv_state), a->conv_w,
            a->conv_b, static_cast<__nv_bfloat16 *>(u), Bn, E, a->d_conv);
    else
        conv_step_kernel<<<(unsigned)((pts + 255) / 256), 256, 0, st>>>(
            static_cast<const float *>(xz), (int64_t)2 * E, static_cast<float *>(a->conv_state), a->conv_w, a->conv_b,
            static_cast<float *>(u), Bn, E, a->d_conv);
    if ((s = hx::check_launch("conv_step_kernel")) != HX_OK) return s;
    if ((s = gemm(u, E, a->W_x, E, dbc, W, Bn, W, E)) != HX_OK) return s;
    if (bf)
        ssm_step_kernel<<<(unsigned)((pts + 127) / 128), 128, 0, st>>>(
            static_cast<const __nv_bfloat16 *>(u), static_cast<const __nv_bfloat16 *>(xz) + E, (int64_t)2 * E,
            static_cast<const __nv_bfloat16 *>(dbc), W, static_cast<const __nv_bfloat16 *>(a->W_dt), a->b_dt, a->A, a->Dskip,
            a->h, static_cast<__nv_bfloat16 *>(y), Bn, E, N, R);
    else
        ssm_step_kernel<<<(unsigned)((pts + 127) / 128), 128, 0, st>>>(
            static_cast<const float *>(u), static_cast<const float *>(xz) + E, (int64_t)2 * E, static_cast<const float *>(dbc),
            W, static_cast<const float *>(a->W_dt), a->b_dt, a->A, a->Dskip, a->h, static_cast<float *>(y), Bn, E, N, R);
    if ((s = hx::check_launch("ssm_step_kernel")) != HX_OK) return s;
    return gemm(y, E, a->W_out, E, a->out, M, Bn, M, E);
}

}  // extern "C"
