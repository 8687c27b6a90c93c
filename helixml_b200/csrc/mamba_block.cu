// One Mamba block forward as a sequence of launches on caller-owned buffers:
//   in_proj GEMM -> causal conv + SiLU -> x_proj GEMM -> dt_proj GEMM -> fused scan
//   (softplus, decay, recurrence, D skip, SiLU(z) gate) -> out_proj GEMM.
// The scan reads u, z, B and C in place: z is the second half of the in_proj output row and B, C
// are column slices of the x_proj output row, all passed as strided views without copies.
#include <cstring>

#include "hx_common.cuh"

// HX_SCAN_AUTO: 0 = dt_proj is a kernel of its own; 1 = the one-pass scan computes the dt projection itself; 2 = the
// look-back form does too.  Measured over the 24 blocks of the byte LM at 32 x 2048 x 1536 (ms): scan with the
// projection inside as tcgen05.mma into tensor memory 10.7; scan 10.1 + dt_proj kernel 1.6; the earlier fused form
// (mma.sync in the producer warp, an fp32 dt tile in shared memory) 12.5-13.2.  At 4 / 8 / 16 rows (look-back form) the
// step is 4.60 / 7.64 / 13.73 ms fused against 4.66 / 7.79 / 14.05.
#ifndef HX_BLOCK_FUSE_DT_AUTO
#define HX_BLOCK_FUSE_DT_AUTO 2
#endif
// 1: conv + SiLU and x_proj as one kernel where its conditions hold; 0: always two kernels.
#ifndef HX_BLOCK_FUSE_CONV_XPROJ
#define HX_BLOCK_FUSE_CONV_XPROJ 1
#endif

namespace hx {
namespace block {

struct Layout {
    size_t xz, u, dbc, dtl, y, scan_ws, scan_ws_bytes, total;
    int64_t W;  // row width of the x_proj output
    int splits; // sequence segments of the scan
};

static hx_scan_args scan_shape(const hx_mamba_block_args *a) {
    hx_scan_args sa;
    memset(&sa, 0, sizeof(sa));
    sa.batch = a->batch; sa.seq_len = a->seq_len; sa.d_inner = a->d_inner; sa.d_state = a->d_state;
    sa.io_dtype = a->io_dtype; sa.variant = a->scan_variant;
    // the block's scan call: u already convolved, gate and softplus present
    sa.a_geometric = a->a_geometric; sa.dt_softplus = 1; sa.z = a->x;  // (z only has to be non-NULL for planning)
    return sa;
}

static Layout plan(const hx_mamba_block_args *a) {
    const size_t es = dtype_size(a->io_dtype);
    const size_t T = (size_t)a->batch * a->seq_len;
    const size_t E = a->d_inner;
    Layout l;
    l.W = a->dt_rank + 2 * a->d_state;
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    size_t off = 0;
    l.xz = off; off += up(T * 2 * E * es);
    l.u = off; off += up(T * E * es);
    l.dbc = off; off += up(T * l.W * es);
    l.dtl = off; off += up(T * E * es);
    l.y = off; off += up(T * E * es);
    // carries of a split scan (the split evens out the load; see hx_selective_scan_suggest_splits)
    hx_scan_args sa = scan_shape(a);
    // variants that chain their segments are planned as such (the parallel-segment suggestion is for the look-back form)
    if (a->scan_variant == HX_SCAN_TILED || a->scan_variant == HX_SCAN_SEQSPLIT || a->scan_variant == HX_SCAN_DIRECT)
        sa.a_geometric = 0;
    l.splits = (a->scan_variant == HX_SCAN_SIMPLE || a->d_state != 16) ? 1 : hx_selective_scan_suggest_splits(&sa);
    sa.seq_splits = l.splits;
    l.scan_ws_bytes = 0;
    if (l.splits > 1) hx_selective_scan_workspace_bytes(&sa, &l.scan_ws_bytes);
    l.scan_ws = off; off += up(l.scan_ws_bytes);
    l.total = off + 256;
    return l;
}

static hx_status validate(const hx_mamba_block_args *a) {
    HX_REQUIRE(a != nullptr, HX_ERR_INVALID_INPUT, "hx_mamba_block_fwd: args is NULL");
    HX_REQUIRE(a->batch >= 0 && a->seq_len >= 0, HX_ERR_INVALID_DIMENSION, "negative batch or seq_len");
    HX_REQUIRE(a->d_model >= 1 && a->d_inner >= 1 && a->d_state >= 1 && a->d_state <= 256 && a->dt_rank >= 1,
               HX_ERR_INVALID_DIMENSION, "bad block dimensions (d_model %d, d_inner %d, d_state %d, dt_rank %d)",
               a->d_model, a->d_inner, a->d_state, a->dt_rank);
    HX_REQUIRE(a->d_conv >= 1 && a->d_conv <= 4, HX_ERR_INVALID_DIMENSION, "d_conv %d outside [1, 4]", a->d_conv);
    HX_REQUIRE(a->io_dtype == HX_F32 || a->io_dtype == HX_BF16, HX_ERR_DTYPE_MISMATCH, "io_dtype %d unsupported",
               a->io_dtype);
    return HX_OK;
}

// True when the dt projection runs inside the scan kernel instead of as a GEMM of its own: bf16, d_state 16,
// a rank the kernel's operand tiles hold, every operand meeting the TMA rules of the scan's tensor maps (rows of
// d_inner and of the x_proj output a multiple of 16 bytes, W_dt 16-byte aligned), and a scan variant that runs the
// one-lane-per-channel kernel (chained or look-back).
static bool fuses_dt(const hx_mamba_block_args *a, int W, int splits) {
    const int R = a->dt_rank;
    if (!(a->io_dtype == HX_BF16 && a->d_state == 16 && R >= 8 && R <= 64 && R % 8 == 0 && W % 8 == 0 &&
          a->d_inner % 8 == 0 && (reinterpret_cast<uintptr_t>(a->W_dt) & 15) == 0))
        return false;
    if (a->scan_variant == HX_SCAN_DIRECT) return true;
    if (a->scan_variant == HX_SCAN_LOOKBACK) return a->a_geometric != 0;
    if (a->scan_variant != HX_SCAN_AUTO) return false;
    hx_scan_args sa = scan_shape(a);
    sa.seq_splits = splits;
    // AUTO fuses where the scan runs one lane per channel (the one-pass kernel below the chain count that switches it
    // to two channels per lane, and the look-back form): there the projection is a tcgen05.mma into tensor memory.
    // With two channels per lane it would be the producer warp's mma.sync through shared memory, which is slower than
    // a dt_proj kernel of its own.
    const hx::scan::ScanKind kind = hx::scan::auto_kind(&sa);
    if (kind == hx::scan::ScanKind::Direct) return HX_BLOCK_FUSE_DT_AUTO >= 1 && hx::scan::auto_channels_per_lane(&sa) == 1;
    if (kind == hx::scan::ScanKind::LookBack) return HX_BLOCK_FUSE_DT_AUTO >= 2 && a->a_geometric != 0;
    return false;
}

// True when conv + SiLU and x_proj run as one kernel (hx_conv1d_silu_xproj_fwd's conditions on the block's buffers;
// the workspace slices are 256-byte aligned).
static bool fuses_conv_xproj(const hx_mamba_block_args *a, int W) {
#if HX_BLOCK_FUSE_CONV_XPROJ
    auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    return a->io_dtype == HX_BF16 && a->d_conv == 4 && a->d_inner % 64 == 0 && W % 8 == 0 && W <= 256 && al16(a->conv_w) &&
           (!a->conv_b || al16(a->conv_b)) && al16(a->W_x);
#else
    (void)a; (void)W;
    return false;
#endif
}

}  // namespace block
}  // namespace hx

extern "C" {

hx_status hx_mamba_block_workspace_bytes(const hx_mamba_block_args *a, size_t *bytes) {
    HX_REQUIRE(bytes != nullptr, HX_ERR_INVALID_INPUT, "bytes is NULL");
    hx_status s = hx::block::validate(a);
    if (s != HX_OK) return s;
    *bytes = hx::block::plan(a).total;
    return HX_OK;
}

hx_status hx_mamba_block_kernel_launches(const hx_mamba_block_args *a, int32_t *launches) {
    HX_REQUIRE(launches != nullptr, HX_ERR_INVALID_INPUT, "launches is NULL");
    hx_status s = hx::block::validate(a);
    if (s != HX_OK) return s;
    // in_proj, conv, x_proj (one kernel with the conv where it can be), dt_proj (unless fused into the scan), scan, out_proj
    if (a->batch == 0 || a->seq_len == 0) {
        *launches = 0;
        return HX_OK;
    }
    const hx::block::Layout l = hx::block::plan(a);
    const bool fused = hx::block::fuses_dt(a, (int)l.W, l.splits);
    // the look-back scan is two launches (aggregate pass, output pass)
    hx_scan_args sa = hx::block::scan_shape(a);
    sa.seq_splits = l.splits;
    const bool lookback = l.splits > 1 && a->d_state == 16 &&
                          (a->scan_variant == HX_SCAN_LOOKBACK ||
                           (a->scan_variant == HX_SCAN_AUTO && hx::scan::auto_kind(&sa) == hx::scan::ScanKind::LookBack));
    *launches = (fused ? 5 : 6) + (lookback ? 1 : 0) - (hx::block::fuses_conv_xproj(a, (int)l.W) ? 1 : 0);
    return HX_OK;
}

hx_status hx_mamba_block_fwd(const hx_mamba_block_args *a, void *stream) {
    using namespace hx::block;
    hx_status s = validate(a);
    if (s != HX_OK) return s;
    if (a->batch == 0 || a->seq_len == 0) return HX_OK;
    HX_REQUIRE(a->x && (a->out || a->residual) && a->W_in && a->W_x && a->W_dt && a->W_out && a->conv_w && a->b_dt && a->A && a->Dskip,
               HX_ERR_INVALID_INPUT, "a required block operand is NULL");
    const Layout l = plan(a);
    HX_REQUIRE(a->workspace && a->workspace_bytes >= l.total, HX_ERR_INVALID_INPUT,
               "hx_mamba_block_fwd needs a workspace of %zu bytes (got %zu)", l.total, a->workspace_bytes);
    char *ws = reinterpret_cast<char *>((reinterpret_cast<uintptr_t>(a->workspace) + 255) & ~uintptr_t(255));
    const size_t es = hx::dtype_size(a->io_dtype);
    const int64_t T = (int64_t)a->batch * a->seq_len;
    HX_REQUIRE(T <= 0x7fffffff, HX_ERR_INVALID_DIMENSION, "batch * seq_len exceeds 2^31");
    const int E = a->d_inner, M = a->d_model, N = a->d_state, R = a->dt_rank, W = (int)l.W;
    void *xz = ws + l.xz, *u = ws + l.u, *dbc = ws + l.dbc, *dtl = ws + l.dtl, *y = ws + l.y;
    const bool bf = a->io_dtype == HX_BF16;

    // bf16: tensor-core GEMM where its alignment rules hold, CUDA-core GEMM otherwise; fp32: CUDA cores
    auto gemm = [&](const void *A, int64_t lda, const void *Wt, int64_t ldw, void *C, int64_t ldc, int m, int n,
                    int k) -> hx_status {
        if (bf && k % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 &&
            (reinterpret_cast<uintptr_t>(Wt) & 15) == 0)
            return hx_gemm_bf16(A, lda, Wt, ldw, nullptr, C, ldc, HX_BF16, m, n, k, 0, stream);
        return hx_gemm_simt(A, lda, Wt, ldw, nullptr, C, ldc, a->io_dtype, a->io_dtype, m, n, k, 0, stream);
    };

    auto mark = [&](int i) {
        if (a->stage_events) cudaEventRecord(static_cast<cudaEvent_t>(a->stage_events[i]), (cudaStream_t)stream);
    };
    mark(0);
    // 1. xz = x W_in^T                                  [T, 2E]
    // The GEMM's epilogue could write [x | silu(z)] (hx_gemm_bf16_cols) so that the scan multiplies by the gate
    // instead of computing it.  Measured at d_model 768, 65 536 tokens: the in_proj GEMM becomes epilogue-bound
    // (5.8 -> 7.1 ms over 24 blocks) and the scan gains nothing, so the block does not do it.
    const bool gate_in_gemm = false;
    if (gate_in_gemm)
        s = hx_gemm_bf16_cols(a->x, M, a->W_in, M, nullptr, xz, 2 * E, HX_BF16, (int)T, 2 * E, M, 3 /* fast SiLU */, E, stream);
    else
        s = gemm(a->x, M, a->W_in, M, xz, 2 * E, (int)T, 2 * E, M);
    if (s != HX_OK) return s;
    if (a->conv_state &&
        (s = hx_conv_state_from_prefill(xz, (int64_t)a->seq_len * 2 * E, 2 * E, a->conv_state, a->batch, a->seq_len, E,
                                        a->io_dtype, stream)) != HX_OK)
        return s;
    mark(1);
    // 2. u = silu(conv(xs)), xs = xz[:, :E]            [T, E]
    // 3. [dt_low | B | C] = u W_x^T                     [T, R + 2N]
    // One kernel does both where it can (the conv's tile of u is the tensor core's A operand, so u is not read
    // back); otherwise the conv kernel and a GEMM.
    bool fused_cx = fuses_conv_xproj(a, W);
    if (fused_cx) {
        s = hx_conv1d_silu_xproj_fwd(xz, (int64_t)a->seq_len * 2 * E, 2 * E, a->conv_w, a->conv_b, a->W_x, E, u,
                                     (int64_t)a->seq_len * E, E, dbc, W, a->batch, a->seq_len, E, a->d_conv, W, a->io_dtype,
                                     stream);
        if (s == HX_ERR_UNSUPPORTED_OPERATION) fused_cx = false;  // an operand the one kernel does not take: two kernels
        else if (s != HX_OK) return s;
        else mark(2);
    }
    if (!fused_cx) {
        if ((s = hx_conv1d_silu_fwd(xz, (int64_t)a->seq_len * 2 * E, 2 * E, a->conv_w, a->conv_b, u, (int64_t)a->seq_len * E,
                                    E, a->batch, a->seq_len, E, a->d_conv, a->io_dtype, stream)) != HX_OK)
            return s;
        mark(2);
        if ((s = gemm(u, E, a->W_x, E, dbc, W, (int)T, W, E)) != HX_OK) return s;
    }
    mark(3);
    // 4. dt_lin = dt_low W_dt^T                          [T, E]   (bias and softplus happen inside the scan)
    // With bf16 operands and enough chains for the one-lane-per-channel scan, the projection is done inside the
    // scan kernel (its producer warp, tensor cores) and this GEMM, its 2*T*E-byte write and read disappear.
    const bool fuse_dt = fuses_dt(a, W, l.splits);
    if (!fuse_dt && (s = gemm(dbc, W, a->W_dt, R, dtl, E, (int)T, E, R)) != HX_OK) return s;
    mark(4);
    // 5. fused scan on strided views
    hx_scan_args sa;
    memset(&sa, 0, sizeof(sa));
    sa.batch = a->batch; sa.seq_len = a->seq_len; sa.d_inner = E; sa.d_state = N; sa.d_conv = a->d_conv;
    sa.io_dtype = a->io_dtype; sa.dt_softplus = 1; sa.variant = a->scan_variant;
    sa.x = u; sa.x_batch_stride = (int64_t)a->seq_len * E; sa.x_row_stride = E;
    sa.dt = dtl; sa.dt_batch_stride = (int64_t)a->seq_len * E; sa.dt_row_stride = E;
    if (fuse_dt) {
        sa.dt = nullptr;
        sa.dt_low = dbc; sa.dt_low_batch_stride = (int64_t)a->seq_len * W; sa.dt_low_row_stride = W;
        sa.W_dt = a->W_dt; sa.dt_rank = R;
    }
    sa.z = static_cast<char *>(xz) + (size_t)E * es; sa.z_batch_stride = (int64_t)a->seq_len * 2 * E; sa.z_row_stride = 2 * E;
    sa.Bm = static_cast<char *>(dbc) + (size_t)R * es; sa.B_batch_stride = (int64_t)a->seq_len * W; sa.B_row_stride = W;
    sa.Cm = static_cast<char *>(dbc) + (size_t)(R + N) * es; sa.C_batch_stride = (int64_t)a->seq_len * W; sa.C_row_stride = W;
    sa.y = y; sa.y_batch_stride = (int64_t)a->seq_len * E; sa.y_row_stride = E;
    sa.A = a->A; sa.Dskip = a->Dskip; sa.dt_bias = a->b_dt;
    sa.h_last = a->h_last;
    sa.z_is_gate = gate_in_gemm ? 1 : 0;
    sa.conv_w = nullptr; sa.conv_b = nullptr;  // u is already activated
    sa.a_geometric = a->a_geometric;
    if (l.splits > 1) {
        sa.seq_splits = l.splits;
        sa.workspace = ws + l.scan_ws;
        sa.workspace_bytes = l.scan_ws_bytes;
    }
    if ((s = hx_selective_scan_fwd(&sa, stream)) != HX_OK) return s;
    mark(5);
    // 6. out = y W_out^T                                 [T, M]
    // With a residual stream the tensor-core GEMM adds its tiles straight into it (fp32, TMA reduce): the bf16
    // block output, its write and the read of it by the next norm disappear.
    if (a->residual) {
        const bool tc_out = bf && E % 8 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 &&
                            (reinterpret_cast<uintptr_t>(a->W_out) & 15) == 0;
        if (tc_out) {
            s = hx_gemm_bf16_acc(y, E, a->W_out, E, a->residual, M, (int)T, M, E, stream);
        } else {
            HX_REQUIRE(a->out != nullptr, HX_ERR_INVALID_INPUT, "this path needs `out` as scratch for the residual update");
            if ((s = gemm(y, E, a->W_out, E, a->out, M, (int)T, M, E)) != HX_OK) return s;
            s = hx::residual_add(a->residual, a->out, a->io_dtype, T * M, (cudaStream_t)stream);
        }
    } else {
        s = gemm(y, E, a->W_out, E, a->out, M, (int)T, M, E);
    }
    mark(6);
    return s;
}

}  // extern "C"
