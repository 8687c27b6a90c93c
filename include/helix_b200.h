/*
 * helix_b200.h -- C ABI of the B200 (sm_100a) state-space hot path.
 *
 * This is the seam a Rust `extern "C"` block in crates/backend-cuda binds.  The reference
 * has no usable FFI for this path: its build script compiles kernels.cu into a static
 * library of C++-mangled __global__ functions with no host launchers
 * (crates/backend-cuda/build.rs:26-52), `execute_ssm_kernel` returns Ok(()) without doing
 * anything (crates/backend-cuda/src/cuda_backend.rs:238-247) and `SsmKernel::execute_forward`
 * copies its input to its output (crates/backend-cuda/src/cuda_kernels.rs:169-180).  Each
 * entry point below names the reference interface it stands in for.
 *
 * Conventions
 *  - Plain pointers and sizes only.  Device pointers unless a name says `host`.
 *  - The caller owns every buffer (inputs, outputs, workspaces); the library keeps no
 *    pointer after a call returns.  Compute entry points never allocate device memory.
 *  - `stream` is a cudaStream_t passed as void* (NULL = default stream).  Launches are
 *    asynchronous with respect to the host and ordered on that stream.
 *  - Every entry point returns an hx_status whose values map one to one onto the
 *    reference's TensorError variants (crates/tensor-core/src/error.rs:7-37); bad input is
 *    reported, never trapped.  hx_last_error() gives the calling thread's last message.
 *  - All entry points are re-entrant and thread-safe: the kernel-level ones keep no state between calls, and a
 *    module handle serialises the calls threads make on it with a lock.  The byte LM keeps its activation buffers
 *    and its decode state inside the module, so all serving calls on ONE handle must be queued on one stream
 *    (stream order keeps a later call from overwriting what an earlier one still reads); use one handle per stream.
 *  - Strides are in ELEMENTS of the tensor's dtype.  The innermost (channel) stride is 1.
 */
#ifndef HELIX_B200_H
#define HELIX_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define HX_API __attribute__((visibility("default")))
#else
#define HX_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* crates/tensor-core/src/error.rs:7-37, same order. */
typedef enum hx_status {
    HX_OK = 0,
    HX_ERR_SHAPE_MISMATCH = 1,
    HX_ERR_INVALID_DIMENSION = 2,
    HX_ERR_DEVICE_MISMATCH = 3,
    HX_ERR_DTYPE_MISMATCH = 4,
    HX_ERR_UNSUPPORTED_OPERATION = 5,
    HX_ERR_ALLOCATION_FAILED = 6,
    HX_ERR_BACKEND = 7,
    HX_ERR_SERIALIZATION = 8,
    HX_ERR_INVALID_CHECKPOINT = 9,
    HX_ERR_INVALID_INPUT = 10
} hx_status;

/* Storage types.  The reference's DType has no bf16 (crates/tensor-core/src/dtype.rs:8-37);
 * HX_BF16 is the addition the device tensor type needs. */
typedef enum hx_dtype { HX_F32 = 0, HX_BF16 = 1, HX_U8 = 2 } hx_dtype;

/* Kernel selection for hx_selective_scan_fwd. */
typedef enum hx_scan_variant {
    HX_SCAN_AUTO = 0,     /* pick the fastest kernel that supports the arguments */
    HX_SCAN_SIMPLE = 1,   /* one thread per (batch, channel); any d_state <= 256; the parity baseline */
    HX_SCAN_TILED = 2,    /* state split over lanes, shared-memory staged tiles; d_state == 16 */
    HX_SCAN_SEQSPLIT = 3, /* HX_SCAN_TILED with the sequence split over CTAs and carries passed
                             through `workspace` by a bounded look-back */
    HX_SCAN_DIRECT = 4,   /* one lane per channel (all 16 states in its registers), 1 or 2 channels per lane,
                             no traffic between lanes; d_state == 16; best when batch * d_inner is large */
    HX_SCAN_LOOKBACK = 5  /* HX_SCAN_DIRECT with the sequence cut into seq_splits segments that run at the SAME time
                             (for few chains: small batch * d_inner, long sequences).  Two launches: every segment
                             but the last first computes its aggregate from a zero state (end state and sum of dt,
                             no outputs), then every segment folds the aggregates of its predecessors into its start
                             state (the look-back) and scans with outputs.  Needs a_geometric = 1, d_state == 16 and
                             `workspace`; no flag or wait between CTAs */
} hx_scan_variant;

HX_API const char *hx_version(void);
/* Message of the last failing call made by this thread ("" if none). */
HX_API const char *hx_last_error(void);
HX_API const char *hx_status_name(hx_status s);

/* ---- device memory (stands in for CudaBackend::allocate / deallocate / copy_to / copy_from,
 *      which store tensors in a host HashMap, crates/backend-cuda/src/cuda_backend.rs:26,449-520) */
HX_API hx_status hx_device_count(int *count);
HX_API hx_status hx_set_device(int device);
HX_API hx_status hx_alloc(void **dptr, size_t bytes);
HX_API hx_status hx_free(void *dptr);
HX_API hx_status hx_host_alloc(void **hptr, size_t bytes);   /* pinned host memory */
HX_API hx_status hx_host_free(void *hptr);
HX_API hx_status hx_memcpy_h2d(void *dst, const void *src_host, size_t bytes, void *stream);
HX_API hx_status hx_memcpy_d2h(void *dst_host, const void *src, size_t bytes, void *stream);
HX_API hx_status hx_memset(void *dptr, int value, size_t bytes, void *stream);
HX_API hx_status hx_stream_synchronize(void *stream);

/* ---- fused selective scan (the centrepiece).
 * Stands in for nn::ssm::MambaBlock::{conv1d, selective_ssm} (crates/nn/src/ssm.rs:467-483),
 * the SSMOp::{Conv1d, Discretize, SelectiveScan} names (crates/tensor-core/src/ops.rs:148-153)
 * and CudaBackend::execute_ssm_kernel (crates/backend-cuda/src/cuda_backend.rs:238-247).
 *
 *   c[b,t,d]  = conv_b[d] + sum_j conv_w[d,j] * x[b, t-(K-1)+j, d]     (conv_w != NULL)
 *   u         = c / (1 + exp(-c))                                       (u = x when conv_w == NULL)
 *   dt        = softplus(dt_raw + dt_bias)  (softplus(v) = v for v > 20; plain sum if dt_softplus == 0)
 *   h_t[n]    = exp(dt * A[d,n]) * h_{t-1}[n] + (dt * u) * Bm[b,t,n],   h_{-1} = 0
 *   y[b,t,d]  = (sum_n Cm[b,t,n] * h_t[n] + Dskip[d] * u) * silu(z[b,t,d])
 * State and all arithmetic are fp32 whatever io_dtype is. */
typedef struct hx_scan_args {
    int32_t batch, seq_len, d_inner, d_state;
    int32_t d_conv;           /* taps K of the causal depthwise conv (1..4); ignored when conv_w == NULL */
    int32_t io_dtype;         /* hx_dtype of x, dt, z, Bm, Cm, y: HX_F32 or HX_BF16 */
    int32_t dt_softplus;      /* 1: dt = softplus(dt_raw + dt_bias) */
    int32_t variant;          /* hx_scan_variant */
    const void *x;            /* [batch, seq_len, d_inner] */
    const void *dt;           /* [batch, seq_len, d_inner] raw (pre-softplus) step sizes */
    const void *z;            /* [batch, seq_len, d_inner] gate input, or NULL */
    const void *Bm;           /* [batch, seq_len, d_state] */
    const void *Cm;           /* [batch, seq_len, d_state] */
    void *y;                  /* [batch, seq_len, d_inner] */
    int64_t x_batch_stride, x_row_stride;
    int64_t dt_batch_stride, dt_row_stride;
    int64_t z_batch_stride, z_row_stride;
    int64_t B_batch_stride, B_row_stride;
    int64_t C_batch_stride, C_row_stride;
    int64_t y_batch_stride, y_row_stride;
    const float *A;           /* [d_inner, d_state] fp32, A = -exp(A_log) */
    const float *Dskip;       /* [d_inner] fp32 or NULL */
    const float *conv_w;      /* [d_inner, d_conv] fp32 or NULL */
    const float *conv_b;      /* [d_inner] fp32 or NULL */
    const float *dt_bias;     /* [d_inner] fp32 or NULL */
    float *h_last;            /* [batch, d_inner, d_state] fp32 final state, or NULL */
    void *workspace;          /* split sequences only: hx_selective_scan_workspace_bytes() bytes */
    size_t workspace_bytes;
    int32_t seq_splits;       /* > 1: cut the sequence into this many segments that run as separate CTAs (needs
                                 `workspace`).  HX_SCAN_TILED / DIRECT: in order, each starting from its
                                 predecessor's final state, which evens out the load when batch * d_inner / tile
                                 is not a multiple of the SM slots.  HX_SCAN_LOOKBACK: at the same time.
                                 HX_SCAN_AUTO: chained when chains are plentiful, look-back when they are few and
                                 A is geometric.  HX_SCAN_SEQSPLIT / LOOKBACK: 0 = four segments */
    int32_t a_geometric;      /* 1: the caller asserts A[d][n] == (n+1) * A[d][0] (checked once with
                                 hx_scan_check_geometric); then exp(dt*A[d][n]) is evaluated as a power of
                                 exp(dt*A[d][0]), one exp per point instead of d_state */
    int32_t lanes_per_channel;/* HX_SCAN_TILED / SEQSPLIT: lanes that share one channel's 16 states
                                 (1, 2 or 4; 0 = choose from the problem size) */
    int32_t reserved;         /* tuning selector, 0 = default.  HX_SCAN_DIRECT: channels per lane (1 or 2) */
    /* Optional fused dt projection (bf16 I/O, HX_SCAN_DIRECT / HX_SCAN_LOOKBACK, or HX_SCAN_AUTO when it picks one
     * of them): when W_dt != NULL the raw step sizes are computed inside the kernel as
     *   dt_raw[b,t,d] = sum_r dt_low[b,t,r] * W_dt[d,r]      (fp32 accumulation on the tensor cores: tcgen05.mma into
     *                                                          tensor memory with one channel per lane in the block's
     *                                                          configuration, mma.sync otherwise)
     * and `dt` is ignored.  dt_low is [batch, seq_len, dt_rank] with its own strides (a column slice of the
     * x_proj output), W_dt is [d_inner, dt_rank] row-major like nn::Linear; dt_rank <= 64 and a multiple of 8.
     * Other kernels report HX_ERR_UNSUPPORTED_OPERATION for it. */
    const void *dt_low;
    const void *W_dt;
    int64_t dt_low_batch_stride, dt_low_row_stride;
    int32_t dt_rank;
    int32_t z_is_gate;        /* 1: `z` already holds the gate silu(z) (the block's in_proj writes it that way with
                                 hx_gemm_bf16_cols), so the scan multiplies by it instead of activating it */
} hx_scan_args;

HX_API hx_status hx_selective_scan_fwd(const hx_scan_args *args, void *stream);
/* Bytes of `workspace` a split scan of these dimensions needs (HX_SCAN_SEQSPLIT, HX_SCAN_LOOKBACK, or any variant
 * with seq_splits > 1; 0 otherwise).  One size serves the chained and the look-back form. */
HX_API hx_status hx_selective_scan_workspace_bytes(const hx_scan_args *args, size_t *bytes);
/* Number of sequence segments (a power of two, 1 = do not split) HX_SCAN_AUTO works best with for these dimensions
 * on the current device: chained segments that even out the load when chains are plentiful, parallel segments
 * (look-back form, needs args->a_geometric) when they are few.  Pass it as args->seq_splits with a workspace. */
HX_API int32_t hx_selective_scan_suggest_splits(const hx_scan_args *args);
/* The same operation on HOST activations: x, dt, z, Bm, Cm are read from (preferably pinned) host memory
 * with the strides given in args, staged into `dev_workspace` (caller-owned device memory of
 * hx_selective_scan_host_workspace_bytes() bytes), scanned, and y is copied back to the host pointer
 * args->y.  A, Dskip, conv_w, conv_b, dt_bias and h_last remain device pointers (they are parameters,
 * resident on the device).  Copies and the kernel are queued on `stream`; synchronise it before reading y.
 * This is the call a host-tensor backend (the reference's CudaBackend keeps tensors in host memory,
 * crates/backend-cuda/src/cuda_backend.rs:26) makes per forward. */
HX_API hx_status hx_selective_scan_host(const hx_scan_args *args, void *dev_workspace, size_t dev_workspace_bytes,
                                 void *stream);
HX_API hx_status hx_selective_scan_host_workspace_bytes(const hx_scan_args *args, size_t *bytes);
/* ---- the sequence-split scan without any allocation.  (No counterpart in the reference: its CUDA backend
 * never reaches a kernel.)
 * Some callers cannot provide the carry workspace HX_SCAN_SEQSPLIT asks for, because they must not call
 * cudaMalloc at that point: a backend that handed every byte of device memory to its own pool at start-up
 * and whose `Module::forward(&self, &T)` receives no allocator, or a serving thread that must stay out of
 * the CUDA allocator's lock while requests are in flight.  For them this entry point runs the same kernel
 * as hx_selective_scan_fwd(variant = HX_SCAN_SEQSPLIT) with the carries kept in an array that is part of the
 * library's device image (HX_SCAN_NOALLOC_SCRATCH_BYTES; each GPU that loads the library holds it until the
 * process exits).  args->variant, args->workspace and args->workspace_bytes are ignored; inputs and outputs
 * are the caller's as usual.  It calls no cudaMalloc / cudaFree and no allocating library routine.
 *  - Limit: the carries need 68 * (segments - 1) * batch * d_inner bytes plus flags; a problem that needs more
 *    than HX_SCAN_NOALLOC_SCRATCH_BYTES is refused with HX_ERR_INVALID_INPUT and a message giving both sizes.
 *  - The first call on a device looks up the array's device address (once per device, that device must be
 *    current); make that first call before starting any stream capture.
 *  - All calls on a device share the one array.  The flags are cleared at the start of every call, so a call
 *    never sees the previous call's contents, but two calls that overlap on the GPU (different streams) race
 *    on it: keep calls to this entry point ordered on one stream per device. */
#define HX_SCAN_NOALLOC_SCRATCH_BYTES (8u << 20)
HX_API hx_status hx_selective_scan_fwd_noalloc(const hx_scan_args *args, void *stream);
/* Synchronous helper, meant for weight-load time: *is_geometric = 1 when every row of A [d_inner, d_state]
 * satisfies A[d][n] == (n+1) * A[d][0] to fp32 rounding (true for the S4D-real initialisation
 * A_log[d][n] = log(n+1)).  Copies A to the host. */
HX_API hx_status hx_scan_check_geometric(const float *A, int32_t d_inner, int32_t d_state, int32_t *is_geometric);
/* Device-side wait failures (a bounded wait on a barrier or a flag that ran out) are recorded in a
 * per-device status word instead of trapping.  Synchronises the device, returns the word (0 = none) and
 * clears it when `clear` is non-zero.  A non-zero word means the outputs of the launches since the last
 * clear are not valid; map it to TensorError::BackendError. */
HX_API hx_status hx_device_status(int32_t *status, int32_t clear);
/* The same as a Result: synchronises, clears the word, and returns HX_ERR_BACKEND (TensorError::BackendError) with
 * a message naming the waits that ran out when it was non-zero, HX_OK otherwise. */
HX_API hx_status hx_device_check(void);
/* Test aid for the path above (no counterpart in the reference): launches the chained two-segment direct scan for
 * `args` (d_state 16, seq_splits 2, workspace given) WITHOUT its first segment and with the carry wait limited to
 * `polls` polls of 40 ns, so that segment 1's wait for a flag nobody publishes runs out after polls * 40 ns: the
 * kernel records the event in the status word, scans on from a zero state and returns normally.  y is not valid
 * afterwards; hx_device_check() reports the event.  The default limit (2^22 polls) is restored on `stream`. */
HX_API hx_status hx_debug_scan_orphan_segment(const hx_scan_args *args, int32_t polls, void *stream);

/* ---- the one exchange of the multi-GPU path: all-gather of a channel-sharded y over NVLink.
 * The wide scan shards d_inner over the GPUs of one node (one process per GPU; B and C replicated; no collective
 * inside the scan).  Afterwards every rank PUSHES its y[:, :, col0 : col0 + d_shard] into the full
 * [batch, seq_len, d_full] buffer of every rank, its own included, with plain 16-byte stores through peer-mapped
 * pointers: one kernel per rank, nothing is loaded from a peer, the result has the [B, L, D] layout directly.
 * The reference has no distributed code (no counterpart); an NCCL all-gather would concatenate on the outermost
 * axis instead.
 *   hx_ipc_export / hx_ipc_open / hx_ipc_close: CUDA IPC plumbing for one process per GPU.  Export the base
 *   pointer of an hx_alloc allocation into a 64-byte handle, send the handle to the peers by any host channel,
 *   open it there (maps the allocation and enables peer access), close it before the owner frees it.
 *   hx_allgather_y_push: queues this rank's push of batch rows [row_begin, row_end) on `stream` (so a caller can
 *   scan rows in groups and push a finished group on a second stream under the scan of the next).  dst[g] is rank
 *   g's full buffer as mapped in THIS process (dst[rank] is the local one).  Widths and col0 must be multiples of
 *   16 bytes.  The buffers are complete everywhere once every rank has synchronised its stream and the ranks have
 *   met at a host barrier. */
#define HX_MAX_PEERS 8
#define HX_IPC_HANDLE_BYTES 64
typedef struct hx_gather_args {
    int32_t world, rank;
    int32_t batch, seq_len, d_shard, d_full;
    int32_t col0;             /* first channel of this rank's shard in the full tensor */
    int32_t io_dtype;
    const void *y_local;      /* [batch, seq_len, d_shard] dense */
    void *dst[HX_MAX_PEERS];  /* [batch, seq_len, d_full] dense, one per rank */
    int32_t row_begin, row_end;
    int32_t max_ctas_per_sm;  /* 0 = 4: the kernel is bound by the link and may share the GPU with a scan */
    int32_t reserved;
} hx_gather_args;
HX_API hx_status hx_ipc_export(const void *dptr, void *handle64);
HX_API hx_status hx_ipc_open(const void *handle64, void **dptr);
HX_API hx_status hx_ipc_close(void *dptr);
HX_API hx_status hx_allgather_y_push(const hx_gather_args *args, void *stream);

/* Measures, on the current device, how many results per second one arithmetic pipe retires: fp32
 * fused multiply-adds (scalar, or the packed two-wide form, counted per lane) or special-function
 * ex2.approx results.  The scan is bound by these pipes rather than by HBM, so the benchmark reports it
 * against max(bytes / bandwidth, exps / ex2 rate, fp32 operations / fma rate) with the rates measured here.
 * Synchronous; `scratch` is device memory of at least 8 * 256 * 4 bytes per SM (results nobody reads).
 * No counterpart in the reference. */
typedef enum hx_probe_kind { HX_PROBE_FMA = 0, HX_PROBE_FMA2 = 1, HX_PROBE_EX2 = 2 } hx_probe_kind;
HX_API hx_status hx_probe_pipe(int32_t kind, void *scratch, size_t scratch_bytes, double *per_second, void *stream);

/* ---- causal depthwise conv + SiLU alone: u = silu(conv(x)).  In the full block the x_proj GEMM
 *      consumes u before the scan can run.  Stands in for nn::ssm::MambaBlock::conv1d
 *      (crates/nn/src/ssm.rs:467-471, `input.clone()` in the reference). */
HX_API hx_status hx_conv1d_silu_fwd(const void *x, int64_t x_batch_stride, int64_t x_row_stride,
                             const float *conv_w, const float *conv_b, void *u,
                             int64_t u_batch_stride, int64_t u_row_stride, int32_t batch,
                             int32_t seq_len, int32_t d_inner, int32_t d_conv, int32_t io_dtype,
                             void *stream);

/* The conv + SiLU above and the x_proj product that follows it in a Mamba block, in one kernel (bf16):
 *   u = silu(conv(x)) [batch, seq_len, d_inner];  x_dbl[b*seq_len + t, 0:n_out] = u[b,t,:] . W_x^T, W_x [n_out, d_inner]
 * (nn::ssm::MambaBlock::conv1d + silu + x_proj, crates/nn/src/ssm.rs:467-471 and the x_proj Linear of forward_mamba).
 * The tile of u the conv produces in shared memory is the tensor core's A operand, so u is written once for the scan
 * and not read back.  Takes bf16, d_conv 4, d_inner a multiple of 64, n_out a multiple of 8 up to 256, conv_w / conv_b
 * / x_dbl 16-byte aligned, x_dbl_row_stride (elements) a multiple of 8, x / u / W_x meeting the TMA rules (16-byte
 * aligned bases and row strides); anything else returns HX_ERR_UNSUPPORTED_OPERATION and the caller runs
 * hx_conv1d_silu_fwd and hx_gemm_bf16.  u equals hx_conv1d_silu_fwd's bit for bit. */
HX_API hx_status hx_conv1d_silu_xproj_fwd(const void *x, int64_t x_batch_stride, int64_t x_row_stride,
                                   const float *conv_w, const float *conv_b, const void *W_x, int64_t ldw,
                                   void *u, int64_t u_batch_stride, int64_t u_row_stride, void *x_dbl,
                                   int64_t x_dbl_row_stride, int32_t batch, int32_t seq_len, int32_t d_inner,
                                   int32_t d_conv, int32_t n_out, int32_t io_dtype, void *stream);

/* ---- diagonal S4 recurrence, one (abar, bbar, C) triple per (channel, state):
 *   h_t = exp(delta[d] A[d,n]) h_{t-1} + delta[d] Bp[d,n] u[b,t,d];  y = sum_n Cp[d,n] h_t[n] + Dskip[d] u.
 * Stands in for nn::ssm::S4Block::forward_ssm + discretize (crates/nn/src/ssm.rs:103-186) in the
 * per-channel form of the benchmark configuration.  u, y: [batch, seq_len, d_model], dense. */
HX_API hx_status hx_s4_diag_fwd(const void *u, const float *A, const float *Bp, const float *Cp,
                         const float *delta, const float *Dskip, void *y, int32_t batch,
                         int32_t seq_len, int32_t d_model, int32_t d_state, int32_t io_dtype,
                         void *stream);

/* ---- the reference-literal S4 recurrence (crates/nn/src/ssm.rs:138-186): one shared state vector
 * of d_state entries driven by all d_model inputs.
 *   a = exp(dt A_real) cos(dt A_imag);  state_t = a state_{t-1} + (dt Bm) u_t;  y_t = Cm state_t + Dv u_t
 * u is [d_model, seq_len] fp32 (the layout forward_ssm requires, ssm.rs:142-147); y is the time-major
 * buffer [seq_len, d_model] the reference's stack() produces (crates/backend-cpu/src/lib.rs:281-296).
 * workspace: hx_s4_ref_workspace_bytes(seq_len, d_state) bytes of device memory. */
HX_API hx_status hx_s4_ref_forward_ssm(const float *u, const float *A_real, const float *A_imag,
                                const float *Bm, const float *Cm, const float *Dv, float dt,
                                float *y, int32_t d_model, int32_t seq_len, int32_t d_state,
                                void *workspace, size_t workspace_bytes, void *stream);
HX_API size_t hx_s4_ref_workspace_bytes(int32_t seq_len, int32_t d_state);

/* ---- the reference-literal nn::ssm::MambaBlock::forward_mamba (crates/nn/src/ssm.rs:435-464): the conv is the
 * identity (:467-471), B and C are computed and dropped (:447-449), selective_ssm is the S4 recurrence on delta
 * (:474-483), and the result is scaled by the gate broadcast along rows (:458-459):
 *   delta = x . delta_proj           [M, M] . [M, M]   (x must be square: forward_ssm wants dim0 == d_model)
 *   y     = S4.forward_ssm(delta)    buffer [M, M] time-major, dt = 0.1
 *   out[i][j] = y[i][j] * gate[j]
 * All operands fp32.  workspace: hx_mamba_ssm_ref_workspace_bytes(d_model, d_state) bytes of device memory. */
HX_API hx_status hx_mamba_ssm_ref_forward(const float *x, const float *delta_proj, const float *gate, const float *A_real,
                                   const float *A_imag, const float *Bm, const float *Cm, const float *Dv, float *out,
                                   int32_t d_model, int32_t d_state, void *workspace, size_t workspace_bytes,
                                   void *stream);
HX_API size_t hx_mamba_ssm_ref_workspace_bytes(int32_t d_model, int32_t d_state);

/* ---- dense projections: C[M,N] = A[M,K] . W[N,K]^T (+ bias[N]), bf16 operands, fp32 accumulation
 *      in tensor memory (tcgen05), C written as bf16 or fp32.  Stands in for nn::Linear::forward
 *      (crates/nn/src/lib.rs:120-134) and the orphan cuBLAS sgemm call
 *      (crates/backend-cuda/src/ops_impl.rs:222-236).
 *      lda / ldw / ldc are row strides in elements; K, lda, ldw must be multiples of 8 and the
 *      base pointers 16-byte aligned (TMA rules).  epilogue: 0 none, 1 SiLU, 2 softplus.
 *      With M <= 64 and K a multiple of 32 (a decode step) the work goes to a kernel that streams W through
 *      N/8 CTAs (16 warps each, K split between them) with warp-level tensor-core instructions instead of one
 *      128-row tcgen05 tile. */
HX_API hx_status hx_gemm_bf16(const void *A, int64_t lda, const void *W, int64_t ldw, const float *bias,
                       void *C, int64_t ldc, int32_t c_dtype, int32_t M, int32_t N, int32_t K,
                       int32_t epilogue, void *stream);
/* Same, with the activation applied only to the columns n >= epilogue_first_col (a multiple of 32): the block's
 * in_proj writes [x | silu(z)] in one pass, so that the scan multiplies by the gate instead of computing it.
 * epilogue 3 = SiLU with the hardware's approximate exp2 / reciprocal (bf16 outputs). */
HX_API hx_status hx_gemm_bf16_cols(const void *A, int64_t lda, const void *W, int64_t ldw, const float *bias,
                            void *C, int64_t ldc, int32_t c_dtype, int32_t M, int32_t N, int32_t K,
                            int32_t epilogue, int32_t epilogue_first_col, void *stream);
/* C[M,N] += A[M,K] . W[N,K]^T with an fp32 C: the epilogue adds its tile into C through the memory system (TMA
 * reduce), so a block's out_proj can accumulate straight into the fp32 residual stream. */
HX_API hx_status hx_gemm_bf16_acc(const void *A, int64_t lda, const void *W, int64_t ldw, float *C, int64_t ldc,
                           int32_t M, int32_t N, int32_t K, void *stream);
/* Tile form of the tcgen05 kernel for wide shapes (N > 128, at least 512 rows, TMA-storable C, epilogue none or the
 * accumulating one).  CTA pairs: two CTAs of a thread-block cluster share a [256 x 256] tile, each loads its 128 rows
 * of A and HALF of the W tile, the leader issues tcgen05.mma.cta_group::2.  mode 0: one CTA per [128 x 256] tile
 * always; 1 (the build's default): pairs where they measured faster (the accumulating epilogue on at least four
 * waves of pair tiles); 2: pairs wherever the shape allows; a negative mode changes nothing.  *pairs (may be NULL)
 * receives how many pairs the current device can hold at once (0: the pair kernel cannot be used there and single
 * CTAs run whatever the mode).  Process-wide; HX_GEMM_PAIR in the environment sets the initial mode.  Results are
 * bit-identical in every mode (each element is one k-ascending tensor-memory sum).  No counterpart in the reference. */
HX_API hx_status hx_gemm_pair_mode(int32_t mode, int32_t *pairs);
/* Same contract on CUDA cores in fp32 (any alignment, fp32 or bf16 operands): the small-shape and
 * fp32 path (the reference is fp32 throughout). */
HX_API hx_status hx_gemm_simt(const void *A, int64_t lda, const void *W, int64_t ldw, const float *bias,
                       void *C, int64_t ldc, int32_t ab_dtype, int32_t c_dtype, int32_t M,
                       int32_t N, int32_t K, int32_t epilogue, void *stream);

/* ---- RMSNorm over the last axis with optional fused residual add.  The residual stream is fp32:
 *   if (residual) { residual += x (x may be NULL: nothing added); src = residual } else src = x
 *   y = src / sqrt(mean(src^2) + eps) * w
 * Stands in for nn::RMSNorm::forward (crates/nn/src/lib.rs:258-285). */
HX_API hx_status hx_rmsnorm_fwd(const void *x, int32_t x_dtype, float *residual, const float *w, void *y,
                         int32_t y_dtype, int64_t rows, int32_t d, float eps, void *stream);

/* ---- byte embedding gather: out[i, :] = emb[tokens[i], :]
 *      (examples/ssm_byte_lm feeds byte ids to its model, examples/ssm_byte_lm/src/main.rs:104-130). */
HX_API hx_status hx_embedding_fwd(const uint8_t *tokens, const void *emb, int32_t emb_dtype, void *out,
                           int32_t out_dtype, int64_t n_tokens, int32_t d_model, void *stream);

/* ---- elementwise helpers the exported reference block needs (crates/nn/src/lib.rs:888-906):
 *      y = silu(x)  (TensorActivation::silu, crates/backend-cpu/src/lib.rs:1154-1170). */
HX_API hx_status hx_silu_fwd(const void *x, void *y, int64_t n, int32_t io_dtype, void *stream);

/* ---- one whole Mamba block forward on device buffers (in_proj -> conv+SiLU -> x_proj -> dt_proj ->
 *      fused scan -> out_proj).  Stands in for MambaBlock::forward (crates/nn/src/lib.rs:910,
 *      crates/nn/src/ssm.rs:436).  Weights are row-major [out, in] like nn::Linear.
 *      io_dtype HX_BF16: weights and activations bf16, tensor-core GEMMs.
 *      io_dtype HX_F32 : everything fp32, CUDA-core GEMMs. */
typedef struct hx_mamba_block_args {
    int32_t batch, seq_len, d_model, d_inner, d_state, d_conv, dt_rank;
    int32_t io_dtype;
    const void *x;            /* [batch*seq_len, d_model] */
    void *out;                /* [batch*seq_len, d_model] */
    const void *W_in;         /* [2*d_inner, d_model] */
    const void *W_x;          /* [dt_rank + 2*d_state, d_inner] */
    const void *W_dt;         /* [d_inner, dt_rank] */
    const void *W_out;        /* [d_model, d_inner] */
    const float *conv_w;      /* [d_inner, d_conv] */
    const float *conv_b;      /* [d_inner] or NULL */
    const float *b_dt;        /* [d_inner] */
    const float *A;           /* [d_inner, d_state] */
    const float *Dskip;       /* [d_inner] */
    void *workspace;          /* hx_mamba_block_workspace_bytes() bytes */
    size_t workspace_bytes;
    int32_t scan_variant;     /* hx_scan_variant */
    int32_t a_geometric;      /* as hx_scan_args.a_geometric */
    void **stage_events;      /* NULL, or 7 cudaEvent_t: recorded on `stream` before each of the six stages
                                 (in_proj, conv, x_proj, dt_proj, scan, out_proj) and after the last one; a stage
                                 that is done inside its neighbour's kernel shows as the gap between two marks */
    float *h_last;            /* NULL, or [batch, d_inner, d_state] fp32: the scan's state after the last step */
    void *conv_state;         /* NULL, or [batch, 3, d_inner] io dtype: the conv inputs of the last three steps
                                 (oldest first, zeros where seq_len < 3); with h_last, what hx_mamba_block_step
                                 continues from */
    float *residual;          /* NULL, or the fp32 residual stream [batch*seq_len, d_model]: the block's output is
                                 added into it (by the out_proj epilogue where the tensor-core GEMM runs) and
                                 `out` is not written, unless the fp32 path needs it as scratch */
} hx_mamba_block_args;

HX_API hx_status hx_mamba_block_fwd(const hx_mamba_block_args *args, void *stream);
HX_API hx_status hx_mamba_block_workspace_bytes(const hx_mamba_block_args *args, size_t *bytes);
/* Kernel launches one hx_mamba_block_fwd call with these arguments makes: 6 (in_proj, conv, x_proj, dt_proj,
 * scan, out_proj); one less where conv and x_proj run as one kernel (hx_conv1d_silu_xproj_fwd's conditions), one less
 * where the dt projection is computed inside the scan kernel (bf16, d_state 16, dt_rank a multiple of 8 up to 64, a
 * scan that runs one lane per channel), one more where the scan is the look-back form (two passes): 4 on the
 * benchmark's 32 x 2048 x 768 bf16 block. */
HX_API hx_status hx_mamba_block_kernel_launches(const hx_mamba_block_args *args, int32_t *launches);

/* ---- single-token decode step of the block: the recurrent form of hx_mamba_block_fwd, continuing from
 *      the state a prefill (or an earlier step) left.  x and out are [batch, d_model]; `h` and `conv_state`
 *      are updated in place.  Five launches: in_proj, conv step, x_proj, state step (dt projection, softplus,
 *      h <- exp(dt A) h + dt B u, y = C.h + D u, gate), out_proj.  The reference has no decode path
 *      (its MambaBlock::forward always takes a whole sequence, crates/nn/src/lib.rs:888-906); this is the
 *      step that follows prefill in serving. */
typedef struct hx_mamba_step_args {
    int32_t batch, d_model, d_inner, d_state, d_conv, dt_rank;
    int32_t io_dtype, reserved;
    const void *x;            /* [batch, d_model] */
    void *out;                /* [batch, d_model] */
    const void *W_in, *W_x, *W_dt, *W_out;   /* as hx_mamba_block_args */
    const float *conv_w, *conv_b, *b_dt, *A, *Dskip;
    float *h;                 /* [batch, d_inner, d_state] fp32, in/out */
    void *conv_state;         /* [batch, 3, d_inner] io dtype, in/out */
    void *workspace;          /* hx_mamba_step_workspace_bytes() bytes */
    size_t workspace_bytes;
    /* Residual form (all three or none): the block input is rmsnorm(residual) * norm_w instead of `x`, and the
     * block output is added into `residual` instead of written to `out` (`x` and `out` may then be NULL).  With
     * bf16 weights and d_model a multiple of 32 the norm and the conv step run inside the in_proj kernel and the
     * add inside out_proj: four launches per step instead of six with the norm counted. */
    float *residual;          /* [batch, d_model] fp32, in/out */
    const float *norm_w;      /* [d_model] */
    float norm_eps;
    int32_t reserved2;
} hx_mamba_step_args;
HX_API hx_status hx_mamba_block_step(const hx_mamba_step_args *args, void *stream);
HX_API hx_status hx_mamba_step_workspace_bytes(const hx_mamba_step_args *args, size_t *bytes);
/* The conv window a decode step starts from, taken from the conv input x [batch, seq_len, d_inner]
 * (element strides) of a prefill: conv_state[b][j] = x[b][seq_len-3+j], zeros for negative steps. */
HX_API hx_status hx_conv_state_from_prefill(const void *x, int64_t x_batch_stride, int64_t x_row_stride, void *conv_state,
                                     int32_t batch, int32_t seq_len, int32_t d_inner, int32_t io_dtype, void *stream);

/* =============================================================================================
 * Module-level API: opaque handles over the C++ host layer (helixml_b200/csrc/helix_host.hpp), which
 * restates the reference's module interface for device-resident tensors:
 *   MambaBlock::new(d_model, d_state, d_conv, expand, &device) / forward   crates/nn/src/lib.rs:847,910
 *   S4Block::new(d_model, d_state, &device) / forward_ssm                  crates/nn/src/ssm.rs:39,138
 *   Linear::new / RMSNorm::new / Module::{forward, parameters, parameters_mut}  crates/nn/src/lib.rs:20-39,67,242
 * A Rust `impl Module<DeviceTensor>` forwards to these.  Handles are owned by the caller and freed with
 * hx_tensor_free / hx_module_free.  forward() runs on the default stream of the module's device and
 * returns a new tensor; errors come back as hx_status exactly like the reference's Result<T, TensorError>.
 * ============================================================================================= */
typedef struct hx_tensor hx_tensor;
typedef struct hx_module hx_module;

/* Seed of the parameter initialisers (the reference draws from an unseeded thread_rng,
 * crates/backend-cpu/src/lib.rs:1209). */
HX_API void hx_manual_seed(uint64_t seed);

/* Tensor::from host data (fp32 values, converted to `dtype`), TensorRandom::zeros-style construction is
 * from_host with zeros.  dims has ndim entries (<= 8). */
HX_API hx_status hx_tensor_from_host(const float *data, const int64_t *dims, int32_t ndim, int32_t dtype,
                              int32_t device_id, hx_tensor **out);
HX_API hx_status hx_tensor_from_host_u8(const uint8_t *data, const int64_t *dims, int32_t ndim, int32_t device_id,
                                 hx_tensor **out);
HX_API hx_status hx_tensor_to_host(const hx_tensor *t, float *out, int64_t n);       /* widens bf16 to fp32 */
HX_API hx_status hx_tensor_copy_from_host(hx_tensor *t, const float *data, int64_t n);
HX_API hx_status hx_tensor_info(const hx_tensor *t, int32_t *ndim, int64_t *dims8, int32_t *dtype, int32_t *device_id);
HX_API void *hx_tensor_data(const hx_tensor *t);                                      /* device pointer */
HX_API void hx_tensor_free(hx_tensor *t);

/* ---- tensor primitives on device tensors: what `impl TensorOps / TensorBroadcast / TensorActivation /
 *      TensorRandom / TensorMixedPrecision for DeviceTensor` forwards to, so that the reference's generic blocks
 *      (T: Tensor + TensorOps + TensorRandom + TensorBroadcast + TensorMixedPrecision, crates/nn/src/lib.rs:846,
 *      crates/nn/src/ssm.rs:37) compile and run with the device tensor as T.  Semantics are the CPU tensor's
 *      (crates/backend-cpu/src/lib.rs): every call returns a NEW tensor on the input's device (default stream);
 *      F32 and BF16 storage, arithmetic in fp32.  Utility kernels, not the hot path. */
/* TensorOps::{add, sub, mul, div, max, min, gt} (tensor.rs:64-73,106-109,127; lib.rs:570-632,852-899,951-975):
 * identical shapes or HX_ERR_SHAPE_MISMATCH; gt gives 1.0 / 0.0. */
typedef enum hx_binary_op {
    HX_OP_ADD = 0, HX_OP_SUB = 1, HX_OP_MUL = 2, HX_OP_DIV = 3, HX_OP_MAX = 4, HX_OP_MIN = 5, HX_OP_GT = 6
} hx_binary_op;
HX_API hx_status hx_tensor_binary(int32_t op, const hx_tensor *a, const hx_tensor *b, hx_tensor **out);
/* TensorOps::{sqrt, exp, log, sin, cos, tan, abs, sign, neg, pow(p0), clamp(p0, p1), add_scalar(p0),
 * mul_scalar(p0), gt_scalar(p0)} (tensor.rs:79-130; lib.rs:759-949) and TensorActivation::{relu, gelu, silu,
 * sigmoid, tanh, leaky_relu(p0)} (tensor.rs:191-209; lib.rs:1100-1198).  sign is f32::signum (+-1 also for +-0),
 * gelu the tanh form, silu x / (1 + exp(-x)). */
typedef enum hx_unary_op {
    HX_OP_SQRT = 16, HX_OP_EXP = 17, HX_OP_LOG = 18, HX_OP_SIN = 19, HX_OP_COS = 20, HX_OP_TAN = 21, HX_OP_ABS = 22,
    HX_OP_SIGN = 23, HX_OP_NEG = 24, HX_OP_RELU = 25, HX_OP_GELU = 26, HX_OP_SILU = 27, HX_OP_SIGMOID = 28,
    HX_OP_TANH = 29, HX_OP_POW = 30, HX_OP_CLAMP = 31, HX_OP_ADD_SCALAR = 32, HX_OP_MUL_SCALAR = 33,
    HX_OP_GT_SCALAR = 34, HX_OP_LEAKY_RELU = 35
} hx_unary_op;
HX_API hx_status hx_tensor_unary(int32_t op, const hx_tensor *a, float p0, float p1, hx_tensor **out);
/* TensorOps::matmul (tensor.rs:76; lib.rs:634-757): [M,K].[K,N], [K].[K,N] or [M,K].[K]; the sum runs over k
 * ascending in one fp32 accumulator with the product and the sum rounded separately, as the reference's loop does,
 * so fp32 results are bit-identical to it.  Other ranks: HX_ERR_UNSUPPORTED_OPERATION. */
HX_API hx_status hx_tensor_matmul(const hx_tensor *a, const hx_tensor *b, hx_tensor **out);
/* The same product on raw device pointers, queued on `stream`: C[M,N] = A[M,K] . B[K,N], row-major, dense. */
HX_API hx_status hx_matmul_ref(const void *A, const void *B, void *C, int32_t M, int32_t N, int32_t K, int32_t dtype,
                        void *stream);
/* Tensor::{transpose, slice, cat, stack, reshape, clone} (tensor.rs:34-46; lib.rs:94-335).  slice is 2-D only and
 * cat 1-D only, like the reference.  stack of 1- to 3-D tensors lays the operands one after the other whatever
 * `dim` is and puts the new axis at `dim` in the shape only (lib.rs:281-296: S4Block::forward_ssm relies on it). */
HX_API hx_status hx_tensor_transpose(const hx_tensor *a, int64_t dim0, int64_t dim1, hx_tensor **out);
HX_API hx_status hx_tensor_slice(const hx_tensor *a, const int64_t *start, const int64_t *end, int32_t n, hx_tensor **out);
HX_API hx_status hx_tensor_cat(const hx_tensor *const *tensors, int32_t count, int64_t dim, hx_tensor **out);
HX_API hx_status hx_tensor_stack(const hx_tensor *const *tensors, int32_t count, int64_t dim, hx_tensor **out);
HX_API hx_status hx_tensor_reshape(const hx_tensor *a, const int64_t *dims, int32_t ndim, hx_tensor **out);
HX_API hx_status hx_tensor_clone(const hx_tensor *a, hx_tensor **out);
/* TensorBroadcast::{broadcast_to, expand} (tensor.rs:139-142; lib.rs:1352-1518): trailing axes aligned, axes of
 * size 1 repeated; from 1 to 2, 2 to 3 and 1 to 3 dimensions in the reference's cases, equal ranks axis by axis.
 * unsqueeze / squeeze are hx_tensor_reshape. */
HX_API hx_status hx_tensor_broadcast_to(const hx_tensor *a, const int64_t *dims, int32_t ndim, hx_tensor **out);
/* TensorMixedPrecision::cast / Tensor::to_dtype (tensor.rs:52,238): F32 <-> BF16, round to nearest even.  The device
 * tensor has no other storage type: F16, F64, I8, I32, Bool give HX_ERR_UNSUPPORTED_OPERATION (the reference keeps
 * f32 storage under every label, lib.rs:350-361, so nothing on the path depends on them). */
HX_API hx_status hx_tensor_cast(const hx_tensor *a, int32_t dtype, hx_tensor **out);
/* TensorOps::to_scalar (tensor.rs:133): a one-element tensor, else HX_ERR_INVALID_INPUT.  Synchronises. */
HX_API hx_status hx_tensor_to_scalar(const hx_tensor *a, float *value);
/* TensorOps::from_scalar, TensorRandom::{zeros, ones} = hx_tensor_full; TensorRandom::{eye, arange}
 * (tensor.rs:118,223-232; lib.rs:901-911,1272-1349): arange adds `step` in fp32 while the value is below `end`. */
HX_API hx_status hx_tensor_full(float value, const int64_t *dims, int32_t ndim, int32_t dtype, int32_t device_id,
                         hx_tensor **out);
HX_API hx_status hx_tensor_eye(int64_t n, int32_t dtype, int32_t device_id, hx_tensor **out);
HX_API hx_status hx_tensor_arange(float start, float end, float step, int32_t dtype, int32_t device_id, hx_tensor **out);
/* TensorRandom::{random_normal(mean p0, std p1), random_uniform(min p0, max p1), random_bernoulli(p p0)}
 * (tensor.rs:214-220; lib.rs:1203-1270): F32, drawn from the stream hx_manual_seed seeds. */
typedef enum hx_random_kind { HX_RANDOM_NORMAL = 0, HX_RANDOM_UNIFORM = 1, HX_RANDOM_BERNOULLI = 2 } hx_random_kind;
HX_API hx_status hx_tensor_random(int32_t kind, const int64_t *dims, int32_t ndim, float p0, float p1, int32_t device_id,
                           hx_tensor **out);

HX_API hx_status hx_mamba_block_new(int64_t d_model, int64_t d_state, int64_t d_conv, int64_t expand, int32_t dtype,
                             int32_t device_id, hx_module **out);
HX_API hx_status hx_s4_block_new(int64_t d_model, int64_t d_state, int32_t device_id, hx_module **out);
HX_API hx_status hx_linear_new(int64_t in_features, int64_t out_features, int32_t bias, int32_t dtype,
                        int32_t device_id, hx_module **out);
HX_API hx_status hx_rmsnorm_new(int64_t d_model, float eps, int32_t device_id, hx_module **out);
/* nn::Sequential (crates/nn/src/lib.rs:577-661): Sequential::new(&device), add(module), len(); forward chains the
 * modules, parameters concatenates theirs.  hx_sequential_add takes ownership: the child handle is consumed (do not
 * use or free it afterwards), like the reference's Box<dyn Module>. */
HX_API hx_status hx_sequential_new(int32_t device_id, hx_module **out);
HX_API hx_status hx_sequential_add(hx_module *seq, hx_module *child);
HX_API int32_t hx_sequential_len(const hx_module *seq);
/* The byte-level LM of examples/ssm_byte_lm widened to n_layer x (RMSNorm + MambaBlock + residual), tied
 * embedding [256, d_model] (examples/ssm_byte_lm/src/main.rs:104-130). */
HX_API hx_status hx_byte_lm_new(int64_t n_layer, int64_t d_model, int64_t d_state, int64_t d_conv, int64_t expand,
                         int32_t dtype, int32_t device_id, hx_module **out);

/* Module::forward.  MambaBlock / Linear / RMSNorm / S4Block take [L, d] or [B, L, d]; ByteLM takes U8
 * tokens [B, L] and returns logits [B, L, 256]. */
HX_API hx_status hx_module_forward(const hx_module *m, const hx_tensor *input, hx_tensor **out);
/* nn::ssm::S4Block::forward_ssm: input [d_model, L] fp32, output buffer [L, d_model]. */
HX_API hx_status hx_s4_block_forward_ssm(const hx_module *m, const hx_tensor *input, hx_tensor **out);
/* Serving calls of the byte LM: no allocation after the first call for a given (batch, seq_len); work is
 * queued on `stream`.  _host: tokens from and logits to (pinned) host memory, logits in the model dtype.
 * _device: tokens_dev [B*L] u8 and logits_dev [B*L, 256] on the device. */
HX_API hx_status hx_byte_lm_forward_host(hx_module *m, const uint8_t *tokens_host, void *logits_host, int64_t batch,
                                  int64_t seq_len, void *stream);
HX_API hx_status hx_byte_lm_forward_device(hx_module *m, const uint8_t *tokens_dev, void *logits_dev, int64_t batch,
                                    int64_t seq_len, void *stream);
/* From the second call with the same (tokens pointer, logits pointer, batch, seq_len) on, the three forward calls
 * above and the prefill below replay a CUDA graph of the whole forward (one launch instead of 150 to 200 dependent
 * kernels: what a batch of a few sequences per GPU is bound by).  hx_byte_lm_forward_graph(m, 0) keeps plain
 * launches; a stream that is itself being captured, and the per-stage profile, always get plain launches. */
HX_API hx_status hx_byte_lm_forward_graph(hx_module *m, int32_t enable);
/* Serving with state: hx_byte_lm_prefill_device is hx_byte_lm_forward_device that also keeps, per layer, the
 * scan's final state and the conv window; hx_byte_lm_decode_step_device then advances every sequence of that
 * batch by one token: tokens_dev [batch] u8 in, logits_dev [batch, 256] (model dtype) out, state updated in the
 * module.  The first step after a prefill runs as plain launches, the second is captured into a CUDA graph over
 * the module's own step buffers and every later step replays it (1 + 4 per layer + 2 kernels in one launch on
 * the bf16 path: the norm and the conv step run inside in_proj, the residual add inside out_proj);
 * hx_byte_lm_decode_graph(m, 0) keeps plain launches.  The state belongs to the module: one decoding stream per
 * module.  The reference's example has no decode loop (examples/ssm_byte_lm/src/main.rs:423-444 are placeholders). */
HX_API hx_status hx_byte_lm_prefill_device(hx_module *m, const uint8_t *tokens_dev, void *logits_dev, int64_t batch,
                                    int64_t seq_len, void *stream);
HX_API hx_status hx_byte_lm_decode_step_device(hx_module *m, const uint8_t *tokens_dev, void *logits_dev, int64_t batch,
                                        void *stream);
HX_API hx_status hx_byte_lm_decode_graph(hx_module *m, int32_t enable);
HX_API int64_t hx_byte_lm_launches_per_decode_step(const hx_module *m);
/* Kernel launches of one forward at the shape of the most recent serving call (before any call: of a
 * forward whose blocks do not fuse the dt projection). */
HX_API int64_t hx_byte_lm_launches_per_forward(const hx_module *m);
/* Per-stage timing of the byte LM with CUDA events on the launching stream.  enable = 1 makes the following
 * forward calls record events around every stage; hx_byte_lm_profile_read synchronises, adds the elapsed
 * times of all forwards since the last read (0 embedding, 1 norm, 2 in_proj, 3 conv, 4 x_proj, 5 dt_proj,
 * 6 scan, 7 out_proj, 8 tied head into ms9[9]) and resets. */
HX_API hx_status hx_byte_lm_profile(hx_module *m, int32_t enable);
HX_API hx_status hx_byte_lm_profile_read(hx_module *m, float *ms9, int32_t *forwards);

/* Module::parameters / parameters_mut: parameter `index` as a tensor handle that SHARES the parameter's
 * storage (write it with hx_tensor_copy_from_host, then call hx_module_parameters_updated). */
HX_API int32_t hx_module_num_parameters(const hx_module *m);
HX_API hx_status hx_module_parameter(hx_module *m, int32_t index, hx_tensor **out);
HX_API hx_status hx_module_parameters_updated(hx_module *m);
HX_API const char *hx_module_name(const hx_module *m);
HX_API void hx_module_free(hx_module *m);

/* ---- checkpoints in the reference's on-disk layout (crates/training/src/checkpoint.rs:136-197): a u32
 *      big-endian length, the CheckpointData JSON, then bincode of Vec<CpuTensor> (f32 storage, row-major).
 *      hx_module_save_checkpoint is CheckpointableModule::checkpoint + save_checkpoint_to_file (parameters in
 *      parameters() order, bf16 widened to f32); hx_module_load_checkpoint is load_checkpoint_from_file +
 *      CheckpointableModule::restore (crates/nn/src/lib.rs:42-56): a different parameter count gives
 *      HX_ERR_INVALID_CHECKPOINT, a different shape HX_ERR_SHAPE_MISMATCH, a malformed file
 *      HX_ERR_SERIALIZATION, and the module is unchanged.  The hx_checkpoint_* calls work on host arrays only
 *      (no GPU needed): the same file format for callers that hold their tensors on the host. */
typedef struct hx_checkpoint_meta {
    uint64_t epoch, step;
    double training_loss, validation_loss, learning_rate;
    uint64_t timestamp_secs;  /* seconds since the Unix epoch */
} hx_checkpoint_meta;
typedef struct hx_checkpoint hx_checkpoint;
HX_API hx_status hx_module_save_checkpoint(const hx_module *m, const char *path, const hx_checkpoint_meta *meta);
HX_API hx_status hx_module_load_checkpoint(hx_module *m, const char *path, hx_checkpoint_meta *meta_out);
HX_API hx_status hx_checkpoint_write(const char *path, const hx_checkpoint_meta *meta, int32_t n_tensors,
                              const float *const *data, const int64_t *const *dims, const int32_t *ndims);
HX_API hx_status hx_checkpoint_open(const char *path, hx_checkpoint **out);
HX_API int32_t hx_checkpoint_num_tensors(const hx_checkpoint *ck);
HX_API hx_status hx_checkpoint_meta_get(const hx_checkpoint *ck, hx_checkpoint_meta *meta);
/* data and dims point into the checkpoint object and stay valid until hx_checkpoint_close */
HX_API hx_status hx_checkpoint_tensor(const hx_checkpoint *ck, int32_t index, const float **data, const int64_t **dims,
                               int32_t *ndim);
HX_API void hx_checkpoint_close(hx_checkpoint *ck);

#ifdef __cplusplus
}
#endif
#endif /* HELIX_B200_H */
