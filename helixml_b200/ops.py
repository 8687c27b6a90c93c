"""Array-level wrappers: torch CUDA tensors in, torch CUDA tensors out, every op a call through
the C ABI on torch's current stream.  torch is used for device memory and streams only."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return L.HX_F32
    if t.dtype == torch.bfloat16:
        return L.HX_BF16
    if t.dtype == torch.uint8:
        return L.HX_U8
    raise L.HxError(4, f"unsupported dtype {t.dtype}")


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _f32(t):
    if t is None:
        return None
    assert t.dtype == torch.float32 and t.is_contiguous(), "parameter tensors are contiguous fp32"
    return t


def _view3(t: torch.Tensor):
    """(batch_stride, row_stride) in elements of a [B, L, D] view whose last stride is 1."""
    if t.dim() != 3 or t.stride(2) != 1:
        raise L.HxError(1, f"expected a [B, L, D] tensor with unit inner stride, got {tuple(t.shape)} / {t.stride()}")
    return t.stride(0), t.stride(1)


def check_geometric(A: torch.Tensor) -> bool:
    flag = C.c_int32(0)
    L.check(L.lib().hx_scan_check_geometric(_p(_f32(A)), A.shape[0], A.shape[1], C.byref(flag)))
    return bool(flag.value)


def probe_pipe(kind: str) -> float:
    """Results per second of one arithmetic pipe on the current GPU: 'fma' (scalar fp32 fused multiply-adds),
    'fma2' (the packed two-wide form, counted per lane) or 'ex2' (special-function exponentials)."""
    if kind not in ("fma", "fma2", "ex2"):
        raise L.HxError(10, f"unknown probe {kind!r}")
    code = {"fma": 0, "fma2": 1, "ex2": 2}[kind]
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    scratch = torch.empty(sms * 8 * 256, device="cuda", dtype=torch.float32)
    out = C.c_double(0.0)
    L.check(L.lib().hx_probe_pipe(code, _p(scratch), scratch.numel() * 4, C.byref(out), _stream()))
    return out.value


def scan_workspace_bytes(batch, seq_len, d_inner, dtype, seq_splits=0) -> int:
    a = L.ScanArgs()
    a.batch, a.seq_len, a.d_inner, a.d_state = batch, seq_len, d_inner, 16
    a.io_dtype = L.HX_BF16 if dtype == torch.bfloat16 else L.HX_F32
    a.variant = L.SCAN_SEQSPLIT
    a.seq_splits = seq_splits
    n = C.c_size_t(0)
    L.check(L.lib().hx_selective_scan_workspace_bytes(C.byref(a), C.byref(n)))
    return n.value


def suggest_splits(batch, seq_len, d_inner, dtype, a_geometric=True) -> int:
    """hx_selective_scan_suggest_splits: sequence segments HX_SCAN_AUTO works best with for this shape."""
    a = L.ScanArgs()
    a.batch, a.seq_len, a.d_inner, a.d_state = batch, seq_len, d_inner, 16
    a.io_dtype = L.HX_BF16 if dtype == torch.bfloat16 else L.HX_F32
    a.a_geometric = 1 if a_geometric else 0
    return int(L.lib().hx_selective_scan_suggest_splits(C.byref(a)))


def selective_scan(x, dt, A, Bm, Cm, D=None, z=None, conv_w=None, conv_b=None, dt_bias=None, dt_softplus=True,
                   variant=L.SCAN_AUTO, a_geometric=None, lanes_per_channel=0, return_state=False, out=None,
                   workspace=None, seq_splits=0, tune=0, dt_low=None, W_dt=None, z_is_gate=False):
    """Fused selective scan (hx_selective_scan_fwd).  x, dt, z, y: [B, L, D]; Bm, Cm: [B, L, N].
    z_is_gate: z already holds silu(z)."""
    Bsz, Lq, Dm = x.shape
    N = A.shape[1]
    y = out if out is not None else torch.empty((Bsz, Lq, Dm), dtype=x.dtype, device=x.device)
    h = torch.empty((Bsz, Dm, N), dtype=torch.float32, device=x.device) if return_state else None
    a = L.ScanArgs()
    a.batch, a.seq_len, a.d_inner, a.d_state = Bsz, Lq, Dm, N
    a.d_conv = conv_w.shape[1] if conv_w is not None else 0
    a.io_dtype = _dt(x)
    a.dt_softplus = 1 if dt_softplus else 0
    a.variant = variant
    if W_dt is not None:
        # fused dt projection: dt = dt_low @ W_dt.T inside the kernel
        a.dt_low, a.W_dt = dt_low.data_ptr(), W_dt.contiguous().data_ptr()
        a.dt_low_batch_stride, a.dt_low_row_stride = _view3(dt_low)
        a.dt_rank = W_dt.shape[1]
    for name, t in (("x", x), ("dt", dt), ("z", z), ("y", y)):
        if t is None:
            continue
        if t.dtype != x.dtype:
            raise L.HxError(4, f"{name} has dtype {t.dtype}, expected {x.dtype}")
        if tuple(t.shape) != (Bsz, Lq, Dm):
            raise L.HxError(1, f"{name} has shape {tuple(t.shape)}, expected {(Bsz, Lq, Dm)}")
        bs, rs = _view3(t)
        setattr(a, name, t.data_ptr())
        setattr(a, f"{name}_batch_stride", bs)
        setattr(a, f"{name}_row_stride", rs)
    for name, field, t in (("Bm", "B", Bm), ("Cm", "C", Cm)):
        if t.dtype != x.dtype:
            raise L.HxError(4, f"{name} has dtype {t.dtype}, expected {x.dtype}")
        if tuple(t.shape) != (Bsz, Lq, N):
            raise L.HxError(1, f"{name} has shape {tuple(t.shape)}, expected {(Bsz, Lq, N)}")
        bs, rs = _view3(t)
        setattr(a, name, t.data_ptr())
        setattr(a, f"{field}_batch_stride", bs)
        setattr(a, f"{field}_row_stride", rs)
    a.A = _f32(A).data_ptr()
    for name, t in (("Dskip", D), ("conv_w", conv_w), ("conv_b", conv_b), ("dt_bias", dt_bias)):
        if t is not None:
            setattr(a, name, _f32(t).data_ptr())
    if h is not None:
        a.h_last = h.data_ptr()
    if a_geometric is None:
        a_geometric = check_geometric(A)
    a.a_geometric = 1 if a_geometric else 0
    a.lanes_per_channel = lanes_per_channel
    a.seq_splits = seq_splits
    a.reserved = tune
    a.z_is_gate = 1 if z_is_gate else 0
    if variant in (L.SCAN_SEQSPLIT, L.SCAN_LOOKBACK) or seq_splits > 1:
        n = C.c_size_t(0)
        L.check(L.lib().hx_selective_scan_workspace_bytes(C.byref(a), C.byref(n)))
        if workspace is None:
            workspace = torch.empty(max(n.value, 1), dtype=torch.uint8, device=x.device)
        a.workspace = workspace.data_ptr()
        a.workspace_bytes = workspace.numel() * workspace.element_size()
    L.check(L.lib().hx_selective_scan_fwd(C.byref(a), _stream()))
    return (y, h) if return_state else y


def conv1d_silu(x, conv_w, conv_b=None, out=None):
    Bsz, Lq, Dm = x.shape
    u = out if out is not None else torch.empty((Bsz, Lq, Dm), dtype=x.dtype, device=x.device)
    xb, xr = _view3(x)
    ub, ur = _view3(u)
    L.check(L.lib().hx_conv1d_silu_fwd(_p(x), xb, xr, _p(_f32(conv_w)), _p(_f32(conv_b)), _p(u), ub, ur, Bsz, Lq, Dm,
                                       conv_w.shape[1], _dt(x), _stream()))
    return u


def conv1d_silu_xproj(x, conv_w, conv_b, w_x, out_u=None, out_xdbl=None):
    """u = silu(conv(x)) and x_dbl = u @ w_x.T in one kernel (hx_conv1d_silu_xproj_fwd): x [B, L, E] bf16 (a strided
    half of the in_proj output is fine), conv_w [E, 4] fp32, w_x [n_out, E] bf16.  Returns (u, x_dbl [B, L, n_out]);
    raises UnsupportedOperation for shapes the fused kernel does not take."""
    Bsz, Lq, Dm = x.shape
    n_out = w_x.shape[0]
    u = out_u if out_u is not None else torch.empty((Bsz, Lq, Dm), dtype=x.dtype, device=x.device)
    xd = out_xdbl if out_xdbl is not None else torch.empty((Bsz, Lq, n_out), dtype=x.dtype, device=x.device)
    xb, xr = _view3(x)
    ub, ur = _view3(u)
    if not xd.is_contiguous():
        raise L.HxError(1, "x_dbl must be contiguous")
    L.check(L.lib().hx_conv1d_silu_xproj_fwd(_p(x), xb, xr, _p(_f32(conv_w)), _p(_f32(conv_b)), _p(w_x), w_x.stride(0), _p(u), ub,
                                             ur, _p(xd), n_out, Bsz, Lq, Dm, conv_w.shape[1], n_out, _dt(x), _stream()))
    return u, xd


def s4_diag(u, A, Bp, Cp, delta, D=None):
    Bsz, Lq, Dm = u.shape
    u = u.contiguous()
    y = torch.empty_like(u)
    L.check(L.lib().hx_s4_diag_fwd(_p(u), _p(_f32(A)), _p(_f32(Bp)), _p(_f32(Cp)), _p(_f32(delta)), _p(_f32(D)), _p(y),
                                   Bsz, Lq, Dm, A.shape[1], _dt(u), _stream()))
    return y


def s4_ref_forward_ssm(u, A_real, A_imag, Bm, Cm, Dv, dt=0.1):
    """Reference-literal S4 recurrence: u [d_model, L] fp32 -> time-major buffer [L, d_model]."""
    M, Lq = u.shape
    N = A_real.shape[0]
    y = torch.empty((Lq, M), dtype=torch.float32, device=u.device)
    n = L.lib().hx_s4_ref_workspace_bytes(Lq, N)
    ws = torch.empty(max(n, 1), dtype=torch.uint8, device=u.device)
    L.check(L.lib().hx_s4_ref_forward_ssm(_p(_f32(u)), _p(_f32(A_real)), _p(_f32(A_imag)), _p(_f32(Bm)), _p(_f32(Cm)),
                                          _p(_f32(Dv)), C.c_float(dt), _p(y), M, Lq, N, _p(ws), n, _stream()))
    return y


def gemm(a, w, bias=None, out_dtype=None, epilogue=L.EPI_NONE, tensor_cores=None, out=None, epilogue_first_col=0):
    """C = a @ w.T (+ bias) (+ activation).  a [M, K] (row stride arbitrary), w [N, K].
    epilogue_first_col (tensor-core path): the activation applies to columns >= it (a multiple of 32)."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise L.HxError(1, f"a is {tuple(a.shape)} but w is {tuple(w.shape)}")
    assert a.stride(1) == 1 and w.stride(1) == 1
    out_dtype = out_dtype or a.dtype
    c = out if out is not None else torch.empty((M, N), dtype=out_dtype, device=a.device)
    if tensor_cores is None:
        tensor_cores = a.dtype == torch.bfloat16
    if tensor_cores:
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            raise L.HxError(4, "the tensor-core GEMM takes bf16 operands")
        L.check(L.lib().hx_gemm_bf16_cols(_p(a), a.stride(0), _p(w), w.stride(0), _p(_f32(bias)), _p(c), c.stride(0), _dt(c),
                                          M, N, K, epilogue, epilogue_first_col, _stream()))
    else:
        if a.dtype != w.dtype:
            raise L.HxError(4, "a and w must share a dtype")
        L.check(L.lib().hx_gemm_simt(_p(a), a.stride(0), _p(w), w.stride(0), _p(_f32(bias)), _p(c), c.stride(0), _dt(a),
                                     _dt(c), M, N, K, epilogue, _stream()))
    return c


def gemm_pair_mode(mode: int = -1) -> int:
    """Tile form of the wide tensor-core shapes (hx_gemm_pair_mode): 0 single CTAs, 1 CTA pairs where they measured
    faster (the default), 2 pairs wherever the shape allows; a negative mode only asks.  Returns how many CTA pairs
    the current device holds at once (0: pairs unusable there)."""
    n = C.c_int32(0)
    L.check(L.lib().hx_gemm_pair_mode(mode, C.byref(n)))
    return n.value


def gemm_acc(a, w, c):
    """c += a @ w.T (hx_gemm_bf16_acc): a [M, K], w [N, K] bf16, c [M, N] fp32, updated in place."""
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or c.dtype != torch.float32:
        raise L.HxError(4, "gemm_acc takes bf16 operands and an fp32 accumulator")
    if tuple(c.shape) != (M, N) or w.shape[1] != K:
        raise L.HxError(1, f"shapes {tuple(a.shape)}, {tuple(w.shape)}, {tuple(c.shape)} do not fit")
    L.check(L.lib().hx_gemm_bf16_acc(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), c.stride(0), M, N, K,
                                     _stream()))
    return c


def rmsnorm(x, w, eps=1e-5, residual=None, out_dtype=None):
    """y = rmsnorm(residual + x) with residual (fp32) updated in place, or rmsnorm(x) without it."""
    src = x if x is not None else residual
    d = src.shape[-1]
    rows = src.numel() // d
    out_dtype = out_dtype or (x.dtype if x is not None else torch.float32)
    y = torch.empty(src.shape, dtype=out_dtype, device=src.device)
    if x is not None:
        x = x.contiguous()
    L.check(L.lib().hx_rmsnorm_fwd(_p(x), _dt(x) if x is not None else L.HX_F32, _p(residual), _p(_f32(w)), _p(y), _dt(y),
                                   rows, d, C.c_float(eps), _stream()))
    return y


def embedding(tokens, emb, out_dtype=torch.float32):
    n = tokens.numel()
    out = torch.empty((*tokens.shape, emb.shape[1]), dtype=out_dtype, device=emb.device)
    L.check(L.lib().hx_embedding_fwd(_p(tokens.contiguous()), _p(emb.contiguous()), _dt(emb), _p(out), _dt(out), n,
                                     emb.shape[1], _stream()))
    return out


def silu(x):
    x = x.contiguous()
    y = torch.empty_like(x)
    L.check(L.lib().hx_silu_fwd(_p(x), _p(y), x.numel(), _dt(x), _stream()))
    return y


def mamba_block_workspace_bytes(batch, seq_len, d_model, d_inner, d_state, d_conv, dt_rank, dtype) -> int:
    a = L.MambaBlockArgs()
    a.batch, a.seq_len, a.d_model, a.d_inner = batch, seq_len, d_model, d_inner
    a.d_state, a.d_conv, a.dt_rank = d_state, d_conv, dt_rank
    a.io_dtype = L.HX_BF16 if dtype == torch.bfloat16 else L.HX_F32
    n = C.c_size_t(0)
    L.check(L.lib().hx_mamba_block_workspace_bytes(C.byref(a), C.byref(n)))
    return n.value


def mamba_block(x, w: dict, d_state: int, d_conv: int, workspace=None, scan_variant=L.SCAN_AUTO, a_geometric=None,
                out=None, h_last=None, conv_state=None, residual=None):
    """One Mamba block forward (hx_mamba_block_fwd).  x [B, L, M]; w: device tensors W_in, W_x, W_dt,
    W_out in x.dtype and conv_w, conv_b, b_dt, A, D in fp32.  h_last [B, E, N] fp32 and conv_state [B, 3, E]
    (x.dtype), when given, receive the state a decode step continues from."""
    Bsz, Lq, M = x.shape
    x = x.contiguous()
    E = w["W_in"].shape[0] // 2
    R = w["W_dt"].shape[1]
    y = out if out is not None else torch.empty_like(x)
    a = L.MambaBlockArgs()
    a.batch, a.seq_len, a.d_model, a.d_inner = Bsz, Lq, M, E
    a.d_state, a.d_conv, a.dt_rank = d_state, d_conv, R
    a.io_dtype = _dt(x)
    a.x, a.out = x.data_ptr(), y.data_ptr()
    for k in ("W_in", "W_x", "W_dt", "W_out"):
        if w[k].dtype != x.dtype:
            raise L.HxError(4, f"{k} has dtype {w[k].dtype}, expected {x.dtype}")
        setattr(a, k, w[k].contiguous().data_ptr())
    a.conv_w = _f32(w["conv_w"]).data_ptr()
    if w.get("conv_b") is not None:
        a.conv_b = _f32(w["conv_b"]).data_ptr()
    a.b_dt = _f32(w["b_dt"]).data_ptr()
    a.A = _f32(w["A"]).data_ptr()
    a.Dskip = _f32(w["D"]).data_ptr()
    # the scan's plan (and with it the workspace size) depends on the variant and on whether A is geometric
    a.scan_variant = scan_variant
    if a_geometric is None:
        a_geometric = check_geometric(w["A"])
    a.a_geometric = 1 if a_geometric else 0
    n = C.c_size_t(0)
    L.check(L.lib().hx_mamba_block_workspace_bytes(C.byref(a), C.byref(n)))
    if workspace is None:
        workspace = torch.empty(n.value, dtype=torch.uint8, device=x.device)
    a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    if h_last is not None:
        a.h_last = h_last.data_ptr()
    if conv_state is not None:
        a.conv_state = conv_state.data_ptr()
    if residual is not None:  # fp32 [B, L, M]: the block output is added into it
        a.residual = residual.data_ptr()
    L.check(L.lib().hx_mamba_block_fwd(C.byref(a), _stream()))
    return y


def mamba_block_step(x, w: dict, d_state: int, d_conv: int, h, conv_state, workspace=None, out=None, residual=None,
                     norm_w=None, norm_eps=1e-5):
    """One decode step of the block (hx_mamba_block_step): x [B, M]; h [B, E, N] fp32 and conv_state [B, 3, E]
    (x.dtype) are updated in place.  Residual form: residual [B, M] fp32 and norm_w [M] given, x only supplies the
    dtype: the input is rmsnorm(residual) * norm_w and the output is added into residual."""
    Bsz, M = x.shape
    x = x.contiguous()
    E = w["W_in"].shape[0] // 2
    R = w["W_dt"].shape[1]
    y = out if out is not None else torch.empty_like(x)
    a = L.MambaStepArgs()
    a.batch, a.d_model, a.d_inner, a.d_state, a.d_conv, a.dt_rank = Bsz, M, E, d_state, d_conv, R
    a.io_dtype = _dt(x)
    a.x, a.out = x.data_ptr(), y.data_ptr()
    for k in ("W_in", "W_x", "W_dt", "W_out"):
        if w[k].dtype != x.dtype:
            raise L.HxError(4, f"{k} has dtype {w[k].dtype}, expected {x.dtype}")
        setattr(a, k, w[k].contiguous().data_ptr())
    a.conv_w = _f32(w["conv_w"]).data_ptr()
    if w.get("conv_b") is not None:
        a.conv_b = _f32(w["conv_b"]).data_ptr()
    a.b_dt = _f32(w["b_dt"]).data_ptr()
    a.A = _f32(w["A"]).data_ptr()
    a.Dskip = _f32(w["D"]).data_ptr()
    if h.dtype != torch.float32 or conv_state.dtype != x.dtype:
        raise L.HxError(4, "h must be fp32 and conv_state must have the dtype of x")
    a.h, a.conv_state = h.data_ptr(), conv_state.data_ptr()
    if residual is not None:
        a.residual, a.norm_w, a.norm_eps = residual.data_ptr(), _f32(norm_w).data_ptr(), norm_eps
    n = C.c_size_t(0)
    L.check(L.lib().hx_mamba_step_workspace_bytes(C.byref(a), C.byref(n)))
    if workspace is None:
        workspace = torch.empty(n.value, dtype=torch.uint8, device=x.device)
    a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    L.check(L.lib().hx_mamba_block_step(C.byref(a), _stream()))
    return y


class HostScan:
    """hx_selective_scan_host on pinned host activations: owns the pinned buffers and the device
    staging area, so that each call is exactly the H2D copies, the kernel and the D2H copy."""

    def __init__(self, batch, seq_len, d_inner, d_state, dtype, A, D=None, conv_w=None, conv_b=None, dt_bias=None,
                 gate=True, variant=L.SCAN_AUTO, lanes_per_channel=0, device="cuda"):
        self.shape = (batch, seq_len, d_inner, d_state)
        self.dtype = dtype
        pin = lambda *s: torch.empty(s, dtype=dtype).pin_memory()
        self.x, self.dt = pin(batch, seq_len, d_inner), pin(batch, seq_len, d_inner)
        self.z = pin(batch, seq_len, d_inner) if gate else None
        self.Bm, self.Cm = pin(batch, seq_len, d_state), pin(batch, seq_len, d_state)
        self.y = pin(batch, seq_len, d_inner)
        self.params = dict(A=A, D=D, conv_w=conv_w, conv_b=conv_b, dt_bias=dt_bias)
        a = L.ScanArgs()
        a.batch, a.seq_len, a.d_inner, a.d_state = batch, seq_len, d_inner, d_state
        a.d_conv = conv_w.shape[1] if conv_w is not None else 0
        a.io_dtype = L.HX_BF16 if dtype == torch.bfloat16 else L.HX_F32
        a.dt_softplus, a.variant, a.lanes_per_channel = 1, variant, lanes_per_channel
        for name, t in (("x", self.x), ("dt", self.dt), ("z", self.z), ("y", self.y)):
            if t is not None:
                setattr(a, name, t.data_ptr())
                setattr(a, f"{name}_batch_stride", t.stride(0))
                setattr(a, f"{name}_row_stride", t.stride(1))
        for name, f, t in (("Bm", "B", self.Bm), ("Cm", "C", self.Cm)):
            setattr(a, name, t.data_ptr())
            setattr(a, f"{f}_batch_stride", t.stride(0))
            setattr(a, f"{f}_row_stride", t.stride(1))
        a.A = _f32(A).data_ptr()
        for name, t in (("Dskip", D), ("conv_w", conv_w), ("conv_b", conv_b), ("dt_bias", dt_bias)):
            if t is not None:
                setattr(a, name, _f32(t).data_ptr())
        a.a_geometric = 1 if check_geometric(A) else 0
        n = C.c_size_t(0)
        L.check(L.lib().hx_selective_scan_host_workspace_bytes(C.byref(a), C.byref(n)))
        self.ws = torch.empty(n.value, dtype=torch.uint8, device=device)
        self.args = a
        es = self.x.element_size()
        self.h2d_bytes = sum(t.numel() * es for t in (self.x, self.dt, self.z, self.Bm, self.Cm) if t is not None)
        self.d2h_bytes = self.y.numel() * es

    def run(self):
        L.check(L.lib().hx_selective_scan_host(C.byref(self.args), _p(self.ws), self.ws.numel(), _stream()))
        return self.y
