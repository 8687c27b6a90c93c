"""ctypes binding to oracle/liboracle.so (the C restatement).  TEST INFRASTRUCTURE ONLY.

Every wrapper takes and returns numpy arrays; `prec` selects the f32 build (the
reference's arithmetic) or the f64 shadow build."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force: bool = False) -> str:
    path = os.path.join(_HERE, "liboracle.so")
    srcs = [os.path.join(_HERE, f) for f in ("oracle.c", "oracle_body.inc", "Makefile")]
    stale = not os.path.exists(path) or any(os.path.getmtime(s) > os.path.getmtime(path) for s in srcs)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return path


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        _LIB.orc_num_threads.restype = C.c_int
    return _LIB


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))


def _dt(prec):
    return (np.float32, "f32") if prec == "f32" else (np.float64, "f64")


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    return None if a is None else np.ascontiguousarray(a, dtype=dtype)


def _i(v):
    return C.c_int64(int(v))


def add(a, b, prec="f32"):
    dt, s = _dt(prec)
    a, b = _c(a, dt), _c(b, dt)
    out = np.empty_like(a)
    getattr(lib(), "orc_r_add_" + s)(_p(a), _p(b), _p(out), _i(a.size))
    return out


def matmul(a, b, prec="f32"):
    dt, s = _dt(prec)
    a, b = _c(a, dt), _c(b, dt)
    out = np.empty((a.shape[0], b.shape[1]), dtype=dt)
    getattr(lib(), "orc_r_matmul_" + s)(_p(a), _p(b), _p(out), _i(a.shape[0]), _i(a.shape[1]), _i(b.shape[1]))
    return out


def silu(x, prec="f32"):
    dt, s = _dt(prec)
    x = _c(x, dt)
    out = np.empty_like(x)
    getattr(lib(), "orc_r_silu_" + s)(_p(x), _p(out), _i(x.size))
    return out


def linear(x, w, bias=None, prec="f32"):
    dt, s = _dt(prec)
    x, w, bias = _c(x, dt), _c(w, dt), _c(bias, dt)
    M, K = x.shape
    out = np.empty((M, w.shape[0]), dtype=dt)
    getattr(lib(), "orc_r_linear_" + s)(_p(x), _p(w), _p(bias), _p(out), _i(M), _i(K), _i(w.shape[0]))
    return out


def rmsnorm(x, w, eps=1e-5, prec="f32"):
    dt, s = _dt(prec)
    x, w = _c(x, dt), _c(w, dt)
    out = np.empty_like(x)
    real = C.c_float if prec == "f32" else C.c_double
    getattr(lib(), "orc_r_rmsnorm_" + s)(_p(x), _p(w), _p(out), _i(x.size // x.shape[-1]), _i(x.shape[-1]), real(eps))
    return out


def s4_forward_ssm(u, A_real, A_imag, Bm, Cm, Dv, dt=0.1, prec="f32"):
    """Oracle-R S4: u [M, L] -> buffer [L, M]."""
    d, s = _dt(prec)
    u, A_real, A_imag, Bm, Cm, Dv = (_c(a, d) for a in (u, A_real, A_imag, Bm, Cm, Dv))
    M, L = u.shape
    N = A_real.shape[0]
    out = np.empty((L, M), dtype=d)
    real = C.c_float if prec == "f32" else C.c_double
    getattr(lib(), "orc_r_s4_forward_ssm_" + s)(_p(u), _p(A_real), _p(A_imag), _p(Bm), _p(Cm), _p(Dv),
                                                 real(dt), _p(out), _i(M), _i(L), _i(N))
    return out


def mamba_exported(x, wg, bg, wo, bo, prec="f32"):
    d, s = _dt(prec)
    x, wg, bg, wo, bo = (_c(a, d) for a in (x, wg, bg, wo, bo))
    L, M = x.shape
    E = wg.shape[0]
    out = np.empty((L, M), dtype=d)
    getattr(lib(), "orc_r_mamba_exported_" + s)(_p(x), _p(wg), _p(bg), _p(wo), _p(bo), _p(out), _i(L), _i(M), _i(E))
    return out


def mamba_ssm(x, delta_proj, gate, A_real, A_imag, Bm, Cm, Dv, prec="f32"):
    d, s = _dt(prec)
    x, delta_proj, gate, A_real, A_imag, Bm, Cm, Dv = (_c(a, d) for a in (x, delta_proj, gate, A_real, A_imag, Bm, Cm, Dv))
    M = x.shape[0]
    out = np.empty((M, M), dtype=d)
    getattr(lib(), "orc_r_mamba_ssm_" + s)(_p(x), _p(delta_proj), _p(gate), _p(A_real), _p(A_imag), _p(Bm), _p(Cm),
                                            _p(Dv), _p(out), _i(M), _i(A_real.shape[0]))
    return out


def selective_scan(x, dt, A, Bm, Cm, D=None, z=None, conv_w=None, conv_b=None, dt_bias=None,
                   dt_softplus=True, return_state=False, prec="f32"):
    d, s = _dt(prec)
    x, dt, z, Bm, Cm, A, D, conv_w, conv_b, dt_bias = (_c(a, d) for a in (x, dt, z, Bm, Cm, A, D, conv_w, conv_b, dt_bias))
    B, L, Dm = x.shape
    N = A.shape[1]
    K = conv_w.shape[1] if conv_w is not None else 0
    y = np.empty((B, L, Dm), dtype=d)
    h = np.empty((B, Dm, N), dtype=d) if return_state else None
    getattr(lib(), "orc_m_selective_scan_" + s)(_p(x), _p(dt), _p(z), _p(Bm), _p(Cm), _p(A), _p(D), _p(conv_w),
                                                 _p(conv_b), _p(dt_bias), C.c_int(1 if dt_softplus else 0), _p(y),
                                                 _p(h), _i(B), _i(L), _i(Dm), _i(N), _i(K))
    return (y, h) if return_state else y


def conv_silu(xs, conv_w, conv_b=None, prec="f32"):
    d, s = _dt(prec)
    xs, conv_w, conv_b = _c(xs, d), _c(conv_w, d), _c(conv_b, d)
    B, L, Dm = xs.shape
    u = np.empty((B, L, Dm), dtype=d)
    getattr(lib(), "orc_m_conv_silu_" + s)(_p(xs), _p(conv_w), _p(conv_b), _p(u), _i(B), _i(L), _i(Dm),
                                            _i(conv_w.shape[1]), _i(Dm))
    return u


def s4_diag(u, A, Bp, Cp, delta, D=None, prec="f32"):
    d, s = _dt(prec)
    u, A, Bp, Cp, delta, D = (_c(a, d) for a in (u, A, Bp, Cp, delta, D))
    B, L, Dm = u.shape
    y = np.empty((B, L, Dm), dtype=d)
    getattr(lib(), "orc_m_s4_diag_" + s)(_p(u), _p(A), _p(Bp), _p(Cp), _p(delta), _p(D), _p(y), _i(B), _i(L),
                                          _i(Dm), _i(A.shape[1]))
    return y


def mamba_block(x, w: dict, d_state: int, d_conv: int, return_parts=False, prec="f32"):
    """Oracle-M block.  x [B,L,M]; w as produced by synth.mamba_block_weights."""
    d, s = _dt(prec)
    x = _c(x, d)
    W = {k: _c(v, d) for k, v in w.items()}
    B, L, M = x.shape
    E = W["W_in"].shape[0] // 2
    R = W["W_dt"].shape[1]
    out = np.empty((B, L, M), dtype=d)
    parts = None
    if return_parts:
        parts = {"u": np.empty((B, L, E), dtype=d), "dbc": np.empty((B, L, R + 2 * d_state), dtype=d),
                 "dtlin": np.empty((B, L, E), dtype=d), "y": np.empty((B, L, E), dtype=d)}
    getattr(lib(), "orc_m_mamba_block_" + s)(
        _p(x), _p(W["W_in"]), _p(W["conv_w"]), _p(W.get("conv_b")), _p(W["W_x"]), _p(W["W_dt"]), _p(W["b_dt"]),
        _p(W["A"]), _p(W["D"]), _p(W["W_out"]), _p(out),
        _p(parts["u"]) if parts else None, _p(parts["dbc"]) if parts else None,
        _p(parts["dtlin"]) if parts else None, _p(parts["y"]) if parts else None,
        _i(B), _i(L), _i(M), _i(E), _i(d_state), _i(d_conv), _i(R))
    return (out, parts) if return_parts else out


def byte_lm(tokens, emb, layers: list, normf_w, d_state: int, d_conv: int, eps=1e-5, return_hidden=False, prec="f32"):
    """Oracle-M byte LM.  tokens uint8 [B,L]; layers: list of dicts with the block weights plus "norm_w"."""
    d, s = _dt(prec)
    tokens = np.ascontiguousarray(tokens, dtype=np.uint8)
    B, L = tokens.shape
    emb = _c(emb, d)
    normf_w = _c(normf_w, d)
    V, M = emb.shape
    Ls = [{k: _c(v, d) for k, v in l.items()} for l in layers]
    E = Ls[0]["W_in"].shape[0] // 2
    R = Ls[0]["W_dt"].shape[1]
    nl = len(Ls)

    def arr(key):
        return (C.c_void_p * nl)(*[l[key].ctypes.data for l in Ls])

    logits = np.empty((B, L, V), dtype=d)
    hidden = np.empty((B, L, M), dtype=d) if return_hidden else None
    real = C.c_float if prec == "f32" else C.c_double
    getattr(lib(), "orc_m_byte_lm_" + s)(
        _p(tokens), _p(emb), arr("norm_w"), arr("W_in"), arr("conv_w"), arr("conv_b"), arr("W_x"), arr("W_dt"),
        arr("b_dt"), arr("A"), arr("D"), arr("W_out"), _p(normf_w), real(eps), _p(logits), _p(hidden),
        _i(nl), _i(B), _i(L), _i(M), _i(E), _i(d_state), _i(d_conv), _i(R), _i(V))
    return (logits, hidden) if return_hidden else logits


def round_bf16(x):
    x = _c(x, np.float32)
    out = np.empty_like(x)
    lib().orc_round_bf16(_p(x), _p(out), _i(x.size))
    return out


def byte_lm_bf16_storage(tokens, emb, layers: list, normf_w, d_state: int, d_conv: int, eps=1e-5):
    """The byte LM of byte_lm() with every value rounded to bf16 at the points where a bf16 activation path has
    to store it (the normed block input, the in_proj output, u, the x_proj output, the scan output, the logits),
    f32 arithmetic everywhere else and an f32 residual stream.  This is not a second oracle: it measures how far
    bf16 STORAGE alone moves the f32 result, i.e. the floor no bf16 implementation of the model can go below,
    so that a test can tell rounding of the format from error of a kernel.  tokens [B, L] -> logits [B, L, 256]."""
    rb = round_bf16
    tokens = np.asarray(tokens)
    out = []
    for row in tokens:
        h = np.asarray(emb, np.float32)[row].astype(np.float32)
        for w in layers:
            E, R = w["W_in"].shape[0] // 2, w["W_dt"].shape[1]
            x = rb(rmsnorm(h, w["norm_w"], eps))
            xz = rb(linear(x, w["W_in"]))
            u = rb(conv_silu(np.ascontiguousarray(xz[:, :E])[None], w["conv_w"], w.get("conv_b"))[0])
            dbc = rb(linear(u, w["W_x"]))
            dt = linear(np.ascontiguousarray(dbc[:, :R]), w["W_dt"])
            y = selective_scan(u[None], dt[None], w["A"], np.ascontiguousarray(dbc[None, :, R:R + d_state]),
                               np.ascontiguousarray(dbc[None, :, R + d_state:]), D=w["D"], z=np.ascontiguousarray(xz[:, E:])[None],
                               dt_bias=w["b_dt"])[0]
            h = h + linear(rb(y), w["W_out"])
        out.append(rb(linear(rb(rmsnorm(h, normf_w, eps)), emb)))
    return np.stack(out)
