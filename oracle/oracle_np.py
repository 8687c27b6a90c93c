"""numpy twin of the C oracle (TEST INFRASTRUCTURE ONLY).

Vectorised over (batch, channel) and sequential in time, in the dtype of its inputs.
It exists to cross-check oracle.c: the two were written separately from the same
description and must agree (exactly where the operation order is the same, to a few
ulp where numpy's exp differs from libm's)."""
from __future__ import annotations

import numpy as np


def silu(x):
    return x / (1 + np.exp(-x))


def softplus(v):
    with np.errstate(over="ignore"):
        return np.where(v > 20, v, np.log(1 + np.exp(v))).astype(v.dtype)


def linear(x, w, bias=None):
    """x [M,K], w [N,K]; sequential-k accumulation like crates/backend-cpu/src/lib.rs:659-667."""
    out = np.zeros((x.shape[0], w.shape[0]), dtype=x.dtype)
    for k in range(x.shape[1]):
        out += x[:, k:k + 1] * w[None, :, k]
    return out + bias if bias is not None else out


def rmsnorm(x, w, eps=1e-5):
    """crates/nn/src/lib.rs:258-285 (eps jitter dropped)."""
    ss = np.zeros(x.shape[:-1], dtype=x.dtype)
    for j in range(x.shape[-1]):
        ss += x[..., j] * x[..., j]
    rms = np.sqrt(ss / x.dtype.type(x.shape[-1]) + x.dtype.type(eps))
    return x / rms[..., None] * w


def s4_forward_ssm(u, A_real, A_imag, Bm, Cm, Dv, dt=0.1):
    """crates/nn/src/ssm.rs:103-186.  u [M,L] -> buffer [L,M]."""
    t = u.dtype.type
    a = np.exp(A_real * t(dt)) * np.cos(A_imag * t(dt))
    Bd = Bm * t(dt)
    M, L = u.shape
    N = a.shape[0]
    state = np.zeros(N, dtype=u.dtype)
    out = np.empty((L, M), dtype=u.dtype)
    for k in range(L):
        ut = u[:, k]
        s = np.zeros(N, dtype=u.dtype)
        for m in range(M):
            s += Bd[:, m] * ut[m]
        state = a * state + s
        y = np.zeros(M, dtype=u.dtype)
        for n in range(N):
            y += Cm[:, n] * state[n]
        out[k] = y + Dv * ut
    return out


def mamba_exported(x, wg, bg, wo, bo):
    """crates/nn/src/lib.rs:888-906."""
    return linear(silu(linear(x, wg, bg)), wo, bo)


def conv_silu(xs, conv_w, conv_b=None):
    B, L, D = xs.shape
    K = conv_w.shape[1]
    c = np.zeros_like(xs) if conv_b is None else np.broadcast_to(conv_b, xs.shape).astype(xs.dtype).copy()
    for j in range(K):
        sh = K - 1 - j
        if sh < L:
            c[:, sh:, :] += conv_w[:, j] * xs[:, :L - sh, :]
    return silu(c)


def selective_scan(x, dt, A, Bm, Cm, D=None, z=None, conv_w=None, conv_b=None, dt_bias=None, dt_softplus=True,
                   return_state=False):
    B, L, Dm = x.shape
    N = A.shape[1]
    u = conv_silu(x, conv_w, conv_b) if conv_w is not None else x
    v = dt + dt_bias if dt_bias is not None else dt
    dtv = softplus(v) if dt_softplus else v
    h = np.zeros((B, Dm, N), dtype=x.dtype)
    y = np.empty_like(x)
    for t in range(L):
        xin = dtv[:, t, :] * u[:, t, :]
        h = np.exp(dtv[:, t, :, None] * A[None]) * h + xin[:, :, None] * Bm[:, t, None, :]
        acc = np.zeros((B, Dm), dtype=x.dtype)
        for n in range(N):
            acc += Cm[:, t, None, n] * h[:, :, n]
        if D is not None:
            acc = acc + D * u[:, t, :]
        if z is not None:
            acc = acc * silu(z[:, t, :])
        y[:, t, :] = acc
    return (y, h) if return_state else y


def s4_diag(u, A, Bp, Cp, delta, D=None):
    B, L, Dm = u.shape
    N = A.shape[1]
    abar = np.exp(delta[:, None] * A)
    bbar = delta[:, None] * Bp
    h = np.zeros((B, Dm, N), dtype=u.dtype)
    y = np.empty_like(u)
    for t in range(L):
        h = abar[None] * h + bbar[None] * u[:, t, :, None]
        acc = np.zeros((B, Dm), dtype=u.dtype)
        for n in range(N):
            acc += Cp[None, :, n] * h[:, :, n]
        y[:, t, :] = acc + (D * u[:, t, :] if D is not None else 0)
    return y


def mamba_block(x, w, d_state, d_conv):
    B, L, M = x.shape
    E = w["W_in"].shape[0] // 2
    R = w["W_dt"].shape[1]
    xz = linear(x.reshape(B * L, M), w["W_in"]).reshape(B, L, 2 * E)
    xs, z = xz[..., :E], xz[..., E:]
    u = conv_silu(xs, w["conv_w"], w.get("conv_b"))
    dbc = linear(u.reshape(B * L, E), w["W_x"])
    dtl = linear(np.ascontiguousarray(dbc[:, :R]), w["W_dt"]).reshape(B, L, E)
    Bm = dbc[:, R:R + d_state].reshape(B, L, d_state)
    Cm = dbc[:, R + d_state:].reshape(B, L, d_state)
    y = selective_scan(u, dtl, w["A"], Bm, Cm, D=w["D"], z=z, dt_bias=w["b_dt"], dt_softplus=True)
    return linear(y.reshape(B * L, E), w["W_out"]).reshape(B, L, M)


# ---------------------------------------------------------------- tensor primitives (Oracle-R)
# CpuTensor's own arithmetic, crates/backend-cpu/src/lib.rs.  Element-wise work goes through ndarray, i.e. plain
# IEEE f32 operations, which numpy's float32 arrays reproduce bit for bit.

def t_binary(name, a, b):
    """add/sub/mul/div (:570-632), max/min (:852-899), gt (:951-975): identical shapes, else ShapeMismatch."""
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    if a.shape != b.shape:
        raise ValueError("ShapeMismatch")
    with np.errstate(all="ignore"):
        return {"add": lambda: a + b, "sub": lambda: a - b, "mul": lambda: a * b, "div": lambda: a / b,
                "max": lambda: np.fmax(a, b), "min": lambda: np.fmin(a, b),
                "gt": lambda: (a > b).astype(np.float32)}[name]().astype(np.float32)


def t_unary(name, x, p0=0.0, p1=0.0):
    """pow .. neg (:759-899), scalar ops (:913-949), activations (:1100-1198).  Evaluated in float64 and rounded,
    which stands in for Rust's f32 libm to within 1 ulp."""
    x32 = np.asarray(x, np.float32)
    x = x32.astype(np.float64)
    p0f, p1f = np.float32(p0), np.float32(p1)
    with np.errstate(all="ignore"):
        if name == "sign":  # f32::signum: 1.0 for +0.0, -1.0 for -0.0, NaN for NaN
            r = np.where(np.isnan(x32), x32, np.copysign(np.float32(1), x32))
        elif name == "gelu":
            c = np.float32(np.sqrt(np.float32(2.0) / np.float32(np.pi)))
            r = 0.5 * x * (1.0 + np.tanh(float(c) * (x + 0.044715 * x ** 3)))
        else:
            r = {"sqrt": lambda: np.sqrt(x), "exp": lambda: np.exp(x), "log": lambda: np.log(x), "sin": lambda: np.sin(x),
                 "cos": lambda: np.cos(x), "tan": lambda: np.tan(x), "abs": lambda: np.abs(x), "neg": lambda: -x,
                 "relu": lambda: np.maximum(x, 0.0), "silu": lambda: x / (1.0 + np.exp(-x)),
                 "sigmoid": lambda: 1.0 / (1.0 + np.exp(-x)), "tanh": lambda: np.tanh(x),
                 "pow": lambda: np.power(x, float(p0f)), "clamp": lambda: np.minimum(np.maximum(x32, p0f), p1f),
                 "add_scalar": lambda: x32 + p0f, "mul_scalar": lambda: x32 * p0f,
                 "gt_scalar": lambda: (x32 > p0f).astype(np.float32),
                 "leaky_relu": lambda: np.where(x32 >= 0, x32, p0f * x32)}[name]()
    return np.asarray(r).astype(np.float32)


def t_matmul(a, b):
    """(2,2), (1,2), (2,1) products, k ascending into one f32 accumulator, product and sum rounded separately
    (:634-757).  Other ranks: UnsupportedOperation."""
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    if (a.ndim, b.ndim) not in ((2, 2), (1, 2), (2, 1)):
        raise ValueError("UnsupportedOperation")
    A = a.reshape(1, -1) if a.ndim == 1 else a
    Bm = b.reshape(-1, 1) if b.ndim == 1 else b
    if A.shape[1] != Bm.shape[0]:
        raise ValueError("ShapeMismatch")
    out = np.zeros((A.shape[0], Bm.shape[1]), np.float32)
    for k in range(A.shape[1]):
        out = (out + (A[:, k:k + 1] * Bm[k:k + 1, :]).astype(np.float32)).astype(np.float32)
    return out.reshape(-1) if (a.ndim == 1 or b.ndim == 1) else out


def t_transpose(a, d0, d1):
    """permuted_axes(...).to_owned() (:115-137)."""
    return np.ascontiguousarray(np.swapaxes(np.asarray(a), d0, d1))


def t_slice(a, start, end):
    """2-D only (:139-183)."""
    a = np.asarray(a)
    if len(start) != a.ndim or len(end) != a.ndim:
        raise ValueError("ShapeMismatch")
    for i in range(a.ndim):
        if start[i] >= a.shape[i] or end[i] > a.shape[i] or start[i] >= end[i]:
            raise ValueError("InvalidDimension")
    if a.ndim != 2:
        raise ValueError("UnsupportedOperation")
    return np.ascontiguousarray(a[start[0]:end[0], start[1]:end[1]])


def t_cat(ts, dim):
    """1-D only (:184-252)."""
    if ts[0].ndim != 1:
        raise ValueError("UnsupportedOperation")
    return np.concatenate(ts)


def t_stack(ts, dim):
    """The buffer is the operands one after the other, [count, operand shape...], whatever `dim`; the shape LABEL
    has the new axis inserted at `dim` (:254-335).  Returns (buffer, label)."""
    buf = np.stack([np.asarray(t) for t in ts], axis=0)
    label = list(ts[0].shape)
    label.insert(dim, len(ts))
    return buf, tuple(label)


def t_broadcast_to(a, shape):
    """Trailing axes aligned, axes of size 1 repeated (:1352-1518)."""
    return np.ascontiguousarray(np.broadcast_to(np.asarray(a), shape))
