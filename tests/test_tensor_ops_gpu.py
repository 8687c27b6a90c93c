"""The reference's tensor traits on the device tensor (hx_tensor_* through the C ABI) against the CPU restatement
of CpuTensor's arithmetic (oracle/oracle_np.py t_*, crates/backend-cpu/src/lib.rs).  Add, sub, mul, div, the
scalar forms, matmul and the structural ops are bit-exact; the libm functions are within the fp32 parity gate."""
import numpy as np
import pytest

from conftest import FP32_TOL, fp32_tol_err
from helixml_b200 import _lib, nn, synth
from oracle import cbind, oracle_np as onp

pytestmark = pytest.mark.gpu


def T(a, dtype=nn.F32):
    return nn.Tensor.from_numpy(np.asarray(a, np.float32), dtype)


def variant_of(fn):
    with pytest.raises(_lib.HxError) as e:
        fn()
    return e.value.variant


def test_reference_known_answers_on_device():
    """The two numeric tests the reference holds for these primitives: ones + ones = 2
    (crates/backend-cpu/src/lib.rs:1733-1744) and ones[2,3] . ones[3,4] = 3 (:1747-1758)."""
    s = nn.Tensor.ones([2, 3]).add(nn.Tensor.ones([2, 3]))
    assert s.shape == (2, 3) and np.array_equal(s.numpy(), np.full((2, 3), 2.0, np.float32))
    m = nn.Tensor.ones([2, 3]).matmul(nn.Tensor.ones([3, 4]))
    assert m.shape == (2, 4) and np.array_equal(m.numpy(), np.full((2, 4), 3.0, np.float32))


@pytest.mark.parametrize("name", ["add", "sub", "mul", "div", "max", "min", "gt"])
def test_binary_ops_bit_exact(name):
    a = synth.normal(60, "a", (7, 33))
    b = synth.normal(60, "b", (7, 33))
    got = getattr(T(a), name)(T(b)).numpy()
    assert np.array_equal(got, onp.t_binary(name, a, b))
    assert variant_of(lambda: getattr(T(a), name)(T(b[:, :32]))) == "ShapeMismatch"


@pytest.mark.parametrize("name,p0,p1", [("sqrt", 0, 0), ("exp", 0, 0), ("log", 0, 0), ("sin", 0, 0), ("cos", 0, 0), ("tan", 0, 0),
                                        ("abs", 0, 0), ("sign", 0, 0), ("neg", 0, 0), ("relu", 0, 0), ("gelu", 0, 0),
                                        ("silu", 0, 0), ("sigmoid", 0, 0), ("tanh", 0, 0), ("pow", 2.5, 0), ("clamp", -0.5, 0.7),
                                        ("add_scalar", 0.3, 0), ("mul_scalar", 0.1, 0), ("gt_scalar", 0.2, 0),
                                        ("leaky_relu", 0.01, 0)])
def test_unary_ops(name, p0, p1):
    x = synth.normal(61, "x", (5, 41))
    if name in ("sqrt", "log", "pow"):
        x = np.abs(x) + np.float32(0.01)
    x.flat[:2] = (0.0, -0.0)
    if name == "log":
        x.flat[:2] = (1.0, 2.0)
    t = T(x)
    args = {"pow": (p0,), "clamp": (p0, p1), "add_scalar": (p0,), "mul_scalar": (p0,), "gt_scalar": (p0,), "leaky_relu": (p0,)}.get(name, ())
    got = getattr(t, name)(*args).numpy()
    ref = onp.t_unary(name, x, p0, p1)
    if name in ("abs", "sign", "neg", "relu", "clamp", "add_scalar", "mul_scalar", "gt_scalar", "leaky_relu", "sqrt"):
        assert np.array_equal(got, ref)
    else:
        assert fp32_tol_err(got, ref) <= FP32_TOL


@pytest.mark.parametrize("shapes", [((9, 37), (37, 21)), ((37,), (37, 21)), ((9, 37), (37,)), ((100, 100), (100, 100))])
def test_matmul_is_the_reference_loop(shapes):
    a = synth.normal(62, "a", shapes[0])
    b = synth.normal(62, "b", shapes[1])
    got = T(a).matmul(T(b)).numpy()
    ref = onp.t_matmul(a, b)
    assert got.shape == ref.shape and np.array_equal(got, ref)
    if a.ndim == 2 and b.ndim == 2:  # and the C oracle's matmul agrees (crates/backend-cpu/src/lib.rs:657-668)
        assert np.array_equal(got, cbind.matmul(a, b))


def test_matmul_shape_errors():
    a, b = T(np.ones((3, 4))), T(np.ones((5, 6)))
    assert variant_of(lambda: a.matmul(b)) == "ShapeMismatch"
    assert variant_of(lambda: T(np.ones((2, 3, 4))).matmul(b)) == "UnsupportedOperation"


def test_structural_ops():
    x = synth.normal(63, "x", (6, 10))
    t = T(x)
    assert np.array_equal(t.transpose(0, 1).numpy(), onp.t_transpose(x, 0, 1))
    x3 = synth.normal(63, "x3", (3, 4, 5))
    assert np.array_equal(T(x3).transpose(0, 2).numpy(), onp.t_transpose(x3, 0, 2))
    assert variant_of(lambda: t.transpose(0, 2)) == "InvalidDimension"
    assert np.array_equal(t.slice([1, 2], [4, 9]).numpy(), onp.t_slice(x, [1, 2], [4, 9]))
    # the slice S4Block::forward_ssm takes per step: one column of [d_model, L], then reshape to [d_model]
    col = t.slice([0, 3], [6, 4]).reshape([6])
    assert np.array_equal(col.numpy(), x[:, 3])
    assert variant_of(lambda: t.slice([0, 0], [7, 1])) == "InvalidDimension"
    assert variant_of(lambda: t.slice([2, 0], [2, 1])) == "InvalidDimension"
    assert variant_of(lambda: T(x3).slice([0, 0, 0], [1, 1, 1])) == "UnsupportedOperation"
    assert variant_of(lambda: t.reshape([7, 9])) == "ShapeMismatch"
    v = [synth.normal(63, f"v{i}", (5,)) for i in range(3)]
    assert np.array_equal(nn.Tensor.cat([T(a) for a in v], 0).numpy(), onp.t_cat(v, 0))
    assert variant_of(lambda: nn.Tensor.cat([t, t], 0)) == "UnsupportedOperation"
    assert np.array_equal(t.clone().numpy(), x)


@pytest.mark.parametrize("dim", [0, 1])
def test_stack_keeps_the_reference_layout(dim):
    """stack(outputs, 1) in S4Block::forward_ssm (crates/nn/src/ssm.rs:185): the data are the operands one after
    the other whatever `dim`, only the label has the new axis at `dim` (crates/backend-cpu/src/lib.rs:281-296)."""
    v = [synth.normal(64, f"v{i}", (4,)) for i in range(3)]
    s = nn.Tensor.stack([T(a) for a in v], dim)
    buf, label = onp.t_stack(v, dim)
    assert s.shape == label
    assert np.array_equal(s.numpy().reshape(-1), buf.reshape(-1))
    m = [synth.normal(64, f"m{i}", (2, 3)) for i in range(4)]
    s2 = nn.Tensor.stack([T(a) for a in m], dim)
    buf2, label2 = onp.t_stack(m, dim)
    assert s2.shape == label2 and np.array_equal(s2.numpy().reshape(-1), buf2.reshape(-1))
    assert variant_of(lambda: nn.Tensor.stack([T(v[0]), T(m[0])], 0)) == "ShapeMismatch"


def test_broadcast_to():
    b = synth.normal(65, "b", (7,))
    # the bias broadcast of Linear::forward (crates/nn/src/lib.rs:127-131) and the gate of the ssm-Mamba block
    assert np.array_equal(T(b).broadcast_to([5, 7]).numpy(), onp.t_broadcast_to(b, (5, 7)))
    assert np.array_equal(T(b).broadcast_to([2, 5, 7]).numpy(), onp.t_broadcast_to(b, (2, 5, 7)))
    m = synth.normal(65, "m", (5, 7))
    assert np.array_equal(T(m).broadcast_to([3, 5, 7]).numpy(), onp.t_broadcast_to(m, (3, 5, 7)))
    r = synth.normal(65, "r", (1, 7))
    assert np.array_equal(T(r).broadcast_to([5, 7]).numpy(), onp.t_broadcast_to(r, (5, 7)))
    c = synth.normal(65, "c", (5, 1))
    assert np.array_equal(T(c).broadcast_to([5, 7]).numpy(), onp.t_broadcast_to(c, (5, 7)))
    assert variant_of(lambda: T(b).broadcast_to([5, 8])) == "ShapeMismatch"
    assert variant_of(lambda: T(m).broadcast_to([7])) == "ShapeMismatch"


def test_cast_scalar_and_constructors():
    x = synth.normal(66, "x", (4, 9))
    bf = T(x).cast(nn.BF16)
    assert bf.dtype == nn.BF16 and np.array_equal(bf.numpy(), synth.round_bf16(x))
    assert np.array_equal(bf.cast(nn.F32).numpy(), synth.round_bf16(x))
    assert variant_of(lambda: T(x).cast(nn.U8)) == "UnsupportedOperation"
    assert T(np.array([2.5])).to_scalar() == 2.5
    assert variant_of(lambda: T(x).to_scalar()) == "InvalidInput"
    assert np.array_equal(nn.Tensor.zeros([2, 3]).numpy(), np.zeros((2, 3), np.float32))
    assert np.array_equal(nn.Tensor.from_scalar(1.5, [4]).numpy(), np.full(4, 1.5, np.float32))
    assert np.array_equal(nn.Tensor.eye(3).numpy(), np.eye(3, dtype=np.float32))
    ar = nn.Tensor.arange(0.0, 1.0, 0.25).numpy()
    assert np.array_equal(ar, np.array([0.0, 0.25, 0.5, 0.75], np.float32))
    nn.manual_seed(5)
    n1 = nn.Tensor.random_normal([20000], 1.0, 2.0).numpy()
    assert abs(n1.mean() - 1.0) < 0.06 and abs(n1.std() - 2.0) < 0.06
    u = nn.Tensor.random_uniform([20000], -1.0, 3.0).numpy()
    assert u.min() >= -1.0 and u.max() < 3.0 and abs(u.mean() - 1.0) < 0.05
    be = nn.Tensor.random_bernoulli([20000], 0.3).numpy()
    assert set(np.unique(be)) <= {0.0, 1.0} and abs(be.mean() - 0.3) < 0.02
    nn.manual_seed(5)
    assert np.array_equal(nn.Tensor.random_normal([20000], 1.0, 2.0).numpy(), n1)  # the seed makes it reproducible


def test_s4_forward_ssm_composed_from_primitives():
    """S4Block::forward_ssm written with the tensor primitives exactly as the reference writes it
    (crates/nn/src/ssm.rs:103-186: discretize, per-step slice / reshape / matmul / mul / add, stack) gives the
    oracle's output bit for bit, and the fused path (hx_s4_ref_forward_ssm) agrees within the fp32 gate."""
    M, N, L = 6, 4, 9
    A_re = synth.uniform(67, "are", (N,), -0.5, 0.0)
    A_im = synth.normal(67, "aim", (N,))
    Bm = synth.normal(67, "B", (N, M), 0, 0.3)
    Cm = synth.normal(67, "C", (M, N), 0, 0.3)
    Dv = synth.normal(67, "D", (M,), 0, 0.3)
    u = synth.normal(67, "u", (M, L))
    dt = 0.1
    a = T(A_re).mul_scalar(dt).exp().mul(T(A_im).mul_scalar(dt).cos())          # ssm.rs:113-125
    Bd = T(Bm).mul_scalar(dt)                                                    # ssm.rs:130
    state = nn.Tensor.zeros([N])
    outs = []
    ut = T(u)
    for t in range(L):
        u_t = ut.slice([0, t], [M, t + 1]).reshape([M])                          # ssm.rs:168-169
        state = a.mul(state).add(Bd.matmul(u_t))                                 # ssm.rs:172-174
        outs.append(T(Cm).matmul(state).add(T(Dv).mul(u_t)))                     # ssm.rs:177-179
    y = nn.Tensor.stack(outs, 1)                                                 # ssm.rs:185
    assert y.shape == (M, L)                                                     # the label; the buffer is [L, M]
    ref = cbind.s4_forward_ssm(u, A_re, A_im, Bm, Cm, Dv, dt)
    got = y.numpy().reshape(L, M)
    # exp and cos come from different math libraries on the two sides: 1 ulp in `a`, then identical arithmetic
    assert fp32_tol_err(got, ref.reshape(L, M)) <= 1e-6


def test_reference_ssm_mamba_block():
    """nn::ssm::MambaBlock::forward_mamba as the reference computes it (crates/nn/src/ssm.rs:435-483): identity
    conv, delta = x . delta_proj, S4 recurrence on delta, row-broadcast gate; square input only."""
    import ctypes as C
    import torch
    M, N = 48, 8
    x = synth.normal(68, "x", (M, M))
    dp = synth.normal(68, "dp", (M, M), 0, 0.1)
    gate = synth.normal(68, "g", (M,), 0, 0.1)
    A_re = np.zeros(N, np.float32)
    A_im = synth.normal(68, "aim", (N,))
    Bm = synth.normal(68, "B", (N, M), 0, 0.1)
    Cm = synth.normal(68, "C", (M, N), 0, 0.1)
    Dv = synth.normal(68, "D", (M,), 0, 0.1)
    ref = cbind.mamba_ssm(x, dp, gate, A_re, A_im, Bm, Cm, Dv)
    dev = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (x, dp, gate, A_re, A_im, Bm, Cm, Dv)]
    out = torch.empty((M, M), device="cuda")
    L_ = _lib.lib()
    need = L_.hx_mamba_ssm_ref_workspace_bytes(M, N)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(L_.hx_mamba_ssm_ref_forward(*[C.c_void_p(t.data_ptr()) for t in dev], C.c_void_p(out.data_ptr()), M, N,
                                           C.c_void_p(ws.data_ptr()), need, st))
    assert fp32_tol_err(out.cpu().numpy(), np.asarray(ref).reshape(M, M)) <= FP32_TOL
    # too small a workspace is an error, not a fault
    assert L_.hx_mamba_ssm_ref_forward(*[C.c_void_p(t.data_ptr()) for t in dev], C.c_void_p(out.data_ptr()), M, N,
                                       C.c_void_p(ws.data_ptr()), need - 1, st) == 10
