"""CPU tests of the oracle itself: the reference's two known-answer tests for the primitives, the
C restatement against its numpy twin, the f32 build against the f64 shadow, and the committed
golden vectors.  The oracle's S4/Mamba outputs are "parity unpinned" against the reference (it has no
numeric fixture for them); these tests pin the oracle against itself."""
import numpy as np
import pytest

from helixml_b200 import synth
from oracle import cbind, oracle_np as onp


def test_reference_known_answer_add():
    # crates/backend-cpu/src/lib.rs:1733-1744: ones[2,3] + ones[2,3] == 2
    out = cbind.add(np.ones((2, 3), np.float32), np.ones((2, 3), np.float32))
    assert out.shape == (2, 3) and np.all(np.abs(out - 2.0) < 1e-6)


def test_reference_known_answer_matmul():
    # crates/backend-cpu/src/lib.rs:1747-1758: ones[2,3] x ones[3,4] == 3, shape [2,4]
    out = cbind.matmul(np.ones((2, 3), np.float32), np.ones((3, 4), np.float32))
    assert out.shape == (2, 4) and np.all(np.abs(out - 3.0) < 1e-6)


def test_silu_matches_definition():
    x = synth.normal(7, "x", (1000,))
    assert np.allclose(cbind.silu(x), x / (1 + np.exp(-x)), rtol=1e-6, atol=1e-7)


def test_linear_is_sequential_k():
    x = synth.normal(3, "x", (5, 33))
    w = synth.normal(3, "w", (7, 33))
    b = synth.normal(3, "b", (7,))
    assert np.array_equal(cbind.linear(x, w, b), onp.linear(x, w, b))


def test_round_bf16_twins_agree():
    x = np.concatenate([synth.normal(1, "r", (4096,)) * 100, np.array([0.0, -0.0, 1.0, 3.0e38, 1e-40], np.float32)])
    a, b = cbind.round_bf16(x), synth.round_bf16(x)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert np.all((a.view(np.uint32) & 0xFFFF) == 0)


@pytest.mark.parametrize("gate,conv", [(True, True), (False, True), (True, False)])
def test_scan_c_vs_numpy(gate, conv):
    inp = synth.scan_inputs(5, 2, 29, 20, 16, 4, bf16=False)
    kw = dict(D=inp["D"], z=inp["z"] if gate else None, conv_w=inp["conv_w"] if conv else None)
    a, ha = cbind.selective_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], return_state=True, **kw)
    b, hb = onp.selective_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], return_state=True, **kw)
    assert np.max(np.abs(a - b) / (1 + np.abs(b))) < 1e-5
    assert np.max(np.abs(ha - hb) / (1 + np.abs(hb))) < 1e-5


def test_scan_f32_vs_f64_shadow():
    inp = synth.scan_inputs(6, 1, 300, 16, 16, 4, bf16=False)
    kw = dict(D=inp["D"], z=inp["z"], conv_w=inp["conv_w"])
    a = cbind.selective_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], **kw)
    d = cbind.selective_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], prec="f64", **kw)
    # the f32 oracle's own rounding error must sit well inside the 1e-4 parity gate
    assert np.max(np.abs(a - d) / (1 + np.abs(d))) < 2e-5


def test_scan_edge_cases():
    inp = synth.scan_inputs(8, 1, 2, 3, 16, 4, bf16=False)  # L shorter than the conv window
    y = cbind.selective_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], D=inp["D"], z=inp["z"], conv_w=inp["conv_w"])
    y2 = onp.selective_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], D=inp["D"], z=inp["z"], conv_w=inp["conv_w"])
    assert y.shape == (1, 2, 3) and np.allclose(y, y2, rtol=1e-5, atol=1e-6)
    # softplus switches to the identity above 20
    big = np.full((1, 1, 1), 25.0, np.float32)
    one = np.ones((1, 1, 1), np.float32)
    A = -np.ones((1, 16), np.float32)
    Bm = np.ones((1, 1, 16), np.float32)
    y = cbind.selective_scan(one, big, A, Bm, Bm)
    assert np.allclose(y, 16 * 25.0, rtol=1e-6)


def test_s4_diag_c_vs_numpy():
    s = synth.s4_inputs(1, 2, 40, 6, 64)
    assert np.allclose(cbind.s4_diag(s["u"], s["A"], s["B"], s["C"], s["delta"], s["D"]),
                       onp.s4_diag(s["u"], s["A"], s["B"], s["C"], s["delta"], s["D"]), rtol=1e-5, atol=1e-6)


def test_s4_ref_layout_quirk():
    # forward_ssm takes [d_model, L]; the stacked buffer is time-major [L, d_model]
    # (crates/backend-cpu/src/lib.rs:281-296)
    M, L, N = 3, 5, 4
    u = synth.normal(9, "u", (M, L))
    z = np.zeros(N, np.float32)
    y = cbind.s4_forward_ssm(u, z, z, np.zeros((N, M), np.float32), np.zeros((M, N), np.float32), np.ones(M, np.float32))
    assert y.shape == (L, M) and np.array_equal(y, u.T)  # D = 1, everything else 0: y_t = u_t


def test_mamba_ssm_gate_broadcast():
    # crates/nn/src/ssm.rs:458-459: gate [M] is row-broadcast over the square time-major buffer
    M, N = 6, 4
    x = synth.normal(10, "x", (M, M))
    dp = synth.normal(10, "dp", (M, M), 0, 0.1)
    gate = synth.normal(10, "g", (M,))
    Ai = synth.normal(10, "Ai", (N,))
    Bm, Cm = synth.normal(10, "B", (N, M), 0, 0.1), synth.normal(10, "C", (M, N), 0, 0.1)
    Dv = synth.normal(10, "D", (M,))
    out = cbind.mamba_ssm(x, dp, gate, np.zeros(N, np.float32), Ai, Bm, Cm, Dv)
    inner = cbind.s4_forward_ssm(cbind.matmul(x, dp), np.zeros(N, np.float32), Ai, Bm, Cm, Dv)
    assert np.array_equal(out, inner * gate[None, :])


def test_block_c_vs_numpy_and_parts():
    w = synth.mamba_block_weights(4, 32, 16, 4, 2)
    x = synth.uniform(4, "x", (2, 19, 32), -1, 1)
    out, parts = cbind.mamba_block(x, w, 16, 4, return_parts=True)
    assert np.max(np.abs(out - onp.mamba_block(x, w, 16, 4))) < 1e-5
    assert parts["u"].shape == (2, 19, 64) and parts["dbc"].shape == (2, 19, 2 + 32)


def test_byte_lm_runs_and_is_causal():
    layers = []
    for l in range(2):
        w = synth.mamba_block_weights(3, 32, 16, 4, 2, init="0.02", prefix=f"l{l}.")
        w["norm_w"] = np.ones(32, np.float32)
        layers.append(w)
    emb = synth.normal(3, "emb", (256, 32), 0, 0.02)
    tok = synth.random_bytes(3, "tok", (2, 24))
    a = cbind.byte_lm(tok, emb, layers, np.ones(32, np.float32), 16, 4)
    tok2 = tok.copy()
    tok2[:, 12:] = 0
    b = cbind.byte_lm(tok2, emb, layers, np.ones(32, np.float32), 16, 4)
    assert a.shape == (2, 24, 256)
    assert np.array_equal(a[:, :12], b[:, :12]) and not np.array_equal(a[:, 12:], b[:, 12:])


# ---- committed golden vectors -------------------------------------------------------------------

@pytest.mark.parametrize("name", ["scan_f32_small.npz", "scan_bf16_small.npz"])
def test_golden_scan(golden, name):
    g = golden(name)
    kw = dict(D=g["D"], z=g["z"] if int(g["gate"]) else None, conv_w=g["conv_w"],
              conv_b=g["conv_b"] if g["conv_b"].size else None, dt_bias=g["dt_bias"] if g["dt_bias"].size else None)
    y, h = cbind.selective_scan(g["x"], g["dt"], g["A"], g["B"], g["C"], return_state=True, **kw)
    assert np.allclose(y, g["y"], rtol=1e-6, atol=1e-6) and np.allclose(h, g["h_last"], rtol=1e-6, atol=1e-6)
    y2 = onp.selective_scan(g["x"], g["dt"], g["A"], g["B"], g["C"], **kw)
    assert np.max(np.abs(y2 - g["y"]) / (1 + np.abs(g["y"]))) < 2e-5


def test_golden_s4(golden):
    g = golden("s4_diag_small.npz")
    assert np.allclose(cbind.s4_diag(g["u"], g["A"], g["B"], g["C"], g["delta"], g["D"]), g["y"], rtol=1e-6, atol=1e-6)
    r = golden("s4_ref_small.npz")
    assert np.allclose(cbind.s4_forward_ssm(r["u"], r["A_real"], r["A_imag"], r["B"], r["C"], r["D"]), r["y"],
                       rtol=1e-6, atol=1e-7)
    assert np.allclose(onp.s4_forward_ssm(r["u"], r["A_real"], r["A_imag"], r["B"], r["C"], r["D"]), r["y"],
                       rtol=1e-6, atol=1e-7)


def test_golden_mamba(golden):
    e = golden("mamba_exported_cfg0.npz")
    assert np.allclose(cbind.mamba_exported(e["x"], e["wg"], e["bg"], e["wo"], e["bo"]), e["y"], rtol=1e-6, atol=1e-6)
    g = golden("mamba_block_cfg0.npz")
    w = synth.mamba_block_weights(0, 64, 16, 4, 2)
    x = synth.uniform(0, "x", (1, 100, 64), -1, 1)
    assert abs(float(x.astype(np.float64).sum()) - float(g["x_sum"])) < 1e-9  # the seeded streams have not moved
    assert np.allclose(cbind.mamba_block(x, w, 16, 4), g["y"], rtol=1e-5, atol=1e-6)


# ---- builder-derived known answers: the reference holds no numeric fixture for forward_ssm, so this one is derived
# here from the text of crates/nn/src/ssm.rs:103-186 with exact rational arithmetic and an explicit model of fp32
# rounding (round to nearest even, 24-bit significand), independent of numpy's and C's float types.
def _rn32(q):
    """The fp32 value nearest to the rational q (ties to even), as a Fraction.  Normal range only."""
    from fractions import Fraction
    if q == 0:
        return Fraction(0)
    s, a = (1 if q > 0 else -1), abs(q)
    e = 0
    while a >= 2:
        a /= 2
        e += 1
    while a < 1:
        a *= 2
        e -= 1
    m = a * (1 << 23)                      # significand in [2^23, 2^24)
    lo = m.numerator // m.denominator
    rem = m - lo
    if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and lo % 2 == 1):
        lo += 1
    return s * Fraction(lo, 1 << 23) * (Fraction(2) ** e)


def test_forward_ssm_builder_derived_known_answer():
    from fractions import Fraction as Fr
    M, N, L = 2, 2, 3
    A_re, A_im = [Fr(0), Fr(0)], [Fr(0), Fr(0)]          # a = exp(0) * cos(0) = 1 exactly (ssm.rs:113-125)
    Bm = [[Fr(1), Fr(0)], [Fr(3), Fr(2)]]                 # [N, M]
    Cm = [[Fr(1), Fr(1)], [Fr(2), Fr(-1)]]                # [M, N]
    Dv = [Fr(1, 2), Fr(1, 4)]
    u = [[Fr(1), Fr(2), Fr(4)], [Fr(1), Fr(0), Fr(-3)]]   # [M, L]
    dt = _rn32(Fr(1, 10))                                 # the f32 literal 0.1 (ssm.rs:151)
    assert dt == Fr(13421773, 1 << 27)
    a = [Fr(1), Fr(1)]
    Bd = [[_rn32(dt * b) for b in row] for row in Bm]     # B.mul_scalar(dt) (ssm.rs:130)
    state = [Fr(0)] * N
    want = []
    for t in range(L):
        ut = [u[m][t] for m in range(M)]
        bu = []
        for n in range(N):                                # B_d.matmul(u_t): k ascending, product then sum rounded
            acc = Fr(0)
            for m in range(M):
                acc = _rn32(acc + _rn32(Bd[n][m] * ut[m]))
            bu.append(acc)
        state = [_rn32(_rn32(a[n] * state[n]) + bu[n]) for n in range(N)]   # ssm.rs:172-174
        row = []
        for m in range(M):                                # C.matmul(state) + D.mul(u_t) (ssm.rs:177-179)
            acc = Fr(0)
            for n in range(N):
                acc = _rn32(acc + _rn32(Cm[m][n] * state[n]))
            row.append(_rn32(acc + _rn32(Dv[m] * ut[m])))
        want.append(row)
    want = np.array([[float(v) for v in row] for row in want], np.float32)  # exact: every entry is an fp32 value
    f = lambda rows: np.array([[float(v) for v in r] for r in rows], np.float32)
    args = (f(u), np.zeros(N, np.float32), np.zeros(N, np.float32), f(Bm), f(Cm), np.array([float(v) for v in Dv], np.float32))
    got_c = cbind.s4_forward_ssm(*args, 0.1)              # buffer [L, M] (time-major: the stack quirk)
    got_np = onp.s4_forward_ssm(*args, 0.1)
    assert got_c.shape == (L, M)
    assert np.array_equal(got_c, want) and np.array_equal(np.asarray(got_np, np.float32).reshape(L, M), want)
    # a spot value a reader can check by hand: step 0, channel 0 = C[0].state + D[0] u[0] with
    # state = [0.1f, rn(rn(0.3f) + 0.2f)] = [0.1f, 0.5f']
    assert want[0, 0] == np.float32(np.float32(np.float32(0.1) + np.float32(np.float32(np.float32(0.1) * 3) + np.float32(0.2))) + np.float32(0.5))


def test_tensor_primitive_restatement():
    """oracle_np.t_*: the reference's two known answers, the stack layout quirk, and the matmul twin."""
    assert np.array_equal(onp.t_binary("add", np.ones((2, 3)), np.ones((2, 3))), np.full((2, 3), 2, np.float32))
    a, b = synth.normal(9, "a", (5, 17)), synth.normal(9, "b", (17, 6))
    assert np.array_equal(onp.t_matmul(a, b), cbind.matmul(a, b))
    assert np.array_equal(onp.t_matmul(np.ones((2, 3)), np.ones((3, 4))), np.full((2, 4), 3, np.float32))
    buf, label = onp.t_stack([np.arange(3, dtype=np.float32), np.arange(3, 6, dtype=np.float32)], 1)
    assert label == (3, 2) and np.array_equal(buf.reshape(-1), np.arange(6, dtype=np.float32))
    assert np.array_equal(onp.t_unary("sign", np.array([0.0, -0.0, 2.0, -3.0], np.float32)), np.array([1, -1, 1, -1], np.float32))
    with pytest.raises(ValueError):
        onp.t_slice(np.zeros((2, 2, 2)), [0, 0, 0], [1, 1, 1])
