"""GPU parity of the other kernels on the path (S4 recurrences, conv, GEMMs, RMSNorm, embedding, the
whole Mamba block) against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from conftest import BF16_TOL, FP32_TOL, fp32_tol_err, rel_l2, to_dev, to_np
from helixml_b200 import synth
from oracle import cbind

pytestmark = pytest.mark.gpu


def _status_ok():
    from helixml_b200 import _lib
    assert _lib.device_status() == 0, "a bounded device-side wait ran out"


# ------------------------------------------------------------------ S4
@pytest.mark.parametrize("B,L,D,N", [(2, 61, 10, 64), (1, 7, 3, 16), (3, 200, 40, 64), (1, 130, 5, 100), (2, 9, 33, 1)])
def test_s4_diag(B, L, D, N):
    from helixml_b200 import ops
    s = synth.s4_inputs(1, B, L, D, N)
    got = ops.s4_diag(*(to_dev(s[k]) for k in ("u", "A", "B", "C", "delta", "D")))
    ref = cbind.s4_diag(s["u"], s["A"], s["B"], s["C"], s["delta"], s["D"])
    assert fp32_tol_err(to_np(got), ref) <= FP32_TOL


def test_s4_diag_config1_full():
    """Benchmark configuration 1 at full size: batch 8, L 2048, d_model 256, d_state 64, f32, seed 1."""
    from helixml_b200 import ops
    s = synth.s4_inputs(1, 8, 2048, 256, 64)
    got = ops.s4_diag(*(to_dev(s[k]) for k in ("u", "A", "B", "C", "delta", "D")))
    ref = cbind.s4_diag(s["u"], s["A"], s["B"], s["C"], s["delta"], s["D"])
    assert fp32_tol_err(to_np(got), ref) <= FP32_TOL


def test_s4_diag_golden(golden):
    from helixml_b200 import ops
    g = golden("s4_diag_small.npz")
    got = ops.s4_diag(*(to_dev(g[k]) for k in ("u", "A", "B", "C", "delta", "D")))
    assert fp32_tol_err(to_np(got), g["y"]) <= FP32_TOL


@pytest.mark.parametrize("M,L,N", [(12, 45, 16), (64, 64, 16), (256, 300, 64), (5, 1, 8)])
def test_s4_reference_literal(M, L, N):
    """nn::ssm::S4Block::forward_ssm (crates/nn/src/ssm.rs:138-186): [d_model, L] in, time-major [L, d_model] out."""
    from helixml_b200 import ops
    r = {"u": synth.normal(21, "u", (M, L)), "A_real": synth.uniform(21, "Ar", (N,), -0.5, 0.0),
         "A_imag": synth.normal(21, "Ai", (N,)), "B": synth.normal(21, "B", (N, M), 0, 0.1),
         "C": synth.normal(21, "C", (M, N), 0, 0.1), "D": synth.normal(21, "D", (M,), 0, 0.5)}
    got = ops.s4_ref_forward_ssm(*(to_dev(r[k]) for k in ("u", "A_real", "A_imag", "B", "C", "D")))
    ref = cbind.s4_forward_ssm(r["u"], r["A_real"], r["A_imag"], r["B"], r["C"], r["D"])
    assert got.shape == (L, M)
    assert fp32_tol_err(to_np(got), ref) <= FP32_TOL


def test_s4_reference_literal_golden(golden):
    from helixml_b200 import ops
    g = golden("s4_ref_small.npz")
    got = ops.s4_ref_forward_ssm(*(to_dev(g[k]) for k in ("u", "A_real", "A_imag", "B", "C", "D")))
    assert fp32_tol_err(to_np(got), g["y"]) <= FP32_TOL


# ------------------------------------------------------------------ conv, norm, embedding, silu
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("B,L,D,K", [(2, 50, 64, 4), (1, 3, 24, 4), (3, 17, 7, 2), (1, 100, 128, 3)])
def test_conv1d_silu(dtype, B, L, D, K):
    from helixml_b200 import ops
    x = synth.normal(51, "x", (B, L, D))
    w = synth.uniform(51, "w", (D, K), -0.5, 0.5)
    b = synth.uniform(51, "b", (D,), -0.2, 0.2)
    if dtype == "bf16":
        x = synth.round_bf16(x)
    got = ops.conv1d_silu(to_dev(x, "bf16" if dtype == "bf16" else None), to_dev(w), to_dev(b))
    ref = cbind.conv_silu(x, w, b)
    if dtype == "bf16":
        assert rel_l2(to_np(got), ref) <= BF16_TOL
    else:
        assert fp32_tol_err(to_np(got), ref) <= FP32_TOL


@pytest.mark.parametrize("B,L,E,NO", [(1, 128, 64, 16), (2, 300, 128, 80), (1, 5, 64, 40), (3, 1000, 1536, 80), (1, 257, 256, 256),
                                      (2, 131, 192, 8), (20, 1000, 64, 24)])   # the last: enough tiles for the 128-step form
def test_conv_silu_and_x_proj_in_one_kernel(B, L, E, NO):
    """hx_conv1d_silu_xproj_fwd (the conv's tile of u is the tensor core's A operand) against the oracle's conv + SiLU
    and Linear, with x a strided half of a wider buffer as in the block; u must equal the conv kernel's bit for bit.
    Sequence lengths that are not multiples of the tile (64 steps on short grids, 128 otherwise) and output widths
    that are not multiples of 16 are among the cases."""
    import torch
    from helixml_b200 import ops
    xz = synth.round_bf16(synth.normal(67, "xz", (B, L, 2 * E)))
    cw = synth.uniform(67, "cw", (E, 4), -0.5, 0.5)
    cb = synth.normal(67, "cb", (E,), 0, 0.1)
    wx = synth.round_bf16(synth.normal(67, "wx", (NO, E), 0, 0.05))
    xz_d = to_dev(xz, "bf16")
    x_d = xz_d[:, :, :E]
    u = torch.full((B, L, E), 7.0, device="cuda", dtype=torch.bfloat16)
    xd = torch.full((B, L, NO), 7.0, device="cuda", dtype=torch.bfloat16)
    ops.conv1d_silu_xproj(x_d, to_dev(cw), to_dev(cb), to_dev(wx, "bf16"), out_u=u, out_xdbl=xd)
    _status_ok()
    u_ref = cbind.conv_silu(np.ascontiguousarray(xz[:, :, :E]), cw, cb)
    assert rel_l2(to_np(u), u_ref) <= BF16_TOL
    u_sep = ops.conv1d_silu(x_d, to_dev(cw), to_dev(cb))
    assert torch.equal(u, u_sep)
    # x_dbl from the bf16 u the kernel itself produced: fp32 accumulation leaves only the output rounding
    ub = to_np(u).astype(np.float64).reshape(B * L, E)
    ref = (ub @ wx.astype(np.float64).T).reshape(B, L, NO)
    assert rel_l2(to_np(xd), ref) <= 5e-3
    # without a bias
    u2, xd2 = ops.conv1d_silu_xproj(x_d, to_dev(cw), None, to_dev(wx, "bf16"))
    _status_ok()
    assert torch.equal(u2, ops.conv1d_silu(x_d, to_dev(cw), None))


def test_conv_silu_and_x_proj_rejects_what_it_does_not_take():
    import torch
    from helixml_b200 import _lib, ops
    x = torch.zeros(1, 16, 96, device="cuda", dtype=torch.bfloat16)   # d_inner not a multiple of 64
    with pytest.raises(_lib.HxError) as e:
        ops.conv1d_silu_xproj(x, torch.zeros(96, 4, device="cuda"), None, torch.zeros(16, 96, device="cuda", dtype=torch.bfloat16))
    assert e.value.variant == "UnsupportedOperation"
    x = torch.zeros(1, 16, 64, device="cuda", dtype=torch.bfloat16)   # three taps
    with pytest.raises(_lib.HxError) as e:
        ops.conv1d_silu_xproj(x, torch.zeros(64, 3, device="cuda"), None, torch.zeros(16, 64, device="cuda", dtype=torch.bfloat16))
    assert e.value.variant == "UnsupportedOperation"


def test_rmsnorm_and_residual():
    import torch
    from helixml_b200 import ops
    x = synth.normal(52, "x", (37, 96))
    w = synth.uniform(52, "w", (96,), 0.5, 1.5)
    ref = cbind.rmsnorm(x, w, 1e-5)
    assert fp32_tol_err(to_np(ops.rmsnorm(to_dev(x), to_dev(w), 1e-5)), ref) <= FP32_TOL
    res = synth.normal(52, "res", (37, 96))
    r = to_dev(res)
    y = ops.rmsnorm(to_dev(synth.round_bf16(x), "bf16"), to_dev(w), 1e-5, residual=r, out_dtype=torch.bfloat16)
    summed = res + synth.round_bf16(x)
    assert np.allclose(to_np(r), summed, atol=1e-6)
    assert rel_l2(to_np(y), cbind.rmsnorm(summed, w, 1e-5)) <= BF16_TOL


def test_embedding_and_silu():
    import torch
    from helixml_b200 import ops
    emb = synth.normal(53, "emb", (256, 48), 0, 0.02)
    tok = synth.random_bytes(53, "tok", (3, 21))
    out = ops.embedding(to_dev(tok), to_dev(emb))
    assert np.array_equal(to_np(out), emb[tok])
    # bf16 table: the 8-elements-per-thread path (fp32 and bf16 out) and the scalar one (row length not a multiple of 8)
    for d in (48, 44):
        embq = synth.round_bf16(synth.normal(53, "embq", (256, d), 0, 0.02))
        for od in (torch.float32, torch.bfloat16):
            got = ops.embedding(to_dev(tok), to_dev(embq, "bf16"), out_dtype=od)
            assert np.array_equal(to_np(got), embq[tok])
    x = synth.normal(53, "x", (1000,))
    assert fp32_tol_err(to_np(ops.silu(to_dev(x))), cbind.silu(x)) <= FP32_TOL


# ------------------------------------------------------------------ GEMMs
@pytest.mark.parametrize("M,N,K", [(100, 128, 64), (37, 50, 19), (1, 1, 1), (300, 80, 1536 // 8)])
def test_gemm_simt_f32(M, N, K):
    from helixml_b200 import ops
    a, w, b = synth.normal(61, "a", (M, K)), synth.normal(61, "w", (N, K), 0, 0.1), synth.normal(61, "b", (N,))
    got = ops.gemm(to_dev(a), to_dev(w), to_dev(b), tensor_cores=False)
    assert fp32_tol_err(to_np(got), cbind.linear(a, w, b)) <= FP32_TOL


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 128), (1000, 3072, 768), (513, 80, 1536), (300, 1536, 48),
                                   (70, 768, 1536), (4096, 256, 768), (129, 136, 72)])
def test_gemm_tcgen05_bf16(M, N, K):
    """The tensor-core GEMM against the oracle's Linear on bf16-exact operands; fp32 accumulation
    leaves only the output rounding."""
    import torch
    from helixml_b200 import ops
    a = synth.round_bf16(synth.normal(62, "a", (M, K)))
    w = synth.round_bf16(synth.normal(62, "w", (N, K), 0, 0.05))
    got32 = ops.gemm(to_dev(a, "bf16"), to_dev(w, "bf16"), out_dtype=torch.float32)
    _status_ok()
    ref = (a.astype(np.float64) @ w.astype(np.float64).T)
    assert fp32_tol_err(to_np(got32), ref) <= FP32_TOL
    got16 = ops.gemm(to_dev(a, "bf16"), to_dev(w, "bf16"))
    _status_ok()
    assert rel_l2(to_np(got16), ref) <= 5e-3


@pytest.mark.parametrize("M,N,K,lda", [(500, 1536, 48, 80), (130, 200, 8, 8), (40000, 64, 64, 64), (100000, 72, 24, 40), (65, 1536, 48, 48),
                                       (4097, 136, 56, 56)])
def test_gemm_short_inner_dimension_bf16(M, N, K, lda):
    """K <= 64 with a bf16 result goes to the store-shaped kernel (the dt_proj shape): A as a column slice of a wider
    row (the x_proj output), ragged row and column counts, both CTA heights."""
    from helixml_b200 import ops
    wide = synth.round_bf16(synth.normal(65, "a", (M, lda)))
    w = synth.round_bf16(synth.normal(65, "w", (N, K), 0, 0.2))
    got = ops.gemm(to_dev(wide, "bf16")[:, :K], to_dev(w, "bf16"))
    _status_ok()
    ref = wide[:, :K].astype(np.float64) @ w.astype(np.float64).T
    g = to_np(got)
    assert rel_l2(g, ref) <= 5e-3
    # every element is the correctly rounded fp32-accumulated product: within one bf16 step of the exact value
    assert np.max(np.abs(g - ref) / (np.abs(ref) + 1e-2)) <= 2.0 ** -7


def test_gemm_tcgen05_bias_epilogue_and_strides():
    import torch
    from helixml_b200 import _lib, ops
    M, N, K = 200, 96, 48
    wide = synth.round_bf16(synth.normal(63, "a", (M, 80)))
    w = synth.round_bf16(synth.normal(63, "w", (N, K), 0, 0.1))
    b = synth.normal(63, "b", (N,))
    a_dev = to_dev(wide, "bf16")[:, :K]  # a column slice: lda = 80
    got = ops.gemm(a_dev, to_dev(w, "bf16"), to_dev(b), out_dtype=torch.float32, epilogue=_lib.EPI_SOFTPLUS)
    _status_ok()
    lin = wide[:, :K].astype(np.float64) @ w.astype(np.float64).T + b
    ref = np.where(lin > 20, lin, np.log1p(np.exp(lin)))
    assert fp32_tol_err(to_np(got), ref) <= FP32_TOL
    with pytest.raises(_lib.HxError) as e:
        ops.gemm(to_dev(wide, "bf16")[:, :44], to_dev(w, "bf16")[:, :44].contiguous())
    assert e.value.variant == "UnsupportedOperation"


@pytest.mark.parametrize("M,N,K", [(1, 8, 32), (16, 3072, 768), (17, 80, 1536), (32, 768, 1536), (33, 50, 64), (64, 256, 768),
                                   (7, 7, 96), (32, 3072, 768)])
def test_gemm_few_rows_bf16(M, N, K):
    """M <= 64 and K a multiple of 32 go to the weight-streaming kernel (the decode-step shapes)."""
    import torch
    from helixml_b200 import _lib, ops
    a = synth.round_bf16(synth.normal(64, "a", (M, K)))
    w = synth.round_bf16(synth.normal(64, "w", (N, K), 0, 0.05))
    b = synth.normal(64, "b", (N,))
    ref = a.astype(np.float64) @ w.astype(np.float64).T
    got32 = ops.gemm(to_dev(a, "bf16"), to_dev(w, "bf16"), out_dtype=torch.float32)
    assert fp32_tol_err(to_np(got32), ref) <= FP32_TOL
    got16 = ops.gemm(to_dev(a, "bf16"), to_dev(w, "bf16"))
    assert rel_l2(to_np(got16), ref) <= 5e-3
    # bias + SiLU epilogue, A as a column slice of a wider matrix (lda > K)
    wide = synth.round_bf16(synth.normal(64, "wide", (M, K + 40)))
    lin = wide[:, :K].astype(np.float64) @ w.astype(np.float64).T + b
    got = ops.gemm(to_dev(wide, "bf16")[:, :K], to_dev(w, "bf16"), to_dev(b), out_dtype=torch.float32, epilogue=_lib.EPI_SILU)
    assert fp32_tol_err(to_np(got), lin / (1 + np.exp(-lin))) <= FP32_TOL
    _status_ok()


@pytest.mark.parametrize("M", [300, 20])
def test_gemm_activation_on_a_column_range(M):
    """hx_gemm_bf16_cols: [x | silu(z)] in one pass, the activation starting at a column that is a multiple of 32
    (both the tensor-memory kernel and the few-rows kernel)."""
    import torch
    from helixml_b200 import _lib, ops
    N, K, first = 320, 64, 96
    a = synth.round_bf16(synth.normal(66, "a", (M, K)))
    w = synth.round_bf16(synth.normal(66, "w", (N, K), 0, 0.2))
    lin = a.astype(np.float64) @ w.astype(np.float64).T
    ref = lin.copy()
    ref[:, first:] = lin[:, first:] / (1 + np.exp(-lin[:, first:]))
    for epi, tol in ((_lib.EPI_SILU, FP32_TOL), (_lib.EPI_SILU_FAST, 2e-3)):
        got = ops.gemm(to_dev(a, "bf16"), to_dev(w, "bf16"), out_dtype=torch.float32, epilogue=epi, epilogue_first_col=first)
        assert fp32_tol_err(to_np(got), ref) <= tol
    _status_ok()
    with pytest.raises(_lib.HxError) as e:
        ops.gemm(to_dev(a, "bf16"), to_dev(w, "bf16"), epilogue=_lib.EPI_SILU, epilogue_first_col=40)
    assert e.value.variant == "InvalidInput"


@pytest.mark.parametrize("M,N,K", [(300, 768, 1536), (129, 136, 72), (4096, 256, 768), (40, 768, 64), (513, 80, 1536),
                                   (8192, 768, 256)])   # the last: narrow tiles chosen for a fuller last wave
def test_gemm_accumulates_into_fp32(M, N, K):
    """C += A W^T: the epilogue adds its tiles into C (TMA reduce on the tensor-core path, plain read-modify-write
    on the few-rows and unaligned paths); twice in a row to see that nothing is overwritten."""
    import torch
    from helixml_b200 import ops
    a = synth.round_bf16(synth.normal(65, "a", (M, K)))
    w = synth.round_bf16(synth.normal(65, "w", (N, K), 0, 0.05))
    c0 = synth.normal(65, "c", (M, N))
    c = to_dev(c0)
    ops.gemm_acc(to_dev(a, "bf16"), to_dev(w, "bf16"), c)
    prod = a.astype(np.float64) @ w.astype(np.float64).T
    assert fp32_tol_err(to_np(c), c0 + prod) <= FP32_TOL
    ops.gemm_acc(to_dev(a, "bf16"), to_dev(w, "bf16"), c)
    assert fp32_tol_err(to_np(c), c0 + 2 * prod) <= FP32_TOL
    _status_ok()
    # an accumulator whose rows are not 16-byte aligned takes the plain-store path
    wide = torch.zeros(M, N + 3, device="cuda")
    view = wide[:, 1:N + 1]
    view.copy_(to_dev(c0))
    ops.gemm_acc(to_dev(a, "bf16"), to_dev(w, "bf16"), view)
    assert fp32_tol_err(to_np(view), c0 + prod) <= FP32_TOL
    assert float(wide[:, 0].abs().max()) == 0.0 and float(wide[:, N + 1:].abs().max()) == 0.0


@pytest.mark.parametrize("M,N,K", [(512, 256, 64), (1000, 3072, 768), (777, 768, 1536), (2178, 520, 200), (4096, 256, 768),
                                   (20000, 768, 1536)])
def test_gemm_cta_pairs_match_single_ctas(M, N, K):
    """The CTA-pair form of the tensor-core kernel (tcgen05.mma.cta_group::2 on [256 x 256] tiles, each CTA loading
    half of the W tile) against the oracle's Linear, and bit for bit against single CTAs: every element is the same
    k-ascending sum in tensor memory, whichever CTA holds it.  Row counts that leave the second CTA of the last pair
    partly or wholly out of range are among the cases."""
    import torch
    from helixml_b200 import ops
    assert ops.gemm_pair_mode(-1) > 0, "the pair kernel cannot be resident on this device"
    a = synth.round_bf16(synth.normal(66, "a", (M, K)))
    w = synth.round_bf16(synth.normal(66, "w", (N, K), 0, 0.05))
    c0 = synth.normal(66, "c", (M, N))
    ad, wd = to_dev(a, "bf16"), to_dev(w, "bf16")
    ref = a.astype(np.float64) @ w.astype(np.float64).T
    got = {}
    try:
        for mode in (2, 0):
            ops.gemm_pair_mode(mode)
            c = to_dev(c0)
            ops.gemm_acc(ad, wd, c)
            got[mode] = (ops.gemm(ad, wd, out_dtype=torch.float32), ops.gemm(ad, wd), c)
            _status_ok()
    finally:
        ops.gemm_pair_mode(1)
    assert fp32_tol_err(to_np(got[2][0]), ref) <= FP32_TOL
    assert rel_l2(to_np(got[2][1]), ref) <= 5e-3
    assert fp32_tol_err(to_np(got[2][2]), c0 + ref) <= FP32_TOL
    for x, y in zip(got[2], got[0]):
        assert torch.equal(x, y)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_mamba_block_adds_into_residual(dtype):
    """With a residual stream the block's output is added into it (out_proj epilogue on the bf16 path)."""
    import torch
    from helixml_b200 import ops
    bf = dtype == "bf16"
    B, L, M = 2, 90, 128
    w = synth.mamba_block_weights(8, M, 16, 4, 2)
    big = ("W_in", "W_x", "W_dt", "W_out")
    wq = {k: (synth.round_bf16(v) if (bf and k in big) else v) for k, v in w.items()}
    x = synth.normal(8, "x", (B, L, M))
    if bf:
        x = synth.round_bf16(x)
    r0 = synth.normal(8, "r", (B, L, M))
    dev = {k: to_dev(v, "bf16" if (bf and k in big) else None) for k, v in wq.items()}
    resid = to_dev(r0)
    ops.mamba_block(to_dev(x, "bf16" if bf else None), dev, 16, 4, residual=resid)
    _status_ok()
    ref = r0 + cbind.mamba_block(x, wq, 16, 4)
    if bf:
        assert rel_l2(to_np(resid) - r0, ref - r0) <= BF16_TOL
    else:
        assert fp32_tol_err(to_np(resid), ref) <= FP32_TOL


def test_pipe_probes_report_plausible_rates():
    """hx_probe_pipe: the rates the benchmark divides by.  A B200 retires about 128 fp32 FMAs and 16 ex2 results per
    clock and SM; anything within a factor of two of that on the device under test is accepted, and the packed form
    must not be slower per lane than the scalar one."""
    import torch
    from helixml_b200 import _lib, ops
    props = torch.cuda.get_device_properties(0)
    per_clk = props.multi_processor_count * 1.0e9  # at 1 GHz; real clocks are 1.5-2 GHz
    fma, fma2, ex2 = ops.probe_pipe("fma"), ops.probe_pipe("fma2"), ops.probe_pipe("ex2")
    assert 64 * per_clk < fma < 2 * 128 * 2.2 * per_clk
    assert 8 * per_clk < ex2 < 2 * 16 * 2.2 * per_clk
    assert fma2 >= 0.9 * fma
    with pytest.raises(_lib.HxError):
        ops.probe_pipe("fma3")


def test_four_threads_call_concurrently():
    """The reference's 4-thread concurrent matmul test (crates/backend-cpu/tests/integration_tests.rs:68-99) at this
    boundary: four host threads, each on its own stream, run the tensor-core GEMM and the fused scan at the same
    time; every result must equal the single-threaded one."""
    import threading
    import torch
    from helixml_b200 import _lib, ops
    a = to_dev(synth.round_bf16(synth.normal(67, "a", (700, 256))), "bf16")
    w = to_dev(synth.round_bf16(synth.normal(67, "w", (384, 256), 0, 0.05)), "bf16")
    inp = synth.scan_inputs(67, 2, 300, 256, 16, 4, bf16=True)
    dev = {k: to_dev(v, "bf16" if k in ("x", "dt", "z", "B", "C") else None) for k, v in inp.items()}

    def work():
        c = ops.gemm(a, w)
        y = ops.selective_scan(dev["x"], dev["dt"], dev["A"], dev["B"], dev["C"], D=dev["D"], z=dev["z"], conv_w=dev["conv_w"],
                               variant=_lib.SCAN_DIRECT, seq_splits=2)
        return c, y

    want_c, want_y = work()
    torch.cuda.synchronize()
    results, errors = [None] * 4, []

    def run(i):
        try:
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                for _ in range(5):
                    results[i] = work()
            st.synchronize()
        except Exception as e:  # pragma: no cover - reported below
            errors.append(e)

    threads = [threading.Thread(target=run, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    _status_ok()
    for c, y in results:
        assert torch.equal(c, want_c) and torch.equal(y, want_y)


# ------------------------------------------------------------------ the whole block
def test_mamba_block_config0_f32(golden):
    """Benchmark configuration 0: batch 1, L 100, d_model 64, d_state 16, expand 2, conv 4, f32, seed 0."""
    from helixml_b200 import ops
    w = synth.mamba_block_weights(0, 64, 16, 4, 2)
    x = synth.uniform(0, "x", (1, 100, 64), -1, 1)
    got = ops.mamba_block(to_dev(x), {k: to_dev(v) for k, v in w.items()}, 16, 4)
    _status_ok()
    ref = cbind.mamba_block(x, w, 16, 4)
    assert fp32_tol_err(to_np(got), ref) <= FP32_TOL
    assert fp32_tol_err(to_np(got), golden("mamba_block_cfg0.npz")["y"]) <= FP32_TOL


@pytest.mark.parametrize("B,L,M", [(2, 64, 128), (1, 300, 768)])
def test_mamba_block_bf16(B, L, M):
    from helixml_b200 import ops
    w = synth.mamba_block_weights(3, M, 16, 4, 2, init="0.02" if M == 768 else "kaiming")
    big = ("W_in", "W_x", "W_dt", "W_out")
    wq = {k: (synth.round_bf16(v) if k in big else v) for k, v in w.items()}
    x = synth.round_bf16(synth.normal(3, "x", (B, L, M)))
    dev = {k: to_dev(v, "bf16" if k in big else None) for k, v in wq.items()}
    got = ops.mamba_block(to_dev(x, "bf16"), dev, 16, 4)
    _status_ok()
    ref = cbind.mamba_block(x, wq, 16, 4)
    assert rel_l2(to_np(got), ref) <= BF16_TOL


def test_mamba_block_bf16_direct_scan_with_fused_dt():
    """The block with the one-lane-per-channel scan forced: the dt projection then runs inside the scan kernel."""
    from helixml_b200 import _lib, ops
    B, L, M = 2, 200, 768
    w = synth.mamba_block_weights(5, M, 16, 4, 2, init="0.02")
    big = ("W_in", "W_x", "W_dt", "W_out")
    wq = {k: (synth.round_bf16(v) if k in big else v) for k, v in w.items()}
    x = synth.round_bf16(synth.normal(5, "x", (B, L, M)))
    dev = {k: to_dev(v, "bf16" if k in big else None) for k, v in wq.items()}
    ref = cbind.mamba_block(x, wq, 16, 4)
    outs = [to_np(ops.mamba_block(to_dev(x, "bf16"), dev, 16, 4, scan_variant=v)) for v in (_lib.SCAN_DIRECT, _lib.SCAN_TILED)]
    _status_ok()
    for got in outs:
        assert rel_l2(got, ref) <= BF16_TOL
    assert rel_l2(outs[0], outs[1]) <= 1e-2  # fused and unfused dt projection agree


@pytest.mark.parametrize("dtype,L0,steps,M", [("f32", 37, 5, 64), ("f32", 2, 4, 64), ("bf16", 150, 6, 64), ("bf16", 60, 4, 128)])
def test_mamba_block_decode_steps_continue_prefill(dtype, L0, steps, M):
    """Prefill L0 tokens keeping (h, conv window), then `steps` single-token steps: every step's output must be
    the oracle's full-sequence output at that position (the oracle has no step function: it re-runs the block
    over the longer sequence)."""
    import torch
    from helixml_b200 import ops
    B, N, K = 2, 16, 4  # d_model 128 gives dt_rank 8 and d_inner 256: the vectorised state-step kernel
    E = 2 * M
    w = synth.mamba_block_weights(7, M, N, K, 2)
    big = ("W_in", "W_x", "W_dt", "W_out")
    bf = dtype == "bf16"
    wq = {k: (synth.round_bf16(v) if (bf and k in big) else v) for k, v in w.items()}
    x = synth.uniform(7, "x", (B, L0 + steps, M), -1, 1)
    if bf:
        x = synth.round_bf16(x)
    dev = {k: to_dev(v, "bf16" if (bf and k in big) else None) for k, v in wq.items()}
    td = torch.bfloat16 if bf else torch.float32
    xd = to_dev(x, "bf16" if bf else None)
    h = torch.zeros(B, E, N, device="cuda", dtype=torch.float32)
    cs = torch.zeros(B, 3, E, device="cuda", dtype=td)
    ops.mamba_block(xd[:, :L0].contiguous(), dev, N, K, h_last=h, conv_state=cs)
    ref = cbind.mamba_block(x, wq, N, K)  # [B, L0 + steps, M]
    outs = []
    for s in range(steps):
        outs.append(to_np(ops.mamba_block_step(xd[:, L0 + s].contiguous(), dev, N, K, h, cs)))
    _status_ok()
    got = np.stack(outs, axis=1)
    if bf:
        assert rel_l2(got, ref[:, L0:]) <= BF16_TOL
    else:
        assert fp32_tol_err(got, ref[:, L0:]) <= FP32_TOL
    # the conv window now holds the last three conv inputs: a second prefill over everything gives the same state
    h2 = torch.zeros_like(h)
    cs2 = torch.zeros_like(cs)
    ops.mamba_block(xd, dev, N, K, h_last=h2, conv_state=cs2)
    tol = 2e-2 if bf else 1e-4
    assert torch.allclose(cs.float(), cs2.float(), atol=tol, rtol=tol)
    assert (h - h2).abs().max().item() <= tol * (1 + h2.abs().max().item())


@pytest.mark.parametrize("dtype,B,M", [("bf16", 2, 64), ("bf16", 33, 128), ("bf16", 5, 96), ("f32", 3, 64)])
def test_mamba_block_step_residual_form(dtype, B, M):
    """The residual form of the step (norm inside in_proj, add inside out_proj on the bf16 path) against the plain
    form fed with an explicit RMSNorm, and against the oracle's norm + block on a one-token sequence."""
    import torch
    from helixml_b200 import ops
    bf = dtype == "bf16"
    N, K = 16, 4
    E = 2 * M
    w = synth.mamba_block_weights(10, M, N, K, 2)
    big = ("W_in", "W_x", "W_dt", "W_out")
    wq = {k: (synth.round_bf16(v) if (bf and k in big) else v) for k, v in w.items()}
    dev = {k: to_dev(v, "bf16" if (bf and k in big) else None) for k, v in wq.items()}
    td = torch.bfloat16 if bf else torch.float32
    r0 = synth.normal(10, "resid", (B, M))
    nw = synth.uniform(10, "nw", (M,), 0.8, 1.2)
    h0 = synth.normal(10, "h", (B, E, N), 0, 0.1)
    c0 = synth.normal(10, "cs", (B, 3, E))
    if bf:
        c0 = synth.round_bf16(c0)
    # plain form: explicit norm, then the step, then the add
    normed = ops.rmsnorm(to_dev(r0), to_dev(nw), 1e-5, out_dtype=td)
    h_a, cs_a = to_dev(h0), to_dev(c0, "bf16" if bf else None)
    out = ops.mamba_block_step(normed, dev, N, K, h_a, cs_a)
    want = r0 + to_np(out)
    # residual form
    h_b, cs_b = to_dev(h0), to_dev(c0, "bf16" if bf else None)
    resid = to_dev(r0)
    ops.mamba_block_step(torch.empty(B, M, device="cuda", dtype=td), dev, N, K, h_b, cs_b, residual=resid, norm_w=to_dev(nw))
    _status_ok()
    got = to_np(resid)
    if bf:
        assert rel_l2(got - r0, want - r0) <= BF16_TOL
        assert rel_l2(to_np(h_b), to_np(h_a)) <= BF16_TOL and rel_l2(to_np(cs_b), to_np(cs_a)) <= BF16_TOL
    else:
        assert fp32_tol_err(got, want) <= FP32_TOL
        assert fp32_tol_err(to_np(h_b), to_np(h_a)) <= FP32_TOL and np.array_equal(to_np(cs_b), to_np(cs_a))


def test_mamba_block_step_rejects_bad_arguments():
    import torch
    from helixml_b200 import _lib, ops
    w = synth.mamba_block_weights(7, 64, 16, 4, 2)
    dev = {k: to_dev(v) for k, v in w.items()}
    x = torch.zeros(2, 64, device="cuda")
    h = torch.zeros(2, 128, 16, device="cuda")
    cs = torch.zeros(2, 3, 128, device="cuda")
    with pytest.raises(_lib.HxError) as e:
        ops.mamba_block_step(x, dev, 16, 4, h, cs, workspace=torch.empty(16, dtype=torch.uint8, device="cuda"))
    assert e.value.status == 10  # InvalidInput: workspace too small
    with pytest.raises(_lib.HxError) as e:
        ops.mamba_block_step(x, dev, 16, 5, h, cs)
    assert e.value.status == 2   # InvalidDimension: d_conv outside [1, 4]


def test_exported_reference_block(golden):
    """The exported nn::MambaBlock::forward (crates/nn/src/lib.rs:888-906) is out_proj(silu(gate(x))):
    two Linear calls and a SiLU, reproduced with the GEMM's bias and SiLU epilogue."""
    from helixml_b200 import _lib, ops
    g = golden("mamba_exported_cfg0.npz")
    h = ops.gemm(to_dev(g["x"]), to_dev(g["wg"]), to_dev(g["bg"]), epilogue=_lib.EPI_SILU, tensor_cores=False)
    y = ops.gemm(h, to_dev(g["wo"]), to_dev(g["bo"]), tensor_cores=False)
    assert fp32_tol_err(to_np(y), g["y"]) <= FP32_TOL
