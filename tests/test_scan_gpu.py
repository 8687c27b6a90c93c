"""GPU parity of the fused selective scan (through the C ABI) against the CPU oracle.

fp32 gate:  max |got - ref| / (1 + |ref|) <= 1e-4   (the chunked/packed kernels reorder sums)
bf16 gate:  relative L2 error <= 2e-2 against the fp32 oracle run on the same bf16-exact inputs."""
import numpy as np
import pytest

from conftest import BF16_TOL, FP32_TOL, fp32_tol_err, rel_l2, to_dev, to_np
from helixml_b200 import synth
from oracle import cbind

pytestmark = pytest.mark.gpu


def run_gpu(inp, dtype, *, variant, lpc=0, geom=None, gate=True, skip=True, conv=True, conv_b=None, dt_bias=None,
            softplus=True, state=False, seq_splits=0, tune=0, z_is_gate=False):
    from helixml_b200 import ops
    cast = "bf16" if dtype == "bf16" else None
    out = ops.selective_scan(
        to_dev(inp["x"], cast), to_dev(inp["dt"], cast), to_dev(inp["A"]), to_dev(inp["B"], cast), to_dev(inp["C"], cast),
        D=to_dev(inp["D"]) if skip else None, z=to_dev(inp["z"], cast) if gate else None,
        conv_w=to_dev(inp["conv_w"]) if conv else None, conv_b=to_dev(conv_b), dt_bias=to_dev(dt_bias),
        dt_softplus=softplus, variant=variant, a_geometric=geom, lanes_per_channel=lpc, return_state=state,
        seq_splits=seq_splits, tune=tune, z_is_gate=z_is_gate)
    from helixml_b200 import _lib
    assert _lib.device_status() == 0, "a bounded device-side wait ran out"
    if state:
        return to_np(out[0]), to_np(out[1])
    return to_np(out)


def run_ref(inp, *, gate=True, skip=True, conv=True, conv_b=None, dt_bias=None, softplus=True, state=False):
    return cbind.selective_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], D=inp["D"] if skip else None,
                                z=inp["z"] if gate else None, conv_w=inp["conv_w"] if conv else None, conv_b=conv_b,
                                dt_bias=dt_bias, dt_softplus=softplus, return_state=state)


def check(got, ref, dtype):
    if dtype == "bf16":
        assert rel_l2(got, ref) <= BF16_TOL
    else:
        assert fp32_tol_err(got, ref) <= FP32_TOL


SIMPLE, TILED, SEQSPLIT, DIRECT, LOOKBACK = 1, 2, 3, 4, 5


def check_blocks(got, ref, dtype, seg_len, tile=64):
    """The parity gate on every (batch row, sequence segment, channel tile) block by itself: a carry lost at one
    segment boundary of one tile changes a few thousand outputs, which a whole-tensor norm would not show."""
    B, L, D = ref.shape
    worst = 0.0
    for b in range(B):
        for t0 in range(0, L, seg_len):
            for d0 in range(0, D, tile):
                g, r = got[b, t0:t0 + seg_len, d0:d0 + tile], ref[b, t0:t0 + seg_len, d0:d0 + tile]
                worst = max(worst, rel_l2(g, r) if dtype == "bf16" else fp32_tol_err(g, r))
    assert worst <= (BF16_TOL if dtype == "bf16" else FP32_TOL), worst


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_simple_kernel(dtype):
    inp = synth.scan_inputs(31, 2, 50, 40, 16, 4, bf16=dtype == "bf16")
    got, hg = run_gpu(inp, dtype, variant=SIMPLE, state=True)
    ref, hr = run_ref(inp, state=True)
    check(got, ref, dtype)
    assert fp32_tol_err(hg, hr) <= FP32_TOL


@pytest.mark.parametrize("d_state", [1, 8, 16, 24, 64])
def test_simple_kernel_any_d_state(d_state):
    inp = synth.scan_inputs(32, 1, 33, 9, d_state, 4, bf16=False)
    check(run_gpu(inp, "f32", variant=SIMPLE), run_ref(inp), "f32")


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("lpc", [1, 2, 4])
@pytest.mark.parametrize("geom", [True, False])
def test_tiled_kernel(dtype, lpc, geom):
    # L is not a multiple of the chunk, D not a multiple of the tile
    inp = synth.scan_inputs(33, 2, 150, 72, 16, 4, bf16=dtype == "bf16")
    got, hg = run_gpu(inp, dtype, variant=TILED, lpc=lpc, geom=geom, state=True)
    ref, hr = run_ref(inp, state=True)
    check(got, ref, dtype)
    assert fp32_tol_err(hg, hr) <= FP32_TOL if dtype == "f32" else rel_l2(hg, hr) <= BF16_TOL


@pytest.mark.parametrize("dtype,cpl", [("f32", 1), ("bf16", 1), ("bf16", 2)])
@pytest.mark.parametrize("geom", [True, False])
@pytest.mark.parametrize("B,L,D", [(2, 150, 72), (1, 37, 296), (3, 16, 256)])
def test_direct_kernel(dtype, cpl, geom, B, L, D):
    # one lane per channel; L not a chunk multiple, D not a tile multiple (partly and fully empty boxes)
    inp = synth.scan_inputs(43, B, L, D, 16, 4, bf16=dtype == "bf16")
    got, hg = run_gpu(inp, dtype, variant=DIRECT, tune=cpl, geom=geom, state=True)
    ref, hr = run_ref(inp, state=True)
    check(got, ref, dtype)
    assert fp32_tol_err(hg, hr) <= FP32_TOL if dtype == "f32" else rel_l2(hg, hr) <= BF16_TOL


@pytest.mark.parametrize("cpl", [1, 2])
@pytest.mark.parametrize("geom,conv", [(True, False), (True, True), (False, False)])
@pytest.mark.parametrize("B,L,D,R", [(2, 150, 200, 48), (1, 33, 512, 16), (3, 64, 136, 64)])
def test_direct_fused_dt_projection(cpl, geom, conv, B, L, D, R):
    """dt = dt_low . W_dt^T computed inside the scan kernel (producer warp, tensor cores), with dt_low a column
    slice of a wider row as in the Mamba block.  The oracle gets the same product computed in fp32."""
    import torch
    from helixml_b200 import _lib, ops
    inp = synth.scan_inputs(44, B, L, D, 16, 4, bf16=True)
    if not geom:
        inp["A"] = -np.exp(synth.uniform(44, "Alog", (D, 16), -1.0, 2.0)).astype(np.float32)
    dt_low = synth.round_bf16(synth.normal(44, "dt_low", (B, L, R)))
    W_dt = synth.round_bf16(synth.normal(44, "W_dt", (D, R), 0.0, 0.4 / np.sqrt(R)))
    bias = synth.uniform(44, "bias", (D,), -3.0, -1.5)
    dt = (dt_low.reshape(-1, R).astype(np.float64) @ W_dt.astype(np.float64).T).reshape(B, L, D).astype(np.float32)
    ref = cbind.selective_scan(inp["x"], dt, inp["A"], inp["B"], inp["C"], D=inp["D"], z=inp["z"],
                               conv_w=inp["conv_w"] if conv else None, dt_bias=bias)
    wide = torch.zeros((B, L, R + 32), dtype=torch.bfloat16, device="cuda")
    wide[:, :, :R] = to_dev(dt_low, "bf16")
    wide[:, :, R:R + 16] = to_dev(inp["B"], "bf16")
    wide[:, :, R + 16:] = to_dev(inp["C"], "bf16")
    y = ops.selective_scan(to_dev(inp["x"], "bf16"), None, to_dev(inp["A"]), wide[:, :, R:R + 16], wide[:, :, R + 16:],
                           D=to_dev(inp["D"]), z=to_dev(inp["z"], "bf16"), conv_w=to_dev(inp["conv_w"]) if conv else None,
                           dt_bias=to_dev(bias), variant=DIRECT, tune=cpl, a_geometric=geom, dt_low=wide[:, :, :R],
                           W_dt=to_dev(W_dt, "bf16"))
    assert _lib.device_status() == 0
    assert rel_l2(to_np(y), ref) <= BF16_TOL
    # kernels without the fusion say so instead of ignoring W_dt
    with pytest.raises(_lib.HxError) as e:
        ops.selective_scan(to_dev(inp["x"], "bf16"), None, to_dev(inp["A"]), wide[:, :, R:R + 16], wide[:, :, R + 16:],
                           variant=TILED, dt_low=wide[:, :, :R], W_dt=to_dev(W_dt, "bf16"))
    assert e.value.variant == "UnsupportedOperation"


@pytest.mark.parametrize("splits", [2, 8])
def test_direct_fused_dt_projection_chained_segments(splits):
    """The fused dt projection with the sequence cut into chained segments, in the block's configuration (no conv,
    gate and softplus present, geometric A): the instantiation the byte LM runs at full size.  Gate on every
    (row, segment, tile) block, small steps so that a lost carry shows."""
    import torch
    from helixml_b200 import _lib, ops
    B, L, D, R = 3, 520, 200, 48
    inp = synth.scan_inputs(46, B, L, D, 16, 4, bf16=True)
    dt_low = synth.round_bf16(synth.normal(46, "dt_low", (B, L, R)))
    W_dt = synth.round_bf16(synth.normal(46, "W_dt", (D, R), 0.0, 0.4 / np.sqrt(R)))
    bias = synth.uniform(46, "bias", (D,), -5.0, -3.0)
    dt = (dt_low.reshape(-1, R).astype(np.float64) @ W_dt.astype(np.float64).T).reshape(B, L, D).astype(np.float32)
    ref, hr = cbind.selective_scan(inp["x"], dt, inp["A"], inp["B"], inp["C"], D=inp["D"], z=inp["z"], dt_bias=bias,
                                   return_state=True)
    wide = torch.zeros((B, L, R + 32), dtype=torch.bfloat16, device="cuda")
    wide[:, :, :R] = to_dev(dt_low, "bf16")
    wide[:, :, R:R + 16] = to_dev(inp["B"], "bf16")
    wide[:, :, R + 16:] = to_dev(inp["C"], "bf16")
    for variant in (DIRECT, LOOKBACK):
        y, h = ops.selective_scan(to_dev(inp["x"], "bf16"), None, to_dev(inp["A"]), wide[:, :, R:R + 16], wide[:, :, R + 16:],
                                  D=to_dev(inp["D"]), z=to_dev(inp["z"], "bf16"), dt_bias=to_dev(bias), variant=variant,
                                  a_geometric=True, dt_low=wide[:, :, :R], W_dt=to_dev(W_dt, "bf16"), seq_splits=splits,
                                  return_state=True)
        assert _lib.device_status() == 0
        seg = -(-(-(-L // splits)) // 32) * 32
        check_blocks(to_np(y), ref, "bf16", seg, tile=128)
        assert rel_l2(to_np(h), hr) <= BF16_TOL


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("splits", [2, 3, 5, 8])
@pytest.mark.parametrize("conv", [True, False])
def test_lookback_parallel_segments(dtype, splits, conv):
    """HX_SCAN_LOOKBACK: the segments of a chain run at the same time (aggregate pass, then look-back + output
    pass).  L is neither a multiple of the segment nor of the chunk, D not a multiple of the tile, steps are small
    so that the state carries across every boundary; gate on every (row, segment, tile) block and on the final
    state, and agreement with the one-pass kernel."""
    inp = synth.scan_inputs(47, 2, 333, 168, 16, 4, bf16=dtype == "bf16")
    inp["dt"] -= 2.0
    if dtype == "bf16":
        inp["dt"] = synth.round_bf16(inp["dt"])
    got, hg = run_gpu(inp, dtype, variant=LOOKBACK, seq_splits=splits, geom=True, state=True, conv=conv)
    ref, hr = run_ref(inp, state=True, conv=conv)
    seg = -(-(-(-333 // splits)) // 32) * 32
    check_blocks(got, ref, dtype, seg)
    check(hg, hr, dtype)
    one = run_gpu(inp, dtype, variant=DIRECT, geom=True, conv=conv)
    assert (fp32_tol_err(got, one) <= FP32_TOL) if dtype == "f32" else (rel_l2(got, one) <= 1e-2)


def test_lookback_optional_terms_and_single_segment():
    inp = synth.scan_inputs(48, 2, 200, 64, 16, 4, bf16=False)
    inp["dt"] -= 1.5
    cb = synth.uniform(48, "cb", (64,), -0.3, 0.3)
    db = synth.uniform(48, "db", (64,), -1.0, 0.5)
    # no gate, no skip, conv bias and dt bias
    ref = run_ref(inp, gate=False, skip=False, conv_b=cb, dt_bias=db)
    check_blocks(run_gpu(inp, "f32", variant=LOOKBACK, seq_splits=4, geom=True, gate=False, skip=False, conv_b=cb, dt_bias=db),
                 ref, "f32", 64)
    # dt used as given (no softplus)
    raw = dict(inp)
    raw["dt"] = np.abs(inp["dt"]) * 0.02
    check_blocks(run_gpu(raw, "f32", variant=LOOKBACK, seq_splits=3, geom=True, softplus=False), run_ref(raw, softplus=False),
                 "f32", 96)
    # a sequence shorter than one planning chunk is a single segment: plain one-pass kernel
    short = synth.scan_inputs(49, 1, 20, 32, 16, 4, bf16=False)
    check(run_gpu(short, "f32", variant=LOOKBACK, seq_splits=4, geom=True), run_ref(short), "f32")


def test_lookback_needs_geometric_decay():
    """With a general A the aggregate of a segment is not a power of one exponential: HX_SCAN_LOOKBACK says so,
    HX_SCAN_AUTO with seq_splits falls back to a kernel that handles it."""
    from helixml_b200 import _lib
    inp = synth.scan_inputs(50, 1, 300, 64, 16, 4, bf16=False)
    inp["A"] = -np.exp(synth.uniform(50, "Alog", (64, 16), -1.0, 2.0)).astype(np.float32)
    with pytest.raises(_lib.HxError) as e:
        run_gpu(inp, "f32", variant=LOOKBACK, seq_splits=4, geom=False)
    assert e.value.variant == "UnsupportedOperation"
    check(run_gpu(inp, "f32", variant=0, seq_splits=4), run_ref(inp), "f32")


def test_auto_picks_lookback_for_few_chains():
    """Few chains, geometric A, a split given: HX_SCAN_AUTO runs the look-back form (two launches of the direct
    kernel); the result is the oracle's."""
    inp = synth.scan_inputs(51, 1, 1024, 256, 16, 4, bf16=True)
    inp["dt"] = synth.round_bf16(inp["dt"] - 2.0)
    got, hg = run_gpu(inp, "bf16", variant=0, seq_splits=8, state=True)
    ref, hr = run_ref(inp, state=True)
    check_blocks(got, ref, "bf16", 128)
    check(hg, hr, "bf16")


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_tiled_general_decay(dtype):
    # an A that is not geometric: the caller's flag is 0 and every state takes its own exponential
    inp = synth.scan_inputs(34, 1, 90, 64, 16, 4, bf16=dtype == "bf16")
    inp["A"] = -np.exp(synth.uniform(34, "Alog", (64, 16), -1.0, 2.0)).astype(np.float32)
    got = run_gpu(inp, dtype, variant=TILED, lpc=4)  # geom=None: detected on the host
    check(got, run_ref(inp), dtype)


def test_geometric_detection():
    import torch
    from helixml_b200 import ops
    A = torch.from_numpy((-np.exp(synth.a_log_s4d_real(8, 16))).astype(np.float32)).cuda()
    assert ops.check_geometric(A)
    A[3, 5] *= 1.01
    assert not ops.check_geometric(A)


@pytest.mark.parametrize("L", [1, 2, 3, 4, 7, 31, 32, 33, 64])
def test_short_and_ragged_sequences(L):
    inp = synth.scan_inputs(35, 3, L, 16, 16, 4, bf16=False)
    ref = run_ref(inp)
    for variant, lpc in ((SIMPLE, 0), (TILED, 4), (TILED, 1), (DIRECT, 0)):
        check(run_gpu(inp, "f32", variant=variant, lpc=lpc), ref, "f32")


@pytest.mark.parametrize("K", [1, 2, 3, 4])
def test_conv_taps_and_biases(K):
    inp = synth.scan_inputs(36, 2, 45, 24, 16, K, bf16=False)
    cb = synth.uniform(36, "cb", (24,), -0.3, 0.3)
    db = synth.uniform(36, "db", (24,), -1.0, 1.0)
    ref = run_ref(inp, conv_b=cb, dt_bias=db)
    check(run_gpu(inp, "f32", variant=SIMPLE, conv_b=cb, dt_bias=db), ref, "f32")
    check(run_gpu(inp, "f32", variant=TILED, lpc=2, conv_b=cb, dt_bias=db), ref, "f32")
    check(run_gpu(inp, "f32", variant=DIRECT, conv_b=cb, dt_bias=db), ref, "f32")


@pytest.mark.parametrize("gate,skip,conv,softplus", [(False, True, True, True), (True, False, True, True),
                                                      (True, True, False, True), (True, True, True, False),
                                                      (False, False, False, False)])
def test_optional_terms(gate, skip, conv, softplus):
    inp = synth.scan_inputs(37, 2, 40, 32, 16, 4, bf16=False)
    if not softplus:
        inp["dt"] = np.abs(inp["dt"]) * 0.05  # dt is used as given: keep it a sane step size
    ref = run_ref(inp, gate=gate, skip=skip, conv=conv, softplus=softplus)
    for variant, lpc in ((SIMPLE, 0), (TILED, 4), (TILED, 2), (TILED, 1), (DIRECT, 0)):
        check(run_gpu(inp, "f32", variant=variant, lpc=lpc, gate=gate, skip=skip, conv=conv, softplus=softplus), ref, "f32")


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_gate_given_already_activated(dtype):
    """z_is_gate: the caller (the block's in_proj epilogue) hands silu(z) instead of z; every kernel then
    multiplies by it as it is.  The reference result is the oracle on the original z."""
    inp = synth.scan_inputs(39, 2, 70, 128, 16, 4, bf16=dtype == "bf16")
    ref = run_ref(inp)
    pre = dict(inp)
    g = inp["z"].astype(np.float64)
    g = (g / (1.0 + np.exp(-g))).astype(np.float32)
    pre["z"] = synth.round_bf16(g) if dtype == "bf16" else g
    for variant, lpc in ((SIMPLE, 0), (TILED, 2), (TILED, 4), (DIRECT, 0)):
        check(run_gpu(pre, dtype, variant=variant, lpc=lpc, z_is_gate=True), ref, dtype)


def test_softplus_identity_branch():
    inp = synth.scan_inputs(38, 1, 8, 32, 16, 4, bf16=False)
    inp["dt"][:] = np.linspace(15, 30, 8, dtype=np.float32)[None, :, None]  # crosses the v > 20 switch
    inp["A"] *= 1e-3  # keep exp(dt*A) away from zero so the check is not vacuous
    ref = run_ref(inp)
    check(run_gpu(inp, "f32", variant=TILED, lpc=4, geom=True), ref, "f32")
    binp = {k: (synth.round_bf16(v) if k in ("x", "dt", "z", "B", "C") else v) for k, v in inp.items()}
    check(run_gpu(binp, "bf16", variant=TILED, lpc=4, geom=True), run_ref(binp), "bf16")


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_strided_views(dtype):
    """x and z as the two halves of one [B, L, 2D] row, B and C as column slices of a wider row:
    the layout the Mamba block hands to the scan."""
    import torch
    from helixml_b200 import ops
    Bsz, L, D, N, R = 2, 70, 64, 16, 8
    inp = synth.scan_inputs(39, Bsz, L, D, N, 4, bf16=dtype == "bf16")
    cast = "bf16" if dtype == "bf16" else None
    xz = torch.cat([to_dev(inp["x"], cast), to_dev(inp["z"], cast)], dim=2)
    pad = torch.zeros((Bsz, L, R), dtype=xz.dtype, device="cuda")
    dbc = torch.cat([pad, to_dev(inp["B"], cast), to_dev(inp["C"], cast)], dim=2)
    ref = run_ref(inp)
    for variant in (SIMPLE, TILED, DIRECT, 0):
        y = ops.selective_scan(xz[:, :, :D], to_dev(inp["dt"], cast), to_dev(inp["A"]), dbc[:, :, R:R + N],
                               dbc[:, :, R + N:], D=to_dev(inp["D"]), z=xz[:, :, D:], conv_w=to_dev(inp["conv_w"]),
                               variant=variant)
        check(to_np(y), ref, dtype)


def test_auto_falls_back_on_unaligned_views():
    """A view whose base is not 16-byte aligned cannot go through TMA: the tiled variant reports
    UnsupportedOperation, AUTO runs the simple kernel instead."""
    import torch
    from helixml_b200 import _lib, ops
    inp = synth.scan_inputs(40, 1, 20, 16, 16, 4, bf16=False)
    wide = torch.zeros((1, 20, 17 + 16), dtype=torch.float32, device="cuda")
    wide[:, :, 1:17] = to_dev(inp["x"])
    xv = wide[:, :, 1:17]  # base offset 4 bytes, row stride 33 elements
    args = (to_dev(inp["dt"]), to_dev(inp["A"]), to_dev(inp["B"]), to_dev(inp["C"]))
    with pytest.raises(_lib.HxError) as e:
        ops.selective_scan(xv, *args, variant=TILED)
    assert e.value.variant == "UnsupportedOperation"
    y = ops.selective_scan(xv, *args, variant=0)
    ref = cbind.selective_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"])
    check(to_np(y), ref, "f32")


@pytest.mark.parametrize("dtype,lpc", [("f32", 4), ("bf16", 4), ("bf16", 1)])
@pytest.mark.parametrize("splits", [2, 3, 5])
def test_sequence_split_with_carry(dtype, lpc, splits):
    inp = synth.scan_inputs(41, 2, 300, 40, 16, 4, bf16=dtype == "bf16")
    inp["dt"] -= 2.0  # small steps: the state remembers across segment boundaries, so a lost carry would show
    if dtype == "bf16":
        inp["dt"] = synth.round_bf16(inp["dt"])
    got, hg = run_gpu(inp, dtype, variant=SEQSPLIT, lpc=lpc, seq_splits=splits, state=True)
    ref, hr = run_ref(inp, state=True)
    check(got, ref, dtype)
    check(hg, hr, dtype)
    check_blocks(got, ref, dtype, -(-(-(-300 // splits)) // 32) * 32, tile=40)
    # the one-lane-per-channel kernel with the same chained segments
    got_d, hd = run_gpu(inp, dtype, variant=DIRECT, seq_splits=splits, state=True)
    check_blocks(got_d, ref, dtype, -(-(-(-300 // splits)) // 32) * 32, tile=40)
    check(hd, hr, dtype)
    # and it is the same function as the unsplit kernel
    one = run_gpu(inp, dtype, variant=TILED, lpc=lpc)
    assert np.max(np.abs(one - got)) <= (1e-5 if dtype == "f32" else 1e-1)


def test_batch_rows_and_channels_are_independent():
    """Running a subset of batch rows / channels alone gives the same numbers (bit for bit) as the
    full launch: the property the multi-GPU sharding relies on."""
    import torch
    from helixml_b200 import ops
    inp = synth.scan_inputs(42, 4, 96, 128, 16, 4, bf16=True)
    dev = {k: to_dev(v, "bf16" if k in ("x", "dt", "z", "B", "C") else None) for k, v in inp.items()}
    full = ops.selective_scan(dev["x"], dev["dt"], dev["A"], dev["B"], dev["C"], D=dev["D"], z=dev["z"],
                              conv_w=dev["conv_w"], variant=TILED, lanes_per_channel=4)
    rows = ops.selective_scan(dev["x"][1:3], dev["dt"][1:3], dev["A"], dev["B"][1:3], dev["C"][1:3], D=dev["D"],
                              z=dev["z"][1:3], conv_w=dev["conv_w"], variant=TILED, lanes_per_channel=4)
    assert torch.equal(full[1:3], rows)
    sl = slice(64, 128)
    chans = ops.selective_scan(dev["x"][:, :, sl], dev["dt"][:, :, sl], dev["A"][sl].contiguous(), dev["B"], dev["C"],
                               D=dev["D"][sl].contiguous(), z=dev["z"][:, :, sl], conv_w=dev["conv_w"][sl].contiguous(),
                               variant=TILED, lanes_per_channel=4)
    assert torch.equal(full[:, :, sl], chans)


@pytest.mark.parametrize("name,dtype", [("scan_f32_small.npz", "f32"), ("scan_bf16_small.npz", "bf16")])
def test_golden_vectors(golden, name, dtype):
    g = golden(name)
    cb = g["conv_b"] if g["conv_b"].size else None
    db = g["dt_bias"] if g["dt_bias"].size else None
    gate = bool(int(g["gate"]))
    for variant, lpc in ((SIMPLE, 0), (TILED, 4), (TILED, 2), (TILED, 1), (DIRECT, 0)):
        got, hg = run_gpu(g, dtype, variant=variant, lpc=lpc, gate=gate, conv_b=cb, dt_bias=db, state=True)
        check(got, g["y"], dtype)
        check(hg, g["h_last"], dtype)


def test_full_size_config2_sampled_chains():
    """Benchmark configuration 2 at full size (batch 16, L 4096, d_inner 1536, bf16): the tiled kernel
    agrees with the simple kernel everywhere and with the CPU oracle on sampled (batch, channel) chains."""
    import torch
    from helixml_b200 import ops
    Bsz, L, D, N = 16, 4096, 1536, 16
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn((Bsz, L, D), device="cuda", generator=g).to(torch.bfloat16)
    z = torch.randn((Bsz, L, D), device="cuda", generator=g).to(torch.bfloat16)
    dt = (torch.rand((Bsz, L, D), device="cuda", generator=g) * 3 - 4).to(torch.bfloat16)
    Bm = torch.randn((Bsz, L, N), device="cuda", generator=g).to(torch.bfloat16)
    Cm = torch.randn((Bsz, L, N), device="cuda", generator=g).to(torch.bfloat16)
    A = to_dev((-np.exp(synth.a_log_s4d_real(D, N))).astype(np.float32))
    Dk = torch.ones(D, device="cuda")
    cw = to_dev(synth.uniform(2, "conv_w", (D, 4), -0.5, 0.5))
    outs = {}
    for lpc in (1, 2, 4):
        outs[lpc] = ops.selective_scan(x, dt, A, Bm, Cm, D=Dk, z=z, conv_w=cw, variant=TILED, lanes_per_channel=lpc)
    for cpl in (1, 2):
        outs[10 + cpl] = ops.selective_scan(x, dt, A, Bm, Cm, D=Dk, z=z, conv_w=cw, variant=DIRECT, tune=cpl)
    base = ops.selective_scan(x, dt, A, Bm, Cm, D=Dk, z=z, conv_w=cw, variant=SIMPLE)
    from helixml_b200 import _lib
    assert _lib.device_status() == 0
    for lpc, y in outs.items():
        diff = (y.float() - base.float()).norm() / base.float().norm()
        assert float(diff) <= 1e-2, (lpc, float(diff))
    rows, sl = [0, 7, 15], slice(704, 768)
    ref = cbind.selective_scan(to_np(x[rows][:, :, sl]), to_np(dt[rows][:, :, sl]), to_np(A[sl]), to_np(Bm[rows]),
                               to_np(Cm[rows]), D=to_np(Dk[sl]), z=to_np(z[rows][:, :, sl]), conv_w=to_np(cw[sl]))
    for lpc, y in outs.items():
        assert rel_l2(to_np(y[rows][:, :, sl]), ref) <= BF16_TOL


def test_config4_shard_long_sequences_sampled_chains():
    """Benchmark configuration 4 as one GPU of eight sees it (channel shard: batch 64, L 16 384, 640 channels,
    bf16, 5.4 GB): the longest sequences on the path.  AUTO (direct kernel, with and without sequence segments)
    agrees with the simple kernel everywhere and with the CPU oracle on sampled (batch, channel) chains, and the
    final states agree too."""
    import torch
    from helixml_b200 import _lib, ops
    Bsz, L, D, N = 64, 16384, 640, 16
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn((Bsz, L, D), device="cuda", generator=g).to(torch.bfloat16)
    z = torch.randn((Bsz, L, D), device="cuda", generator=g).to(torch.bfloat16)
    dt = (torch.rand((Bsz, L, D), device="cuda", generator=g) * 3 - 4).to(torch.bfloat16)
    Bm = torch.randn((Bsz, L, N), device="cuda", generator=g).to(torch.bfloat16)
    Cm = torch.randn((Bsz, L, N), device="cuda", generator=g).to(torch.bfloat16)
    A = to_dev((-np.exp(synth.a_log_s4d_real(D, N))).astype(np.float32))
    Dk = torch.ones(D, device="cuda")
    cw = to_dev(synth.uniform(4, "conv_w", (D, 4), -0.5, 0.5))
    base, hb = ops.selective_scan(x, dt, A, Bm, Cm, D=Dk, z=z, conv_w=cw, variant=SIMPLE, return_state=True)
    outs = {
        "auto": ops.selective_scan(x, dt, A, Bm, Cm, D=Dk, z=z, conv_w=cw, return_state=True),
        "direct, 4 segments": ops.selective_scan(x, dt, A, Bm, Cm, D=Dk, z=z, conv_w=cw, variant=DIRECT, seq_splits=4,
                                                 return_state=True),
    }
    assert _lib.device_status() == 0
    for name, (y, h) in outs.items():
        assert float((y.float() - base.float()).norm() / base.float().norm()) <= 1e-2, name
        assert float((h - hb).norm() / hb.norm()) <= 1e-2, name
    rows, sl = [0, 63], slice(608, 640)  # the last channels of the shard, first and last batch row
    ref = cbind.selective_scan(to_np(x[rows][:, :, sl]), to_np(dt[rows][:, :, sl]), to_np(A[sl]), to_np(Bm[rows]),
                               to_np(Cm[rows]), D=to_np(Dk[sl]), z=to_np(z[rows][:, :, sl]), conv_w=to_np(cw[sl]))
    for name, (y, _) in outs.items():
        assert rel_l2(to_np(y[rows][:, :, sl]), ref) <= BF16_TOL, name


def test_carry_wait_that_runs_out_is_reported_not_trapped():
    """A chained segment whose predecessor never publishes its carry: the bounded wait gives up (here after 2000
    polls, about 0.1 ms), the kernel records the event and returns, the host sees TensorError::BackendError through
    hx_device_check, and the next launch on the same context is clean.  The predecessor is simply not launched
    (hx_debug_scan_orphan_segment); nothing traps, faults or waits without a limit."""
    import ctypes as C
    import torch
    from helixml_b200 import _lib, ops
    inp = synth.scan_inputs(52, 1, 256, 128, 16, 4, bf16=True)
    dev = {k: to_dev(v, "bf16" if k in ("x", "dt", "z", "B", "C") else None) for k, v in inp.items()}
    y = torch.empty_like(dev["x"])
    a = _lib.ScanArgs()
    a.batch, a.seq_len, a.d_inner, a.d_state, a.d_conv = 1, 256, 128, 16, 4
    a.io_dtype, a.dt_softplus, a.variant, a.seq_splits, a.a_geometric = _lib.HX_BF16, 1, _lib.SCAN_DIRECT, 2, 1
    for name, t in (("x", dev["x"]), ("dt", dev["dt"]), ("z", dev["z"]), ("y", y)):
        setattr(a, name, t.data_ptr())
        setattr(a, f"{name}_batch_stride", t.stride(0))
        setattr(a, f"{name}_row_stride", t.stride(1))
    for name, f, t in (("Bm", "B", dev["B"]), ("Cm", "C", dev["C"])):
        setattr(a, name, t.data_ptr())
        setattr(a, f"{f}_batch_stride", t.stride(0))
        setattr(a, f"{f}_row_stride", t.stride(1))
    a.A, a.Dskip, a.conv_w = dev["A"].data_ptr(), dev["D"].data_ptr(), dev["conv_w"].data_ptr()
    ws = torch.empty(ops.scan_workspace_bytes(1, 256, 128, torch.bfloat16, 2), dtype=torch.uint8, device="cuda")
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert _lib.device_status() == 0
    _lib.check(_lib.lib().hx_debug_scan_orphan_segment(C.byref(a), 2000, st))
    with pytest.raises(_lib.HxError) as e:
        _lib.check_device()
    assert e.value.variant == "BackendError" and "segment carry" in str(e.value)
    assert _lib.device_status() == 0  # the check cleared the word
    # the context is intact and the default limit is back: the complete two-segment scan is right
    got = run_gpu(inp, "bf16", variant=DIRECT, seq_splits=2, geom=True)
    check(got, run_ref(inp), "bf16")
    # argument checks of the test aid itself
    a.seq_splits = 3
    assert _lib.lib().hx_debug_scan_orphan_segment(C.byref(a), 2000, st) == 10


def test_gather_push_places_shards_at_their_columns():
    """hx_allgather_y_push on one GPU: two 'ranks' in one process, each with its own full buffer, both buffers local
    (the kernel only sees pointers).  After both pushes both buffers hold the concatenation of the shards; a push
    of a row range touches those rows only."""
    import ctypes as C
    import torch
    from helixml_b200 import _lib
    B, L, D = 3, 50, 192
    widths = [(0, 128), (128, 192)]
    full = torch.randn(B, L, D, device="cuda").to(torch.bfloat16)
    bufs = [torch.zeros(B, L, D, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for r, (c0, c1) in enumerate(widths):
        shard = full[:, :, c0:c1].contiguous()
        a = _lib.GatherArgs()
        a.world, a.rank, a.batch, a.seq_len, a.d_shard, a.d_full, a.col0, a.io_dtype = 2, r, B, L, c1 - c0, D, c0, _lib.HX_BF16
        a.y_local = shard.data_ptr()
        a.dst[0], a.dst[1] = bufs[0].data_ptr(), bufs[1].data_ptr()
        a.row_begin, a.row_end = (0, B) if r == 0 else (1, 3)
        _lib.check(_lib.lib().hx_allgather_y_push(C.byref(a), st))
    torch.cuda.synchronize()
    for buf in bufs:
        assert torch.equal(buf[:, :, :128], full[:, :, :128])
        assert torch.equal(buf[1:, :, 128:], full[1:, :, 128:])
        assert torch.count_nonzero(buf[0, :, 128:]) == 0  # row 0 of rank 1's shard was not pushed
    a.col0 = 4  # 8 bytes: not a 16-byte multiple
    assert _lib.lib().hx_allgather_y_push(C.byref(a), st) == 5
    a.col0, a.world = 128, 9
    assert _lib.lib().hx_allgather_y_push(C.byref(a), st) == 10
