"""GPU tests of the module-level API (the reference's constructors and forward): same names, same argument
meaning, same error behaviour, outputs checked against the oracle on injected weights."""
import ctypes as C

import numpy as np
import pytest

from conftest import BF16_TOL, FP32_TOL, fp32_tol_err, rel_l2, to_dev
from helixml_b200 import synth
from oracle import cbind

pytestmark = pytest.mark.gpu


def test_mamba_block_creation():
    # crates/nn/src/ssm.rs:590-598 / examples/ssm_example/src/main.rs:26: MambaBlock::new(64, 16, 4, 2, &device)
    from helixml_b200 import nn
    m = nn.MambaBlock(64, 16, 4, 2, nn.Device.cuda(0))
    ps = m.parameters()
    assert m.name == "MambaBlock" and len(ps) == 9
    shapes = [p.shape for p in ps]
    assert shapes == [(256, 64), (128, 4), (128,), (4 + 32, 128), (128, 4), (128,), (128, 16), (128,), (64, 128)]
    A = ps[6].numpy()
    assert np.allclose(A, -np.arange(1, 17, dtype=np.float32)[None, :], rtol=1e-6)  # A_log[d,n] = log(n+1)
    assert np.all(ps[7].numpy() == 1.0)                                             # D = 1
    dt0 = np.log1p(np.exp(ps[5].numpy()))                                           # softplus(bias) in [1e-3, 1e-1]
    assert dt0.min() >= 0.99e-3 and dt0.max() <= 1.01e-1


def test_mamba_block_forward_matches_oracle_config0(golden):
    """Benchmark configuration 0 through the module API: x [100, 64] (2-D, as the reference's example feeds
    it) and [1, 100, 64] give the same numbers as the oracle block on the same injected weights."""
    from helixml_b200 import nn
    w = synth.mamba_block_weights(0, 64, 16, 4, 2)
    x = synth.uniform(0, "x", (1, 100, 64), -1, 1)
    m = nn.MambaBlock(64, 16, 4, 2, nn.Device.cuda(0))
    m.load_weights(w)
    ref = golden("mamba_block_cfg0.npz")["y"]
    y3 = m.forward(nn.Tensor.from_numpy(x)).numpy()
    y2 = m(nn.Tensor.from_numpy(x[0])).numpy()
    assert y3.shape == (1, 100, 64) and y2.shape == (100, 64)
    assert fp32_tol_err(y3, ref) <= FP32_TOL and fp32_tol_err(y2, ref[0]) <= FP32_TOL


def test_mamba_block_errors():
    from helixml_b200 import _lib, nn
    m = nn.MambaBlock(64, 16, 4, 2, nn.Device.cuda(0))
    with pytest.raises(_lib.HxError) as e:
        m.forward(nn.Tensor.from_numpy(np.zeros((10, 32), np.float32)))
    assert e.value.variant == "ShapeMismatch"
    with pytest.raises(_lib.HxError) as e:
        m.forward(nn.Tensor.from_numpy(np.zeros((10, 64), np.float32), dtype=nn.BF16))
    assert e.value.variant == "DTypeMismatch"
    with pytest.raises(_lib.HxError) as e:
        nn.MambaBlock(64, 16, 9, 2, nn.Device.cuda(0))
    assert e.value.variant == "InvalidDimension"
    with pytest.raises(_lib.HxError) as e:
        m.load_parameters([np.zeros(3, np.float32)])
    assert e.value.variant == "InvalidCheckpoint"
    out = m.forward(nn.Tensor.from_numpy(np.zeros((0, 64), np.float32)))
    assert out.shape == (0, 64)


def test_s4_block_creation_and_forward_ssm():
    # crates/nn/src/ssm.rs:560-567: S4Block::new(64, 16); ssm.rs:138-147: forward_ssm wants dim0 == d_model
    from helixml_b200 import _lib, nn
    s4 = nn.S4Block(64, 16, nn.Device.cuda(0))
    ps = s4.parameters()
    assert [p.shape for p in ps[:7]] == [(16,), (16,), (16, 64), (64, 16), (64,), (64,), (16,)]
    assert np.all(ps[0].numpy() == 0) and np.all(ps[4].numpy() == 0)  # A_real and D start at zero
    delta = ps[5].numpy()
    assert delta.min() >= 0.001 and delta.max() <= 0.1
    u = synth.normal(71, "u", (64, 32))
    y = s4.forward_ssm(nn.Tensor.from_numpy(u)).numpy()
    vals = [p.numpy() for p in ps]
    ref = cbind.s4_forward_ssm(u, vals[0], vals[1], vals[2], vals[3], vals[4])
    assert y.shape == (32, 64) and fp32_tol_err(y, ref) <= FP32_TOL
    with pytest.raises(_lib.HxError) as e:
        s4.forward_ssm(nn.Tensor.from_numpy(synth.normal(71, "u2", (32, 64))))
    assert e.value.variant == "ShapeMismatch"


def test_s4_block_forward_diagonal():
    from helixml_b200 import nn
    s = synth.s4_inputs(1, 2, 100, 32, 64)
    s4 = nn.S4Block(32, 64, nn.Device.cuda(0))
    ps = s4.parameters()
    ps[4].copy_from(s["D"]); ps[5].copy_from(s["delta"]); ps[7].copy_from(s["A"]); ps[8].copy_from(s["B"]); ps[9].copy_from(s["C"])
    y = s4.forward(nn.Tensor.from_numpy(s["u"])).numpy()
    assert fp32_tol_err(y, cbind.s4_diag(s["u"], s["A"], s["B"], s["C"], s["delta"], s["D"])) <= FP32_TOL


def test_linear_and_rmsnorm_modules():
    from helixml_b200 import nn
    lin = nn.Linear(48, 20, True, nn.Device.cuda(0))
    w, b = [p.numpy() for p in lin.parameters()]
    assert w.shape == (20, 48) and np.all(b == 0) and 0.1 < w.std() < 0.3  # N(0, sqrt(2/48)) = 0.204
    x = synth.normal(72, "x", (7, 48))
    assert fp32_tol_err(lin(nn.Tensor.from_numpy(x)).numpy(), cbind.linear(x, w, b)) <= FP32_TOL
    norm = nn.RMSNorm(48, 1e-5, nn.Device.cuda(0))
    assert np.all(norm.parameters()[0].numpy() == 1.0)
    x3 = synth.normal(72, "x3", (2, 5, 48))
    assert fp32_tol_err(norm(nn.Tensor.from_numpy(x3)).numpy(), cbind.rmsnorm(x3, np.ones(48, np.float32))) <= FP32_TOL


def _lm_weights(seed, n_layer, M):
    layers = []
    for l in range(n_layer):
        w = synth.mamba_block_weights(seed, M, 16, 4, 2, init="0.02", prefix=f"l{l}.")
        w["norm_w"] = synth.uniform(seed, f"l{l}.norm", (M,), 0.8, 1.2)
        layers.append(w)
    emb = synth.normal(seed, "emb", (256, M), 0, 0.02)
    normf = synth.uniform(seed, "normf", (M,), 0.8, 1.2)
    return emb, layers, normf


def test_byte_lm_f32_matches_oracle():
    from helixml_b200 import nn
    emb, layers, normf = _lm_weights(3, 3, 64)
    tok = synth.random_bytes(3, "tok", (2, 50))
    lm = nn.ByteLM(3, 64, dtype=nn.F32)
    lm.load_weights(emb, layers, normf)
    got = lm.forward(nn.Tensor.from_numpy(tok)).numpy()
    ref = cbind.byte_lm(tok, emb, layers, normf, 16, 4)
    assert got.shape == (2, 50, 256)
    assert fp32_tol_err(got, ref) <= FP32_TOL


def test_byte_lm_bf16_matches_oracle_and_host_call():
    import torch
    from helixml_b200 import _lib, nn
    M, nl, B, L = 128, 4, 2, 96
    emb, layers, normf = _lm_weights(3, nl, M)
    big = ("W_in", "W_x", "W_dt", "W_out")
    layers_q = [{k: (synth.round_bf16(v) if k in big else v) for k, v in l.items()} for l in layers]
    emb_q = synth.round_bf16(emb)
    tok = synth.random_bytes(3, "tok", (B, L))
    lm = nn.ByteLM(nl, M, dtype=nn.BF16)
    lm.load_weights(emb_q, layers_q, normf)
    got = lm.forward(nn.Tensor.from_numpy(tok)).numpy()
    ref = cbind.byte_lm(tok, emb_q, layers_q, normf, 16, 4)
    assert rel_l2(got, ref) <= BF16_TOL
    # the serving call: pinned host tokens in, pinned host logits out
    th = torch.from_numpy(tok).pin_memory()
    lh = torch.empty((B, L, 256), dtype=torch.bfloat16).pin_memory()
    lm.forward_host(th.data_ptr(), lh.data_ptr(), B, L, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert np.array_equal(lh.float().numpy(), got)
    assert _lib.device_status() == 0
    assert lm.launches_per_forward == 1 + nl * 6 + 2   # per block: norm, in_proj, conv + x_proj, dt_proj, scan, out_proj


@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_byte_lm_prefill_then_decode_steps(dtype_name):
    """Prefill L0 bytes keeping the per-layer state, then decode token by token: the logits of every step must be
    the oracle's logits for that position of the longer sequence.  Steps 3+ replay the captured CUDA graph; a run
    with plain launches must give the same bits."""
    import torch
    from helixml_b200 import _lib, nn
    bf = dtype_name == "bf16"
    M, nl, B, L0, steps = 64, 3, 2, 41, 6
    emb, layers, normf = _lm_weights(9, nl, M)
    big = ("W_in", "W_x", "W_dt", "W_out")
    if bf:
        layers = [{k: (synth.round_bf16(v) if k in big else v) for k, v in l.items()} for l in layers]
        emb = synth.round_bf16(emb)
    tok = synth.random_bytes(9, "tok", (B, L0 + steps))
    ref = cbind.byte_lm(tok, emb, layers, normf, 16, 4)  # [B, L0 + steps, 256]
    td = torch.bfloat16 if bf else torch.float32
    tok_d = torch.from_numpy(tok).cuda()
    runs = []
    for graph in (True, False):
        lm = nn.ByteLM(nl, M, dtype=nn.BF16 if bf else nn.F32)
        lm.load_weights(emb, layers, normf)
        lm.decode_graph(graph)
        pre = torch.empty(B, L0, 256, device="cuda", dtype=td)
        lm.prefill_device(tok_d[:, :L0].contiguous().data_ptr(), pre.data_ptr(), B, L0)
        outs = []
        for s in range(steps):
            t1 = tok_d[:, L0 + s].contiguous()
            lg = torch.empty(B, 256, device="cuda", dtype=td)
            lm.decode_step_device(t1.data_ptr(), lg.data_ptr(), B)
            outs.append(lg.float().cpu().numpy())
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        got = np.stack(outs, axis=1)
        if bf:
            assert rel_l2(pre.float().cpu().numpy(), ref[:, :L0]) <= BF16_TOL
            assert rel_l2(got, ref[:, L0:]) <= BF16_TOL
        else:
            assert fp32_tol_err(pre.cpu().numpy(), ref[:, :L0]) <= FP32_TOL
            assert fp32_tol_err(got, ref[:, L0:]) <= FP32_TOL
        assert lm.launches_per_decode_step == 1 + nl * (4 if bf else 7) + 2
        runs.append(got)
    assert np.array_equal(runs[0], runs[1])  # graph replay and plain launches agree bit for bit


def test_byte_lm_decode_without_prefill_is_an_error():
    import torch
    from helixml_b200 import _lib, nn
    lm = nn.ByteLM(1, 64, dtype=nn.F32)
    t = torch.zeros(2, dtype=torch.uint8, device="cuda")
    lg = torch.empty(2, 256, device="cuda")
    with pytest.raises(_lib.HxError) as e:
        lm.decode_step_device(t.data_ptr(), lg.data_ptr(), 2)
    assert e.value.status == 10


def test_module_checkpoint_round_trip(tmp_path):
    """Save a block's parameters in the reference's checkpoint layout, restore them into a freshly initialised
    block: same parameters, same forward; a checkpoint of another architecture is refused and changes nothing."""
    from helixml_b200 import _lib, checkpoint, nn
    nn.manual_seed(11)
    a = nn.MambaBlock(64, 16, 4, 2, dtype=nn.BF16)
    nn.manual_seed(12)
    b = nn.MambaBlock(64, 16, 4, 2, dtype=nn.BF16)
    x = nn.Tensor.from_numpy(synth.round_bf16(synth.normal(11, "x", (2, 40, 64))), dtype=nn.BF16)
    ya = a(x).numpy()
    assert not np.array_equal(ya, b(x).numpy())
    p = str(tmp_path / "checkpoint_epoch_4.pt")
    a.save_checkpoint(p, epoch=4, step=77, training_loss=1.25, learning_rate=3e-4, timestamp_secs=1700000000)
    meta, arrays = checkpoint.read(p)  # the host-side reader sees the same file
    assert meta["epoch"] == 4 and meta["step"] == 77 and len(arrays) == len(a.parameters())
    for t, arr in zip(a.parameters(), arrays):
        assert tuple(arr.shape) == tuple(t.shape) and np.array_equal(t.numpy(), arr)
    got = b.load_checkpoint(p)
    assert got["epoch"] == 4 and got["training_loss"] == 1.25
    assert np.array_equal(b(x).numpy(), ya)
    other = nn.MambaBlock(32, 16, 4, 2, dtype=nn.BF16)
    before = [t.numpy() for t in other.parameters()]
    with pytest.raises(_lib.HxError) as e:
        other.load_checkpoint(p)
    assert e.value.variant == "ShapeMismatch"
    lin = nn.Linear(8, 8)
    with pytest.raises(_lib.HxError) as e:
        lin.load_checkpoint(p)
    assert e.value.variant == "InvalidCheckpoint"
    assert all(np.array_equal(t.numpy(), v) for t, v in zip(other.parameters(), before))


def test_byte_lm_checkpoint_round_trip(tmp_path):
    """A whole byte LM (embedding, per-layer norm and block parameters, final norm) through the reference's
    checkpoint layout: the restored model gives the same logits bit for bit."""
    from helixml_b200 import nn
    nn.manual_seed(21)
    a = nn.ByteLM(2, 64, dtype=nn.BF16)
    nn.manual_seed(22)
    b = nn.ByteLM(2, 64, dtype=nn.BF16)
    tok = synth.random_bytes(21, "tok", (2, 33))
    la = a.forward(nn.Tensor.from_numpy(tok)).numpy()
    assert not np.array_equal(la, b.forward(nn.Tensor.from_numpy(tok)).numpy())
    p = str(tmp_path / "lm.pt")
    a.save_checkpoint(p, epoch=1, step=10)
    meta = b.load_checkpoint(p)
    assert meta["epoch"] == 1 and meta["step"] == 10
    assert np.array_equal(b.forward(nn.Tensor.from_numpy(tok)).numpy(), la)


def _per_position_worst(got, ref):
    """Largest relative L2 error over single positions (one token's output vector each)."""
    g, r = got.reshape(-1, got.shape[-1]).astype(np.float64), ref.reshape(-1, ref.shape[-1]).astype(np.float64)
    return float(np.max(np.linalg.norm(g - r, axis=1) / np.maximum(np.linalg.norm(r, axis=1), 1e-30)))


def test_mamba_block_full_size_config3_shape_sampled_rows():
    """One block at the benchmark's shape, [32, 2048, 768] bf16: the path the byte LM times (tensor-core GEMMs, the
    dt projection as a kernel of its own, the one-lane-per-channel scan with chained sequence segments).  Batch rows are
    independent, so the oracle runs on the first and the last row; the gate is applied to the rows as a whole and
    to every position by itself (a lost carry would spoil the positions after one segment boundary)."""
    import torch
    from helixml_b200 import _lib, ops
    B, L, M = 32, 2048, 768
    w = synth.mamba_block_weights(3, M, 16, 4, 2, init="0.02")
    big = ("W_in", "W_x", "W_dt", "W_out")
    wq = {k: (synth.round_bf16(v) if k in big else v) for k, v in w.items()}
    x = synth.round_bf16(synth.normal(3, "xfull", (B, L, M)))
    dev = {k: to_dev(v, "bf16" if k in big else None) for k, v in wq.items()}
    got = ops.mamba_block(to_dev(x, "bf16"), dev, 16, 4)
    _lib.check_device()
    a = _lib.MambaBlockArgs()
    a.batch, a.seq_len, a.d_model, a.d_inner, a.d_state, a.d_conv, a.dt_rank = B, L, M, 2 * M, 16, 4, 48
    a.io_dtype, a.scan_variant, a.a_geometric = _lib.HX_BF16, _lib.SCAN_AUTO, 1
    a.W_dt = dev["W_dt"].data_ptr()
    n = C.c_int32(0)
    _lib.check(_lib.lib().hx_mamba_block_kernel_launches(C.byref(a), C.byref(n)))
    assert n.value == 4  # in_proj, conv + x_proj (one kernel), scan (one pass, chained segments, dt projection inside), out_proj
    rows = [0, B - 1]
    ref = cbind.mamba_block(x[rows], wq, 16, 4)
    g = got[rows].float().cpu().numpy()
    assert rel_l2(g, ref) <= BF16_TOL
    assert _per_position_worst(g, ref) <= 3 * BF16_TOL


def test_byte_lm_full_size_config3_sampled_sequences():
    """Benchmark configuration 3 at full size: 24 blocks, d_model 768, batch 32 x 2048 bytes, bf16 -- the very call
    bench.py times.  The logits of the first and the last sequence are compared with the CPU oracle of the whole
    model (rows are independent); the launch count shows that every block ran the one-pass scan after a dt_proj
    kernel (the look-back form would be one launch more, the fused dt projection one less)."""
    import torch
    from helixml_b200 import _lib, nn
    nl, M, B, L = 24, 768, 32, 2048
    emb, layers, normf = _lm_weights(3, nl, M)
    big = ("W_in", "W_x", "W_dt", "W_out")
    layers_q = [{k: (synth.round_bf16(v) if k in big else v) for k, v in l.items()} for l in layers]
    emb_q = synth.round_bf16(emb)
    tok = synth.random_bytes(3, "tokfull", (B, L))
    lm = nn.ByteLM(nl, M, dtype=nn.BF16)
    lm.load_weights(emb_q, layers_q, normf)
    tok_d = torch.from_numpy(tok).cuda()
    logits = torch.empty((B, L, 256), dtype=torch.bfloat16, device="cuda")
    lm.forward_device(tok_d.data_ptr(), logits.data_ptr(), B, L, torch.cuda.current_stream().cuda_stream)
    _lib.check_device()
    assert lm.launches_per_forward == 1 + nl * 5 + 2  # norm, in_proj, conv + x_proj, scan (dt projection inside), out_proj per block
    rows = [0, B - 1]
    ref = cbind.byte_lm(tok[rows], emb_q, layers_q, normf, 16, 4)
    g = logits[rows].float().cpu().numpy()
    # 24 blocks deep, the rounding of bf16 STORAGE alone (f32 arithmetic, values rounded where a bf16 path stores
    # them) already moves the f32 result by about 2e-2, the size of the gate; so the model-level check is against
    # that floor: the kernels may add a tenth to it, and they must agree with the storage-rounded model itself far
    # more closely than with the f32 one.
    floor = cbind.byte_lm_bf16_storage(tok[rows], emb_q, layers_q, normf, 16, 4)
    err, err_floor = rel_l2(g, ref), rel_l2(floor, ref)
    assert err <= max(BF16_TOL, 1.1 * err_floor), (err, err_floor)
    assert err <= 1.5 * BF16_TOL
    assert rel_l2(g, floor) <= BF16_TOL, rel_l2(g, floor)
    assert _per_position_worst(g, ref) <= 3 * BF16_TOL


def test_byte_lm_small_batch_runs_the_lookback_scan():
    """Four sequences per GPU is what one of eight GPUs gets of configuration 3's batch: too few chains for one pass,
    so the blocks run the look-back form of the scan (two launches), each pass computing the dt projection itself."""
    import torch
    from helixml_b200 import _lib, nn
    nl, M, B, L = 3, 768, 4, 1024
    emb, layers, normf = _lm_weights(11, nl, M)
    big = ("W_in", "W_x", "W_dt", "W_out")
    layers_q = [{k: (synth.round_bf16(v) if k in big else v) for k, v in l.items()} for l in layers]
    emb_q = synth.round_bf16(emb)
    tok = synth.random_bytes(11, "tok", (B, L))
    lm = nn.ByteLM(nl, M, dtype=nn.BF16)
    lm.load_weights(emb_q, layers_q, normf)
    tok_d = torch.from_numpy(tok).cuda()
    logits = torch.empty((B, L, 256), dtype=torch.bfloat16, device="cuda")
    lm.forward_device(tok_d.data_ptr(), logits.data_ptr(), B, L, torch.cuda.current_stream().cuda_stream)
    _lib.check_device()
    assert lm.launches_per_forward == 1 + nl * 6 + 2  # norm, in_proj, conv + x_proj, aggregate pass, output pass (dt projection inside both), out_proj
    ref = cbind.byte_lm(tok, emb_q, layers_q, normf, 16, 4)
    g = logits.float().cpu().numpy()
    assert rel_l2(g, ref) <= BF16_TOL
    assert _per_position_worst(g, ref) <= 3 * BF16_TOL


def test_byte_lm_handle_shared_by_two_threads():
    """Two threads call forward on ONE byte-LM handle (default stream): the module serialises them, and each gets
    the logits of its own tokens."""
    import threading
    from helixml_b200 import nn
    emb, layers, normf = _lm_weights(12, 2, 64)
    lm = nn.ByteLM(2, 64, dtype=nn.F32)
    lm.load_weights(emb, layers, normf)
    toks = [synth.random_bytes(12, f"t{i}", (2, 70)) for i in range(2)]
    want = [lm.forward(nn.Tensor.from_numpy(t)).numpy() for t in toks]
    got, errors = [None, None], []

    def run(i):
        try:
            for _ in range(5):
                got[i] = lm.forward(nn.Tensor.from_numpy(toks[i])).numpy()
        except Exception as e:  # noqa: BLE001
            errors.append(repr(e))

    th = [threading.Thread(target=run, args=(i,)) for i in range(2)]
    for t in th:
        t.start()
    for t in th:
        t.join()
    assert not errors, errors
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])


@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_byte_lm_forward_graph_replay_equals_plain_launches(dtype_name):
    """The second and later calls of forward_device with the same buffers replay a captured graph of the whole
    forward: same bits as plain launches, also after the tokens in the buffer changed, after a different shape was
    run in between, and for the prefill that keeps the decode state."""
    import torch
    from helixml_b200 import _lib, nn
    bf = dtype_name == "bf16"
    M, nl, B, L = 128, 3, 2, 200
    emb, layers, normf = _lm_weights(13, nl, M)
    td = torch.bfloat16 if bf else torch.float32
    lm = nn.ByteLM(nl, M, dtype=nn.BF16 if bf else nn.F32)
    lm.load_weights(emb, layers, normf)
    toks = [torch.from_numpy(synth.random_bytes(13, f"t{i}", (B, L))).cuda() for i in range(3)]
    buf = torch.empty_like(toks[0])
    out = torch.empty(B, L, 256, device="cuda", dtype=td)
    lm.forward_graph(False)
    want = []
    for t in toks:
        buf.copy_(t)
        lm.forward_device(buf.data_ptr(), out.data_ptr(), B, L)
        torch.cuda.synchronize()
        want.append(out.clone())
    lm.forward_graph(True)
    for rnd in range(2):
        for i, t in enumerate(toks):  # call 1 plain, call 2 captures, later calls replay
            buf.copy_(t)
            lm.forward_device(buf.data_ptr(), out.data_ptr(), B, L)
            torch.cuda.synchronize()
            assert torch.equal(out, want[i]), (rnd, i)
        # another shape in between drops the graphs (they point into the old activation buffers)
        small = torch.empty(1, 64, 256, device="cuda", dtype=td)
        lm.forward_device(toks[0][:1, :64].contiguous().data_ptr(), small.data_ptr(), 1, 64)
    # prefill with state through the graph, then a decode step: same as with plain launches
    nxt = torch.from_numpy(synth.random_bytes(13, "nxt", (B,))).cuda()
    res = []
    for graph in (False, True):
        lm.forward_graph(graph)
        for _ in range(3):
            lm.prefill_device(toks[1].data_ptr(), out.data_ptr(), B, L)
        lg = torch.empty(B, 256, device="cuda", dtype=td)
        lm.decode_step_device(nxt.data_ptr(), lg.data_ptr(), B)
        torch.cuda.synchronize()
        res.append((out.clone(), lg.clone()))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
    assert _lib.device_status() == 0


def test_sequential_chains_modules():
    """nn::Sequential (crates/nn/src/lib.rs:577-661): add() in order, forward chains, parameters concatenates.  The
    reference's own test builds Linear -> activation -> Linear and checks the output shape (lib.rs:1296-1313); here
    the numbers are checked against the oracle as well."""
    from helixml_b200 import _lib, nn
    nn.manual_seed(21)
    seq = nn.Sequential()
    l1, norm, l2 = nn.Linear(48, 96, True), nn.RMSNorm(96), nn.Linear(96, 24, True)
    w1, b1 = [p.numpy() for p in l1.parameters()]
    wn = norm.parameters()[0].numpy()
    w2, b2 = [p.numpy() for p in l2.parameters()]
    for m in (l1, norm, l2):
        seq.add(m)
    assert len(seq) == 3 and seq.name == "Sequential" and len(seq.parameters()) == 5
    assert l1._h is None  # consumed by add
    x = synth.normal(21, "x", (10, 48))
    got = seq(nn.Tensor.from_numpy(x)).numpy()
    ref = cbind.linear(cbind.rmsnorm(cbind.linear(x, w1, b1), wn), w2, b2)
    assert got.shape == (10, 24) and fp32_tol_err(got, ref) <= FP32_TOL
    # an error inside the chain comes back as the module's error
    with pytest.raises(_lib.HxError) as e:
        seq(nn.Tensor.from_numpy(synth.normal(21, "bad", (10, 50))))
    assert e.value.variant == "ShapeMismatch"
    empty = nn.Sequential()
    assert len(empty) == 0 and np.array_equal(empty(nn.Tensor.from_numpy(x)).numpy(), x)
