"""Kernel-level timings with CUDA events, for the shapes of the byte-LM benchmark configuration.

    python -m helixml_b200.kernel_bench gemm [in_proj out_proj x_proj dt_proj lm_head]
    python -m helixml_b200.kernel_bench conv
    python -m helixml_b200.kernel_bench norm
    python -m helixml_b200.kernel_bench s4
    python -m helixml_b200.kernel_bench decode

Each case runs 3 warm-up calls, then 10 timed calls between two events on torch's current stream, queued behind a
2 ms spin kernel so that the host's call rate does not limit the figure."""
from __future__ import annotations

import sys

import torch

from . import ops

GEMM_SHAPES = {"in_proj": (65536, 3072, 768), "out_proj": (65536, 768, 1536), "x_proj": (65536, 80, 1536),
               "dt_proj": (65536, 1536, 48), "lm_head": (65536, 256, 768)}


def _time(fn, reps=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # keep the GPU busy for ~2 ms while the host queues the timed launches, so that a kernel of a few tens of
    # microseconds is timed back to back and not at the rate the host can issue calls
    torch.cuda._sleep(4_000_000)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def gemm(names):
    for name in names or list(GEMM_SHAPES):
        M, N, K = GEMM_SHAPES[name]
        a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = _time(lambda: ops.gemm(a, w, out=c))
        ref = a[:256].float() @ w.float().t()
        err = (c[:256].float() - ref).abs().max().item()
        print(f"gemm {name} M={M} N={N} K={K}: {ms * 1e3:.1f} us, {2 * M * N * K / ms / 1e9:.0f} TFLOP/s, "
              f"max |err| on 256 rows {err:.3g}")


def conv():
    B, L, E = 32, 2048, 1536
    xz = torch.randn(B, L, 2 * E, device="cuda").to(torch.bfloat16)
    w = torch.rand(E, 4, device="cuda") - 0.5
    b = torch.zeros(E, device="cuda")
    u = torch.empty(B, L, E, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: ops.conv1d_silu(xz[:, :, :E], w, b, out=u))
    byt = B * L * E * 2 * 2
    print(f"conv_silu [{B},{L},{E}] bf16 (x read as a strided half of [B,L,2E]): {ms * 1e3:.1f} us, {byt / ms / 1e6:.0f} GB/s")


def norm():
    T, M = 65536, 768
    x = torch.randn(T, M, device="cuda").to(torch.bfloat16)
    r = torch.randn(T, M, device="cuda")
    w = torch.ones(M, device="cuda")
    ms = _time(lambda: ops.rmsnorm(x, w, 1e-5, residual=r, out_dtype=torch.bfloat16))
    byt = T * M * (2 + 4 + 4 + 2)
    print(f"rmsnorm + residual [{T},{M}]: {ms * 1e3:.1f} us, {byt / ms / 1e6:.0f} GB/s")


def s4():
    """Benchmark configuration 1: diagonal S4, f32, batch 8, L 2048, d_model 256, d_state 64."""
    from . import synth
    inp = synth.s4_inputs(1, 8, 2048, 256, 64)
    dev = {k: torch.from_numpy(v).cuda() for k, v in inp.items()}
    ms = _time(lambda: ops.s4_diag(dev["u"], dev["A"], dev["B"], dev["C"], dev["delta"], dev["D"]))
    byt = 2 * 8 * 2048 * 256 * 4
    upd = 8 * 2048 * 256 * 64
    print(f"s4_diag [8,2048,256] N=64 f32: {ms * 1e3:.1f} us, {byt / ms / 1e6:.0f} GB/s, {upd / ms / 1e6:.1f} G state updates/s")
    M, L, N = 256, 2048, 64
    r = {"u": torch.randn(M, L, device="cuda"), "Ar": -torch.rand(N, device="cuda"), "Ai": torch.randn(N, device="cuda"),
         "B": torch.randn(N, M, device="cuda") * 0.1, "C": torch.randn(M, N, device="cuda") * 0.1, "D": torch.randn(M, device="cuda")}
    ms = _time(lambda: ops.s4_ref_forward_ssm(r["u"], r["Ar"], r["Ai"], r["B"], r["C"], r["D"]))
    print(f"s4 reference-literal forward_ssm [256, 2048] N=64 f32: {ms * 1e3:.1f} us")


def decode():
    """Byte LM of benchmark configuration 3 (24 blocks, d_model 768, bf16): prefill 32 x 2048, then single-token
    steps for the whole batch, as plain launches and as replays of the captured CUDA graph."""
    from . import nn
    B, L0, steps = 32, 2048, 64
    nn.manual_seed(3)
    lm = nn.ByteLM(24, 768, dtype=nn.BF16)
    tok = torch.randint(0, 256, (B, L0), device="cuda", dtype=torch.uint8)
    pre = torch.empty(B, L0, 256, device="cuda", dtype=torch.bfloat16)
    nxt = torch.randint(0, 256, (B,), device="cuda", dtype=torch.uint8)
    lg = torch.empty(B, 256, device="cuda", dtype=torch.bfloat16)
    for graph in (False, True):
        lm.decode_graph(graph)
        lm.prefill_device(tok.data_ptr(), pre.data_ptr(), B, L0)
        for _ in range(4):  # the first step is plain, the second captures
            lm.decode_step_device(nxt.data_ptr(), lg.data_ptr(), B)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            lm.decode_step_device(nxt.data_ptr(), lg.data_ptr(), B)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        print(f"decode step, batch {B}, 24 blocks, d_model 768, {'CUDA graph' if graph else 'plain launches'} "
              f"({lm.launches_per_decode_step} kernels): {ms * 1e3:.0f} us/step, {B / ms * 1e3:.0f} tokens/s")


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    {"gemm": lambda: gemm(sys.argv[2:]), "conv": conv, "norm": norm, "s4": s4, "decode": decode}[what]()
