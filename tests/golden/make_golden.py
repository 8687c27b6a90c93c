"""Regenerates tests/golden/*.npz from the CPU oracle (C restatement, f32).

    python tests/golden/make_golden.py

Every case is produced by oracle/oracle.c and cross-checked against the numpy twin
(oracle/oracle_np.py) before it is written.  The reference itself holds no numeric fixture
for S4/Mamba outputs and cannot be built here (no Rust toolchain), so these vectors pin the
oracle against itself over time, not against the reference: parity stays "unpinned" for
those outputs.  Inputs come from helixml_b200.synth (counter-based SplitMix64)."""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from helixml_b200 import synth  # noqa: E402
from oracle import cbind, oracle_np as onp  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def close(a, b, tol=2e-5):
    err = np.max(np.abs(a - b) / (1 + np.abs(b)))
    assert err < tol, err


def scan_case(name, seed, B, L, D, N, K, bf16, gate=True, bias=True):
    inp = synth.scan_inputs(seed, B, L, D, N, K, bf16=bf16)
    dt_bias = synth.uniform(seed, "dt_bias", (D,), -0.5, 0.5) if bias else None
    conv_b = synth.uniform(seed, "conv_b", (D,), -0.2, 0.2) if bias else None
    z = inp["z"] if gate else None
    kw = dict(D=inp["D"], z=z, conv_w=inp["conv_w"], conv_b=conv_b, dt_bias=dt_bias, dt_softplus=True)
    y, h = cbind.selective_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], return_state=True, **kw)
    y2, h2 = onp.selective_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], return_state=True, **kw)
    close(y, y2); close(h, h2)
    np.savez_compressed(os.path.join(OUT, name), x=inp["x"], dt=inp["dt"], z=inp["z"], B=inp["B"], C=inp["C"], A=inp["A"],
                        D=inp["D"], conv_w=inp["conv_w"], conv_b=conv_b if bias else np.zeros(0, np.float32),
                        dt_bias=dt_bias if bias else np.zeros(0, np.float32), gate=np.int32(gate), y=y, h_last=h)


def main():
    # fused selective scan, f32 inputs, ragged sizes (L not a chunk multiple, D not a tile multiple)
    scan_case("scan_f32_small.npz", 11, 2, 37, 24, 16, 4, bf16=False)
    # bf16-exact inputs, no gate / no biases, 3-tap conv
    scan_case("scan_bf16_small.npz", 12, 1, 70, 40, 16, 3, bf16=True, gate=False, bias=False)

    # diagonal S4 (benchmark configuration 1 shrunk)
    s = synth.s4_inputs(1, 2, 61, 10, 64)
    y = cbind.s4_diag(s["u"], s["A"], s["B"], s["C"], s["delta"], s["D"])
    close(y, onp.s4_diag(s["u"], s["A"], s["B"], s["C"], s["delta"], s["D"]))
    np.savez_compressed(os.path.join(OUT, "s4_diag_small.npz"), **s, y=y)

    # reference-literal S4 (crates/nn/src/ssm.rs:138-186), init as S4Block::new (ssm.rs:39-100) but D != 0
    M, L, N = 12, 45, 16
    r = {"u": synth.normal(21, "u", (M, L)), "A_real": np.zeros(N, np.float32), "A_imag": synth.normal(21, "Ai", (N,)),
         "B": synth.normal(21, "B", (N, M), 0, 0.1), "C": synth.normal(21, "C", (M, N), 0, 0.1),
         "D": synth.normal(21, "D", (M,), 0, 0.5)}
    y = cbind.s4_forward_ssm(r["u"], r["A_real"], r["A_imag"], r["B"], r["C"], r["D"])
    assert np.array_equal(y, onp.s4_forward_ssm(r["u"], r["A_real"], r["A_imag"], r["B"], r["C"], r["D"]))
    np.savez_compressed(os.path.join(OUT, "s4_ref_small.npz"), **r, y=y)

    # exported reference MambaBlock (crates/nn/src/lib.rs:888-906): out_proj(silu(gate(x))), config-0 shapes
    L, M, E = 100, 64, 128
    e = {"x": synth.uniform(0, "x", (L, M), -1, 1), "wg": synth.normal(0, "wg", (E, M), 0, np.sqrt(2 / M)),
         "bg": np.zeros(E, np.float32), "wo": synth.normal(0, "wo", (M, E), 0, np.sqrt(2 / E)), "bo": np.zeros(M, np.float32)}
    y = cbind.mamba_exported(e["x"], e["wg"], e["bg"], e["wo"], e["bo"])
    close(y, onp.mamba_exported(e["x"], e["wg"], e["bg"], e["wo"], e["bo"]))
    np.savez_compressed(os.path.join(OUT, "mamba_exported_cfg0.npz"), **e, y=y)

    # full Mamba block, benchmark configuration 0: batch 1, L 100, d_model 64, d_state 16, expand 2, conv 4, seed 0.
    # Weights and input are regenerated from the seed by the tests; only the output and a digest are stored.
    w = synth.mamba_block_weights(0, 64, 16, 4, 2)
    x = synth.uniform(0, "x", (1, 100, 64), -1, 1)
    y = cbind.mamba_block(x, w, 16, 4)
    close(y, onp.mamba_block(x, w, 16, 4))
    np.savez_compressed(os.path.join(OUT, "mamba_block_cfg0.npz"), y=y,
                        x_sum=np.float64(x.astype(np.float64).sum()),
                        w_sum=np.float64(sum(float(v.astype(np.float64).sum()) for v in w.values())))
    print("golden vectors written to", OUT)


if __name__ == "__main__":
    main()
