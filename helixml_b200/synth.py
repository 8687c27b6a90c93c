"""Seeded synthetic inputs for the state-space hot path.

The reference draws every weight and input from an unseeded `rand::thread_rng()`
(crates/backend-cpu/src/lib.rs:1209,1233,1257), so "seed k" of a benchmark
configuration cannot come from it.  This module defines the streams instead: a
counter-based SplitMix64 generator, so element i of stream (seed, name) is a pure
function of (seed, name, i) and does not depend on any library's RNG version.

uniform01: top 24 bits of the 64-bit output times 2^-24 (exact in f32).
normal:    Box-Muller on two uniforms taken from counters 2i and 2i+1, evaluated in f64.
"""
from __future__ import annotations

import zlib

import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def _mix(x: np.ndarray) -> np.ndarray:
    x = (x ^ (x >> np.uint64(30))) * _M1
    x = (x ^ (x >> np.uint64(27))) * _M2
    return x ^ (x >> np.uint64(31))


def stream_key(seed: int, name: str) -> np.uint64:
    """64-bit key of a named stream: mixes the seed with a CRC of the name."""
    with np.errstate(over="ignore"):
        k = np.uint64(seed) * _GOLDEN + np.uint64(zlib.crc32(name.encode()))
        return _mix(np.asarray([k], dtype=np.uint64))[0]


def raw_u64(seed: int, name: str, n: int, offset: int = 0) -> np.ndarray:
    with np.errstate(over="ignore"):
        ctr = np.arange(offset, offset + n, dtype=np.uint64)
        return _mix(stream_key(seed, name) + (ctr + np.uint64(1)) * _GOLDEN)


def uniform01(seed: int, name: str, n: int, offset: int = 0) -> np.ndarray:
    """n values in [0, 1), f64 holding exact multiples of 2^-24."""
    return (raw_u64(seed, name, n, offset) >> np.uint64(40)).astype(np.float64) * (1.0 / (1 << 24))


def uniform(seed: int, name: str, shape, lo: float, hi: float) -> np.ndarray:
    n = int(np.prod(shape))
    return (lo + (hi - lo) * uniform01(seed, name, n)).astype(np.float32).reshape(shape)


def normal(seed: int, name: str, shape, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    n = int(np.prod(shape))
    u = uniform01(seed, name, 2 * n)
    u1 = 1.0 - u[0::2]                      # (0, 1]
    u2 = u[1::2]
    g = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (mean + std * g).astype(np.float32).reshape(shape)


def log_uniform(seed: int, name: str, shape, lo: float, hi: float) -> np.ndarray:
    n = int(np.prod(shape))
    u = uniform01(seed, name, n)
    return np.exp(np.log(lo) + u * (np.log(hi) - np.log(lo))).astype(np.float32).reshape(shape)


def random_bytes(seed: int, name: str, shape) -> np.ndarray:
    n = int(np.prod(shape))
    return (raw_u64(seed, name, n) >> np.uint64(56)).astype(np.uint8).reshape(shape)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """Nearest-even rounding of f32 to bf16, returned widened back to f32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return r.view(np.float32).reshape(x.shape)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """bf16 bit patterns (uint16) of an f32 array, nearest-even."""
    return (round_bf16(x).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


# ----------------------------------------------------------------------------- configurations

def a_log_s4d_real(d_inner: int, d_state: int) -> np.ndarray:
    """A_log[d, n] = log(n + 1); A = -exp(A_log) = -(n + 1) up to one rounding."""
    return np.tile(np.log(np.arange(1, d_state + 1, dtype=np.float32)), (d_inner, 1)).astype(np.float32)


def softplus_inverse(y: np.ndarray) -> np.ndarray:
    y = y.astype(np.float64)
    return (y + np.log(-np.expm1(-y))).astype(np.float32)


def scan_inputs(seed: int, batch: int, seq_len: int, d_inner: int, d_state: int = 16, d_conv: int = 4,
                bf16: bool = True) -> dict:
    """Inputs of the standalone fused selective scan (benchmark configurations 2 and 4):
    u, z ~ N(0,1); dt_raw ~ U[-4,-1]; A = -exp(A_log), A_log[d,n] = log(n+1); B, C ~ N(0,1)
    of shape [batch, L, d_state]; D = 1; conv weights ~ U[-0.5, 0.5].  With bf16=True the
    activations are rounded to bf16-exact values (held in f32)."""
    q = round_bf16 if bf16 else (lambda a: a)
    return {
        "x": q(normal(seed, "x", (batch, seq_len, d_inner))),
        "z": q(normal(seed, "z", (batch, seq_len, d_inner))),
        "dt": q(uniform(seed, "dt", (batch, seq_len, d_inner), -4.0, -1.0)),
        "B": q(normal(seed, "B", (batch, seq_len, d_state))),
        "C": q(normal(seed, "C", (batch, seq_len, d_state))),
        "A": (-np.exp(a_log_s4d_real(d_inner, d_state))).astype(np.float32),
        "D": np.ones((d_inner,), dtype=np.float32),
        "conv_w": uniform(seed, "conv_w", (d_inner, d_conv), -0.5, 0.5),
    }


def s4_inputs(seed: int, batch: int, seq_len: int, d_model: int, d_state: int) -> dict:
    """Inputs of the diagonal S4 recurrence (benchmark configuration 1): u ~ N(0,1);
    A[d,n] = -0.5 (n+1); B, C ~ N(0, 1/d_state) (variance); delta log-uniform in
    [1e-3, 1e-1]; D = 1."""
    std = float(np.sqrt(1.0 / d_state))
    return {
        "u": normal(seed, "u", (batch, seq_len, d_model)),
        "A": np.tile(-0.5 * np.arange(1, d_state + 1, dtype=np.float32), (d_model, 1)),
        "B": normal(seed, "B", (d_model, d_state), 0.0, std),
        "C": normal(seed, "C", (d_model, d_state), 0.0, std),
        "delta": log_uniform(seed, "delta", (d_model,), 1e-3, 1e-1),
        "D": np.ones((d_model,), dtype=np.float32),
    }


def mamba_block_weights(seed: int, d_model: int, d_state: int = 16, d_conv: int = 4, expand: int = 2,
                        init: str = "kaiming", prefix: str = "") -> dict:
    """Weights of one Mamba block.  init="kaiming": N(0, sqrt(2/in)) as the reference's
    Linear::new (crates/nn/src/lib.rs:67-84); init="0.02": N(0, 0.02).  A_log[d,n] = log(n+1),
    D = 1, dt bias = softplus^-1(dt0) with dt0 log-uniform in [1e-3, 1e-1].
    dt_rank = ceil(d_model / 16)."""
    E = d_model * expand
    R = (d_model + 15) // 16
    def w(name, shape, fan_in):
        std = 0.02 if init == "0.02" else float(np.sqrt(2.0 / fan_in))
        return normal(seed, prefix + name, shape, 0.0, std)
    dt0 = log_uniform(seed, prefix + "dt0", (E,), 1e-3, 1e-1)
    return {
        "W_in": w("W_in", (2 * E, d_model), d_model),
        "conv_w": uniform(seed, prefix + "conv_w", (E, d_conv), -0.5, 0.5),
        "conv_b": np.zeros((E,), dtype=np.float32),
        "W_x": w("W_x", (R + 2 * d_state, E), E),
        "W_dt": w("W_dt", (E, R), R),
        "b_dt": softplus_inverse(dt0),
        "A": (-np.exp(a_log_s4d_real(E, d_state))).astype(np.float32),
        "D": np.ones((E,), dtype=np.float32),
        "W_out": w("W_out", (d_model, E), E),
    }
