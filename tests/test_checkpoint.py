"""Checkpoint files in the reference's layout (crates/training/src/checkpoint.rs:136-197): u32 big-endian JSON
length, CheckpointData JSON, bincode of Vec<CpuTensor>.  The expected bytes are rebuilt here, independently of
the library, from the published bincode 1.3 / ndarray 0.15 serde layouts; the reference holds no checkpoint
fixture to compare with (its checkpoint tests only create the manager, checkpoint.rs:290-300), so this pins the
writer against the stated layout, not against a file the reference wrote."""
import json
import os
import struct

import numpy as np
import pytest

from helixml_b200 import _lib, checkpoint


def expected_tensor_bytes(a: np.ndarray) -> bytes:
    a = np.ascontiguousarray(a, dtype="<f4")
    dims = b"".join(struct.pack("<Q", d) for d in a.shape)
    out = struct.pack("<B", 1)                       # ndarray array format version
    out += struct.pack("<Q", a.ndim) + dims          # dim: IxDyn
    out += struct.pack("<Q", a.size) + a.tobytes()   # data, logical order
    out += struct.pack("<Q", a.ndim) + dims          # Shape { dims }
    out += struct.pack("<I", 9)                      # DType::F32
    out += struct.pack("<I", 0)                      # Device::Cpu
    return out


def test_written_file_has_the_reference_layout(tmp_path):
    rng = np.random.default_rng(0)
    arrays = [rng.standard_normal((3, 5)).astype(np.float32), rng.standard_normal((7,)).astype(np.float32),
              np.float32(2.5).reshape(()), rng.standard_normal((2, 1, 4)).astype(np.float32)]
    p = str(tmp_path / "checkpoint_epoch_3.pt")
    checkpoint.write(p, arrays, epoch=3, step=1200, training_loss=0.75, validation_loss=1.0, learning_rate=1e-3,
                     timestamp_secs=1700000000)
    raw = open(p, "rb").read()
    (jl,) = struct.unpack(">I", raw[:4])
    meta = json.loads(raw[4:4 + jl])
    assert list(meta) == ["epoch", "step", "training_loss", "validation_loss", "learning_rate", "timestamp",
                          "model_params_count", "metrics"]
    assert meta["epoch"] == 3 and meta["step"] == 1200 and meta["model_params_count"] == 4
    assert meta["training_loss"] == 0.75 and meta["validation_loss"] == 1.0 and meta["learning_rate"] == 1e-3
    assert meta["timestamp"] == 1700000000
    assert list(meta["metrics"]) == ["training_loss", "validation_loss", "epoch", "step", "learning_rate", "custom_metrics",
                                     "history"]
    assert list(meta["metrics"]["history"]) == ["training_losses", "validation_losses", "learning_rates", "epochs", "steps",
                                                "custom_metrics_history"]
    body = raw[4 + jl:]
    assert body == struct.pack("<Q", 4) + b"".join(expected_tensor_bytes(a) for a in arrays)


def test_round_trip_and_foreign_device_labels(tmp_path):
    rng = np.random.default_rng(1)
    arrays = [rng.standard_normal((4, 6)).astype(np.float32), np.zeros((0, 3), np.float32), rng.standard_normal((5,)).astype(np.float32)]
    p = str(tmp_path / "a.pt")
    checkpoint.write(p, arrays, epoch=1, step=2, training_loss=float("nan"))
    meta, back = checkpoint.read(p)
    assert meta["epoch"] == 1 and meta["step"] == 2 and np.isnan(meta["training_loss"])
    assert len(back) == 3
    for a, b in zip(arrays, back):
        assert a.shape == b.shape and np.array_equal(a, b)
    # a file whose tensors carry Device::Cuda(1) and DType::F16 labels (what a device-resident tensor type in the
    # reference would write) reads the same: storage is f32, the labels are skipped
    raw = open(p, "rb").read()
    (jl,) = struct.unpack(">I", raw[:4])
    body = struct.pack("<Q", 1)
    a = arrays[0]
    dims = b"".join(struct.pack("<Q", d) for d in a.shape)
    body += struct.pack("<B", 1) + struct.pack("<Q", 2) + dims + struct.pack("<Q", a.size) + a.tobytes()
    body += struct.pack("<Q", 2) + dims + struct.pack("<I", 8) + struct.pack("<I", 1) + struct.pack("<Q", 1)
    j = json.dumps({"epoch": 9, "step": 10, "training_loss": 0.5, "validation_loss": None, "learning_rate": 0.1, "timestamp": 5,
                    "model_params_count": 1, "metrics": {"epoch": 0, "step": 0}}, separators=(",", ":")).encode()
    p2 = str(tmp_path / "b.pt")
    open(p2, "wb").write(struct.pack(">I", len(j)) + j + body)
    meta, back = checkpoint.read(p2)
    assert meta["epoch"] == 9 and meta["step"] == 10 and np.isnan(meta["validation_loss"])
    assert np.array_equal(back[0], a)


@pytest.mark.parametrize("damage", ["truncate_header", "truncate_body", "trailing", "bad_version", "count_mismatch", "missing",
                                    "huge_count", "wrapping_shape"])
def test_malformed_files_are_refused(tmp_path, damage):
    p = str(tmp_path / "c.pt")
    checkpoint.write(p, [np.arange(6, dtype=np.float32).reshape(2, 3)], epoch=1)
    raw = open(p, "rb").read()
    (jl,) = struct.unpack(">I", raw[:4])
    if damage == "truncate_header":
        raw = raw[:2]
    elif damage == "truncate_body":
        raw = raw[:-5]
    elif damage == "trailing":
        raw = raw + b"\x00"
    elif damage == "bad_version":
        raw = raw[:4 + jl + 8] + b"\x02" + raw[4 + jl + 9:]
    elif damage == "count_mismatch":
        raw = raw.replace(b'"model_params_count":1', b'"model_params_count":2')
    elif damage in ("huge_count", "wrapping_shape"):
        # after the JSON: u64 tensor count, u8 version, u64 ndim, the dims, u64 element count, the elements.
        # Sizes come from the file: an element count whose byte size wraps around 2^64, or a shape whose product
        # does, must be refused with a status, not reach an allocation.
        o = 4 + jl + 8 + 1 + 8
        d0, d1, cnt = ((1 << 62), 1, (1 << 62)) if damage == "huge_count" else ((1 << 62), 4, 0)
        raw = raw[:o] + struct.pack("<QQQ", d0, d1, cnt) + raw[o + 24:]
    if damage == "missing":
        os.remove(p)
    else:
        open(p, "wb").write(raw)
    with pytest.raises(_lib.HxError) as e:
        checkpoint.read(p)
    assert e.value.variant == ("InvalidCheckpoint" if damage == "count_mismatch" else "SerializationError")
