"""Checkpoint files in the reference's layout (crates/training/src/checkpoint.rs:136-197) for tensors held on
the host: thin ctypes wrappers over hx_checkpoint_write / hx_checkpoint_open.  No GPU is involved."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L


def _meta(epoch=0, step=0, training_loss=0.0, validation_loss=0.0, learning_rate=0.0, timestamp_secs=0) -> L.CheckpointMeta:
    m = L.CheckpointMeta()
    m.epoch, m.step, m.timestamp_secs = epoch, step, timestamp_secs
    m.training_loss, m.validation_loss, m.learning_rate = training_loss, validation_loss, learning_rate
    return m


def meta_dict(m: L.CheckpointMeta) -> dict:
    return {k: getattr(m, k) for k, _ in L.CheckpointMeta._fields_}


def write(path: str, arrays, **meta) -> None:
    """Writes fp32 arrays (any rank up to 8) as the checkpoint's Vec<CpuTensor>."""
    arrs = [np.ascontiguousarray(a, dtype=np.float32) for a in arrays]
    n = len(arrs)
    data = (C.c_void_p * max(n, 1))(*[a.ctypes.data for a in arrs])
    dim_arrays = [np.asarray(a.shape, dtype=np.int64) for a in arrs]
    dims = (C.c_void_p * max(n, 1))(*[d.ctypes.data for d in dim_arrays])
    ndims = (C.c_int32 * max(n, 1))(*[a.ndim for a in arrs])
    m = _meta(**meta)
    L.check(L.lib().hx_checkpoint_write(path.encode(), C.byref(m), n, data, dims, ndims))


def read(path: str):
    """Returns (meta dict, list of fp32 arrays)."""
    h = C.c_void_p()
    L.check(L.lib().hx_checkpoint_open(path.encode(), C.byref(h)))
    try:
        m = L.CheckpointMeta()
        L.check(L.lib().hx_checkpoint_meta_get(h, C.byref(m)))
        out = []
        for i in range(L.lib().hx_checkpoint_num_tensors(h)):
            data, dims, nd = C.c_void_p(), C.c_void_p(), C.c_int32()
            L.check(L.lib().hx_checkpoint_tensor(h, i, C.byref(data), C.byref(dims), C.byref(nd)))
            shape = tuple(np.ctypeslib.as_array(C.cast(dims, C.POINTER(C.c_int64)), (nd.value,)).tolist()) if nd.value else ()
            numel = int(np.prod(shape)) if shape else 1
            if numel:
                a = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_float)), (numel,)).copy().reshape(shape)
            else:
                a = np.zeros(shape, np.float32)
            out.append(a)
        return meta_dict(m), out
    finally:
        L.lib().hx_checkpoint_close(h)
