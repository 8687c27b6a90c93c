"""ctypes binding of include/helix_b200.h.  Loading fails loudly when the shared library has
not been built: there is no CPU or PyTorch fallback for any entry point."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libhelix_b200.so")

HX_OK = 0
HX_F32, HX_BF16, HX_U8 = 0, 1, 2
SCAN_AUTO, SCAN_SIMPLE, SCAN_TILED, SCAN_SEQSPLIT, SCAN_DIRECT, SCAN_LOOKBACK = 0, 1, 2, 3, 4, 5
EPI_NONE, EPI_SILU, EPI_SOFTPLUS, EPI_SILU_FAST = 0, 1, 2, 3

STATUS_NAMES = ["Ok", "ShapeMismatch", "InvalidDimension", "DeviceMismatch", "DTypeMismatch", "UnsupportedOperation",
                "AllocationFailed", "BackendError", "SerializationError", "InvalidCheckpoint", "InvalidInput"]


class HxError(RuntimeError):
    """A non-zero hx_status; `.status` is the code, `.variant` the TensorError variant it maps to."""

    def __init__(self, status: int, message: str):
        self.status = status
        self.variant = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else "Unknown"
        super().__init__(f"{self.variant}: {message}")


class ScanArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("seq_len", C.c_int32), ("d_inner", C.c_int32), ("d_state", C.c_int32),
        ("d_conv", C.c_int32), ("io_dtype", C.c_int32), ("dt_softplus", C.c_int32), ("variant", C.c_int32),
        ("x", C.c_void_p), ("dt", C.c_void_p), ("z", C.c_void_p), ("Bm", C.c_void_p), ("Cm", C.c_void_p),
        ("y", C.c_void_p),
        ("x_batch_stride", C.c_int64), ("x_row_stride", C.c_int64),
        ("dt_batch_stride", C.c_int64), ("dt_row_stride", C.c_int64),
        ("z_batch_stride", C.c_int64), ("z_row_stride", C.c_int64),
        ("B_batch_stride", C.c_int64), ("B_row_stride", C.c_int64),
        ("C_batch_stride", C.c_int64), ("C_row_stride", C.c_int64),
        ("y_batch_stride", C.c_int64), ("y_row_stride", C.c_int64),
        ("A", C.c_void_p), ("Dskip", C.c_void_p), ("conv_w", C.c_void_p), ("conv_b", C.c_void_p),
        ("dt_bias", C.c_void_p), ("h_last", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("seq_splits", C.c_int32), ("a_geometric", C.c_int32), ("lanes_per_channel", C.c_int32),
        ("reserved", C.c_int32),
        ("dt_low", C.c_void_p), ("W_dt", C.c_void_p), ("dt_low_batch_stride", C.c_int64), ("dt_low_row_stride", C.c_int64),
        ("dt_rank", C.c_int32), ("z_is_gate", C.c_int32),
    ]


class MambaBlockArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("seq_len", C.c_int32), ("d_model", C.c_int32), ("d_inner", C.c_int32),
        ("d_state", C.c_int32), ("d_conv", C.c_int32), ("dt_rank", C.c_int32), ("io_dtype", C.c_int32),
        ("x", C.c_void_p), ("out", C.c_void_p), ("W_in", C.c_void_p), ("W_x", C.c_void_p), ("W_dt", C.c_void_p),
        ("W_out", C.c_void_p), ("conv_w", C.c_void_p), ("conv_b", C.c_void_p), ("b_dt", C.c_void_p),
        ("A", C.c_void_p), ("Dskip", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("scan_variant", C.c_int32), ("a_geometric", C.c_int32), ("stage_events", C.c_void_p),
        ("h_last", C.c_void_p), ("conv_state", C.c_void_p), ("residual", C.c_void_p),
    ]


class CheckpointMeta(C.Structure):
    _fields_ = [("epoch", C.c_uint64), ("step", C.c_uint64), ("training_loss", C.c_double), ("validation_loss", C.c_double),
                ("learning_rate", C.c_double), ("timestamp_secs", C.c_uint64)]


class MambaStepArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("d_model", C.c_int32), ("d_inner", C.c_int32), ("d_state", C.c_int32),
        ("d_conv", C.c_int32), ("dt_rank", C.c_int32), ("io_dtype", C.c_int32), ("reserved", C.c_int32),
        ("x", C.c_void_p), ("out", C.c_void_p), ("W_in", C.c_void_p), ("W_x", C.c_void_p), ("W_dt", C.c_void_p),
        ("W_out", C.c_void_p), ("conv_w", C.c_void_p), ("conv_b", C.c_void_p), ("b_dt", C.c_void_p),
        ("A", C.c_void_p), ("Dskip", C.c_void_p), ("h", C.c_void_p), ("conv_state", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("residual", C.c_void_p), ("norm_w", C.c_void_p), ("norm_eps", C.c_float), ("reserved2", C.c_int32),
    ]


class GatherArgs(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("batch", C.c_int32), ("seq_len", C.c_int32),
                ("d_shard", C.c_int32), ("d_full", C.c_int32), ("col0", C.c_int32), ("io_dtype", C.c_int32),
                ("y_local", C.c_void_p), ("dst", C.c_void_p * 8), ("row_begin", C.c_int32), ("row_end", C.c_int32),
                ("max_ctas_per_sm", C.c_int32), ("reserved", C.c_int32)]


_PROTOS = {
    "hx_version": (C.c_char_p, []),
    "hx_last_error": (C.c_char_p, []),
    "hx_status_name": (C.c_char_p, [C.c_int]),
    "hx_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "hx_set_device": (C.c_int, [C.c_int]),
    "hx_alloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "hx_free": (C.c_int, [C.c_void_p]),
    "hx_host_alloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "hx_host_free": (C.c_int, [C.c_void_p]),
    "hx_memcpy_h2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "hx_memcpy_d2h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "hx_memset": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_void_p]),
    "hx_stream_synchronize": (C.c_int, [C.c_void_p]),
    "hx_selective_scan_fwd": (C.c_int, [C.POINTER(ScanArgs), C.c_void_p]),
    "hx_selective_scan_workspace_bytes": (C.c_int, [C.POINTER(ScanArgs), C.POINTER(C.c_size_t)]),
    "hx_selective_scan_suggest_splits": (C.c_int32, [C.POINTER(ScanArgs)]),
    "hx_selective_scan_host": (C.c_int, [C.POINTER(ScanArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "hx_selective_scan_host_workspace_bytes": (C.c_int, [C.POINTER(ScanArgs), C.POINTER(C.c_size_t)]),
    "hx_selective_scan_fwd_noalloc": (C.c_int, [C.POINTER(ScanArgs), C.c_void_p]),
    "hx_scan_check_geometric": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_int32)]),
    "hx_device_status": (C.c_int, [C.POINTER(C.c_int32), C.c_int32]),
    "hx_device_check": (C.c_int, []),
    "hx_debug_scan_orphan_segment": (C.c_int, [C.POINTER(ScanArgs), C.c_int32, C.c_void_p]),
    "hx_ipc_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "hx_ipc_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "hx_ipc_close": (C.c_int, [C.c_void_p]),
    "hx_allgather_y_push": (C.c_int, [C.POINTER(GatherArgs), C.c_void_p]),
    "hx_probe_pipe": (C.c_int, [C.c_int32, C.c_void_p, C.c_size_t, C.POINTER(C.c_double), C.c_void_p]),
    "hx_conv1d_silu_fwd": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                     C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "hx_s4_diag_fwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "hx_s4_ref_forward_ssm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float,
                                        C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_size_t,
                                        C.c_void_p]),
    "hx_s4_ref_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32]),
    "hx_mamba_ssm_ref_forward": (C.c_int, [C.c_void_p] * 9 + [C.c_int32, C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p]),
    "hx_mamba_ssm_ref_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32]),
    "hx_gemm_bf16": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                               C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "hx_gemm_bf16_acc": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                   C.c_int32, C.c_void_p]),
    "hx_gemm_bf16_cols": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                                    C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "hx_gemm_pair_mode": (C.c_int, [C.c_int32, C.c_void_p]),
    "hx_conv1d_silu_xproj_fwd": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                           C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                           C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "hx_gemm_simt": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                               C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "hx_rmsnorm_fwd": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64,
                                 C.c_int32, C.c_float, C.c_void_p]),
    "hx_embedding_fwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int64, C.c_int32,
                                   C.c_void_p]),
    "hx_silu_fwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p]),
    "hx_mamba_block_fwd": (C.c_int, [C.POINTER(MambaBlockArgs), C.c_void_p]),
    "hx_mamba_block_kernel_launches": (C.c_int, [C.POINTER(MambaBlockArgs), C.POINTER(C.c_int32)]),
    "hx_mamba_block_step": (C.c_int, [C.POINTER(MambaStepArgs), C.c_void_p]),
    "hx_mamba_step_workspace_bytes": (C.c_int, [C.POINTER(MambaStepArgs), C.POINTER(C.c_size_t)]),
    "hx_conv_state_from_prefill": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                             C.c_int32, C.c_void_p]),
    "hx_mamba_block_workspace_bytes": (C.c_int, [C.POINTER(MambaBlockArgs), C.POINTER(C.c_size_t)]),
    # ---- module-level API
    "hx_manual_seed": (None, [C.c_uint64]),
    "hx_tensor_from_host": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_tensor_from_host_u8": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_tensor_to_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64]),
    "hx_tensor_copy_from_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64]),
    "hx_tensor_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int64), C.POINTER(C.c_int32),
                                 C.POINTER(C.c_int32)]),
    "hx_tensor_data": (C.c_void_p, [C.c_void_p]),
    "hx_tensor_free": (None, [C.c_void_p]),
    # ---- tensor primitives (TensorOps / TensorBroadcast / TensorActivation / TensorRandom / TensorMixedPrecision)
    "hx_tensor_binary": (C.c_int, [C.c_int32, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]),
    "hx_tensor_unary": (C.c_int, [C.c_int32, C.c_void_p, C.c_float, C.c_float, C.POINTER(C.c_void_p)]),
    "hx_tensor_matmul": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]),
    "hx_matmul_ref": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "hx_tensor_transpose": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.POINTER(C.c_void_p)]),
    "hx_tensor_slice": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_tensor_cat": (C.c_int, [C.POINTER(C.c_void_p), C.c_int32, C.c_int64, C.POINTER(C.c_void_p)]),
    "hx_tensor_stack": (C.c_int, [C.POINTER(C.c_void_p), C.c_int32, C.c_int64, C.POINTER(C.c_void_p)]),
    "hx_tensor_reshape": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_tensor_clone": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "hx_tensor_broadcast_to": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_tensor_cast": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_tensor_to_scalar": (C.c_int, [C.c_void_p, C.POINTER(C.c_float)]),
    "hx_tensor_full": (C.c_int, [C.c_float, C.POINTER(C.c_int64), C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_tensor_eye": (C.c_int, [C.c_int64, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_tensor_arange": (C.c_int, [C.c_float, C.c_float, C.c_float, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_tensor_random": (C.c_int, [C.c_int32, C.POINTER(C.c_int64), C.c_int32, C.c_float, C.c_float, C.c_int32,
                                   C.POINTER(C.c_void_p)]),
    "hx_mamba_block_new": (C.c_int, [C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_s4_block_new": (C.c_int, [C.c_int64, C.c_int64, C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_linear_new": (C.c_int, [C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_rmsnorm_new": (C.c_int, [C.c_int64, C.c_float, C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_sequential_new": (C.c_int, [C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_sequential_add": (C.c_int, [C.c_void_p, C.c_void_p]),
    "hx_sequential_len": (C.c_int32, [C.c_void_p]),
    "hx_byte_lm_new": (C.c_int, [C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32,
                                 C.POINTER(C.c_void_p)]),
    "hx_module_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]),
    "hx_s4_block_forward_ssm": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]),
    "hx_byte_lm_forward_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "hx_byte_lm_forward_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "hx_byte_lm_launches_per_forward": (C.c_int64, [C.c_void_p]),
    "hx_module_save_checkpoint": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(CheckpointMeta)]),
    "hx_module_load_checkpoint": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(CheckpointMeta)]),
    "hx_checkpoint_write": (C.c_int, [C.c_char_p, C.POINTER(CheckpointMeta), C.c_int32, C.POINTER(C.c_void_p),
                                      C.POINTER(C.c_void_p), C.POINTER(C.c_int32)]),
    "hx_checkpoint_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "hx_checkpoint_num_tensors": (C.c_int32, [C.c_void_p]),
    "hx_checkpoint_meta_get": (C.c_int, [C.c_void_p, C.POINTER(CheckpointMeta)]),
    "hx_checkpoint_tensor": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_int32)]),
    "hx_checkpoint_close": (None, [C.c_void_p]),
    "hx_byte_lm_prefill_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "hx_byte_lm_decode_step_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "hx_byte_lm_decode_graph": (C.c_int, [C.c_void_p, C.c_int32]),
    "hx_byte_lm_forward_graph": (C.c_int, [C.c_void_p, C.c_int32]),
    "hx_byte_lm_launches_per_decode_step": (C.c_int64, [C.c_void_p]),
    "hx_byte_lm_profile": (C.c_int, [C.c_void_p, C.c_int32]),
    "hx_byte_lm_profile_read": (C.c_int, [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_int32)]),
    "hx_module_num_parameters": (C.c_int32, [C.c_void_p]),
    "hx_module_parameter": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(C.c_void_p)]),
    "hx_module_parameters_updated": (C.c_int, [C.c_void_p]),
    "hx_module_name": (C.c_char_p, [C.c_void_p]),
    "hx_module_free": (None, [C.c_void_p]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library.  Raises (never falls back) when it is missing or lacks a symbol."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m helixml_b200.build` (there is no fallback path)")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in _PROTOS.items():
            fn = getattr(l, name)  # AttributeError if the symbol is absent
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def exported_symbols():
    return sorted(_PROTOS)


def check(status: int) -> None:
    if status != HX_OK:
        raise HxError(status, lib().hx_last_error().decode())


def check_device() -> None:
    """Raises HxError (BackendError) when a bounded device-side wait ran out since the last check."""
    check(lib().hx_device_check())


def device_status(clear: bool = True) -> int:
    v = C.c_int32(0)
    check(lib().hx_device_status(C.byref(v), 1 if clear else 0))
    return v.value
