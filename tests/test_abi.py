"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the header declares,
the ctypes structures match the C layout, and argument errors come back as the right
TensorError-mapped status without touching a GPU."""
import ctypes as C
import os
import re
import subprocess
import tempfile

import pytest

from helixml_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "helix_b200.h")


def declared_symbols():
    src = open(HEADER).read()
    return sorted(set(re.findall(r"^HX_API [^;(]*?\b(hx_\w+)\(", src, flags=re.M)))


def test_library_exports_every_declared_symbol():
    lib = L.lib()
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/helix_b200.h but not exported"
    assert set(names) == set(L.exported_symbols()), "ctypes prototypes and header disagree"


def test_struct_layout_matches_c():
    prog = r'''
#include <stdio.h>
#include <stddef.h>
#include "helix_b200.h"
int main(void) {
  printf("%zu %zu %zu %zu %zu %zu %zu %zu\n", sizeof(hx_scan_args), offsetof(hx_scan_args, x), offsetof(hx_scan_args, A),
         offsetof(hx_scan_args, seq_splits), sizeof(hx_mamba_block_args), offsetof(hx_mamba_block_args, workspace),
         sizeof(hx_mamba_step_args), offsetof(hx_mamba_step_args, h));
  return 0;
}'''
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "t.c")
        open(src, "w").write(prog)
        exe = os.path.join(d, "t")
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), src, "-o", exe], check=True)
        out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout.split()
    got = [int(v) for v in out]
    want = [C.sizeof(L.ScanArgs), L.ScanArgs.x.offset, L.ScanArgs.A.offset, L.ScanArgs.seq_splits.offset,
            C.sizeof(L.MambaBlockArgs), L.MambaBlockArgs.workspace.offset, C.sizeof(L.MambaStepArgs), L.MambaStepArgs.h.offset]
    assert got == want


def test_header_is_plain_c():
    # the boundary must be consumable from C (and from Rust bindgen): compile it as C99 with warnings on
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-fsyntax-only", "-x", "c", HEADER], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_version_and_status_names():
    lib = L.lib()
    assert b"helix_b200" in lib.hx_version()
    # same order as crates/tensor-core/src/error.rs:7-37
    for code, name in enumerate(L.STATUS_NAMES):
        assert lib.hx_status_name(code).decode() == name


def test_argument_errors_need_no_gpu():
    lib = L.lib()
    assert lib.hx_selective_scan_fwd(None, None) == 10  # InvalidInput
    a = L.ScanArgs()
    a.batch, a.seq_len, a.d_inner, a.d_state = 1, 4, 8, 300
    assert lib.hx_selective_scan_fwd(C.byref(a), None) == 2  # InvalidDimension
    assert b"d_state" in lib.hx_last_error()
    a.d_state = 16
    a.io_dtype = 7
    assert lib.hx_selective_scan_fwd(C.byref(a), None) == 4  # DTypeMismatch
    a.io_dtype = L.HX_F32
    assert lib.hx_selective_scan_fwd(C.byref(a), None) == 10  # NULL operands
    # empty problems succeed without a launch
    a.batch = 0
    assert lib.hx_selective_scan_fwd(C.byref(a), None) == 0
    assert lib.hx_s4_diag_fwd(None, None, None, None, None, None, None, 0, 5, 5, 64, L.HX_F32, None) == 0
    assert lib.hx_s4_diag_fwd(None, None, None, None, None, None, None, 1, 5, 5, 1000, L.HX_F32, None) == 2
    assert lib.hx_gemm_simt(None, 4, None, 4, None, None, 4, L.HX_F32, L.HX_F32, 2, 2, 8, 0, None) == 10
    assert lib.hx_gemm_simt(C.c_void_p(16), 4, C.c_void_p(16), 4, None, C.c_void_p(16), 4, L.HX_F32, L.HX_F32, 2, 2, 8, 0,
                            None) == 1  # lda < K: ShapeMismatch
    n = C.c_size_t(0)
    b = L.MambaBlockArgs()
    b.batch, b.seq_len, b.d_model, b.d_inner, b.d_state, b.d_conv, b.dt_rank = 2, 16, 64, 128, 16, 4, 4
    b.io_dtype = L.HX_F32
    assert lib.hx_mamba_block_workspace_bytes(C.byref(b), C.byref(n)) == 0 and n.value > 2 * 16 * 128 * 4 * 5
    b.d_conv = 9
    assert lib.hx_mamba_block_workspace_bytes(C.byref(b), C.byref(n)) == 2


def test_workspace_size_queries():
    lib = L.lib()
    a = L.ScanArgs()
    a.batch, a.seq_len, a.d_inner, a.d_state, a.io_dtype = 2, 4096, 128, 16, L.HX_BF16
    n = C.c_size_t(123)
    a.variant = L.SCAN_TILED
    assert lib.hx_selective_scan_workspace_bytes(C.byref(a), C.byref(n)) == 0 and n.value == 0
    a.variant, a.seq_splits = L.SCAN_SEQSPLIT, 4
    assert lib.hx_selective_scan_workspace_bytes(C.byref(a), C.byref(n)) == 0
    assert n.value >= 3 * 2 * 128 * 16 * 4
    assert lib.hx_s4_ref_workspace_bytes(100, 16) == 100 * 16 * 4
    st = L.MambaStepArgs()
    st.batch, st.d_model, st.d_inner, st.d_state, st.d_conv, st.dt_rank, st.io_dtype = 4, 64, 128, 16, 4, 4, L.HX_F32
    assert lib.hx_mamba_step_workspace_bytes(C.byref(st), C.byref(n)) == 0 and n.value >= 4 * (2 * 128 + 128 + 36 + 128) * 4
    st.d_conv = 5
    assert lib.hx_mamba_step_workspace_bytes(C.byref(st), C.byref(n)) == 2
    assert lib.hx_mamba_block_step(None, None) == 10
    assert lib.hx_gemm_bf16_cols(C.c_void_p(16), 8, C.c_void_p(16), 8, None, C.c_void_p(16), 8, L.HX_F32, 4, 4, 8, 1, 40, None) == 10


def test_errors_are_thread_local():
    import threading
    lib = L.lib()
    lib.hx_selective_scan_fwd(None, None)
    seen = {}

    def other():
        seen["msg"] = lib.hx_last_error()

    t = threading.Thread(target=other)
    t.start()
    t.join()
    assert seen["msg"] == b"" and b"NULL" in lib.hx_last_error()
