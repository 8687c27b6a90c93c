"""helixml_b200: B200 (sm_100a) implementation of HelixML's state-space hot path
(MambaBlock selective scan, S4Block diagonal recurrence) behind a C ABI.

The compute lives in libhelix_b200.so (hand-written CUDA, built by helixml_b200.build).
This package is the thin host side: a ctypes binding (`_lib`), array-level wrappers over
torch device tensors (`ops`), and mirrors of the reference's module interface (`nn`).
There is no CPU fallback: importing `_lib` raises if the library is missing."""

__all__ = ["synth"]
