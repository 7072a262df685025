"""qwasar_b200 -- B200 (sm_100a) backend for qwasar's gated GQA full-attention path.

The product is the C-ABI shared library built from csrc/ (declared in
include/qwasar_cuda.h).  This package is the thin Python host side: a ctypes
binding that keeps the reference's names and argument order (backend.py) and
the synthetic workload generators the benchmark and the tests share (synth.py).
There is no CPU implementation in here: without the built library, or without
a CUDA device, every entry point fails loudly."""
from .backend import Backend, QwRef, load_library, build_library, LIB_PATH  # noqa: F401
