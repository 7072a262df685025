"""The drop-in boundary without a GPU: the library loads, exports every symbol the
header declares, and declines politely when no device can be brought up."""
import ctypes as C
import os
import re

import pytest

import qwasar_b200
from qwasar_b200 import backend

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "qwasar_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(qw_[a-z0-9_]+)\s*\(", text))
    return names - {"qw_ref_at", "qw_ref_offset"}          # static inline helpers


def test_library_is_built():
    assert os.path.exists(backend.LIB_PATH), "run `make -C qwasar_b200/csrc`"


def test_every_declared_symbol_is_exported():
    lib = C.CDLL(backend.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 50
    for n in sorted(names):
        assert hasattr(lib, n), f"{n} declared in include/qwasar_cuda.h but not exported"


def test_binding_covers_the_header():
    assert set(backend.SIGNATURES) == declared_symbols()


def test_reference_names_present():
    """The subset of qwasar_gpu.h the attention node calls (qwasar_graph.c:619-662)."""
    for n in ["qw_gpu_init", "qw_gpu_shutdown", "qw_buf_alloc", "qw_buf_wrap", "qw_buf_free", "qw_buf_contents",
              "qw_buf_length", "qw_cmd_begin", "qw_cmd_commit", "qw_cmd_wait", "qw_cmd_flush", "qw_cmd_parallel",
              "qw_cmd_free", "qw_cmd_error", "qw_op_split_heads2", "qw_op_rms_norm", "qw_op_rope_partial",
              "qw_rope_tables", "qw_op_kv_write", "qw_op_attn", "qw_op_attn_decode", "qw_op_attn_prefill",
              "qw_op_attn_prefill_as", "qw_op_attn_decode_split", "qw_op_attn_decode_tensor", "qw_op_mul_sigmoid"]:
        assert n in backend.SIGNATURES


def test_host_rope_tables_match_known_answers():
    """qw_rope_tables is host code in the backend (no device needed): tests/test_ops.c:163-182."""
    import numpy as np
    lib = backend.load_library()
    axis = np.zeros(32, np.uint8); inv = np.zeros(32, np.float32)
    sec = np.asarray([11, 11, 10], np.int32)
    lib.qw_rope_tables(axis.ctypes.data, inv.ctypes.data, 64, 1e7, sec.ctypes.data)
    assert axis.tolist() == [0, 1, 2] * 10 + [0, 1]
    assert abs(inv[1] - 0.6042963862) < 1e-7 and abs(inv[31] - 1.654816941254e-07) < 1e-13


def test_cache_element_tag_spells_bf16():
    lib = backend.load_library()
    assert int(lib.qw_kv_element_tag()).to_bytes(4, "little") == b"BF16"


def test_no_device_means_loud_failure():
    """Without a CUDA device init reports why, allocations return NULL and ops encode
    nothing -- there is no CPU path behind the ABI."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present; the failure path is for machines without one")
    lib = backend.load_library()
    err = C.create_string_buffer(256)
    assert lib.qw_gpu_init(err, 256) is False
    assert err.value
    assert lib.qw_buf_alloc(1024) is None
    assert lib.qw_cmd_begin() is None
    assert lib.qw_kv_arena_alloc(1, 1, 64, 256) is None
    with pytest.raises(RuntimeError):
        qwasar_b200.Backend()


def test_documented_knobs_are_the_accepted_ones():
    """Every knob the header documents (`"name" = a | b | c` in the comment above qw_gpu_tune) is
    accepted with each value it lists and refused with another; an unknown knob is refused.  Host
    state only: no device is touched.  The defaults are restored."""
    text = open(os.path.join(ROOT, "include", "qwasar_cuda.h")).read()
    doc = text[text.index("/* Diagnostic knobs"):text.index("qw_gpu_tune(const char *knob")]
    doc = re.sub(r"\n \* ?", " ", doc)
    knobs = {m.group(1): [int(v) for v in re.findall(r"\d+", m.group(2))]
             for m in re.finditer(r'"([a-z0-9_]+)" = (\d+(?: \| \d+)+)', doc)}
    assert set(knobs) >= {"split_kg", "split_kg2", "prefill_tc", "prefill_fuse_q", "pdl", "masked_tc", "qmv_tc", "qmv_pre", "qmm_tc"}
    lib = backend.load_library()
    try:
        for name, values in knobs.items():
            for v in values:
                assert lib.qw_gpu_tune(name.encode(), v), f'{name} = {v} is documented but refused'
            assert not lib.qw_gpu_tune(name.encode(), 97), f"{name} accepts a value the header does not list"
        assert not lib.qw_gpu_tune(b"no_such_knob", 1)
        assert not lib.qw_gpu_tune(None, 1)
    finally:
        for name, values in knobs.items():                      # back to the defaults: the first value listed, split_kg 6
            lib.qw_gpu_tune(name.encode(), 6 if name == "split_kg" else values[0])
