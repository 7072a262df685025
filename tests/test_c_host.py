"""The boundary from plain C: tests/c/attn_node.c is the reference's attention node written in C99
against include/qwasar_cuda.h (the op sequence of qw_encode_attention_layer, qwasar_graph.c:619-662,
and the fused call), compiled with -std=c99 -pedantic -Werror and linked against the library.  It
references every entry point the header declares, so a missing definition fails the link.

Without a GPU the program stops at qw_gpu_init with the library's message (exit 0): that is the
compile-and-link check.  On a GPU it runs both forms of the node and compares them with the
oracle (max rel err per output vector <= 1e-2, appended V bit-exact)."""
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "c", "attn_node.c")


@pytest.fixture(scope="module")
def attn_node(tmp_path_factory):
    import qwasar_b200  # noqa: F401  (the library must be built)
    from oracle import oracle as orc
    orc.Oracle()                                              # builds oracle/_build if needed
    exe = str(tmp_path_factory.mktemp("c") / "attn_node")
    libdir, ordir = os.path.join(ROOT, "qwasar_b200"), os.path.join(ROOT, "oracle", "_build")
    cmd = ["gcc", "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-O1", "-I" + os.path.join(ROOT, "include"), SRC, "-o", exe,
           "-L" + libdir, "-lqwasar_cuda", "-L" + ordir, "-lqworacle", "-lm", "-Wl,-rpath," + libdir, "-Wl,-rpath," + ordir]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_header_compiles_as_c99_and_every_entry_point_links(attn_node):
    header = open(os.path.join(ROOT, "include", "qwasar_cuda.h")).read()
    declared = set(re.findall(r"^[A-Za-z_][\w \*]*?\b(qw_\w+)\s*\(", header, flags=re.M)) - {"qw_ref_at", "qw_ref_offset"}
    listed = set(re.findall(r"\(any_fn\)(qw_\w+)", open(SRC).read()))
    assert declared == listed, (sorted(declared - listed), sorted(listed - declared))
    r = subprocess.run([attn_node], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert f"entry points referenced: {len(listed)}" in r.stdout
    assert "device:" in r.stdout or "qw_gpu_init:" in r.stdout    # a device, or the library's refusal without one


# the reference checkout: $QWASAR_REF, or beside this repository as oracle/Makefile assumes
REF_HEADER = os.path.join(os.environ.get("QWASAR_REF") or os.path.join(os.path.dirname(ROOT), "reference"), "qwasar_gpu.h")


@pytest.mark.skipif(not os.path.exists(REF_HEADER), reason="the reference checkout is not present on this machine")
def test_header_coexists_with_the_reference_header(tmp_path):
    """A translation unit of the reference includes qwasar_gpu.h first; this header must then add
    only what is new: every declaration the two share has to match, or -Werror stops the compile."""
    src = tmp_path / "both.c"
    src.write_text('#include "qwasar_gpu.h"\n#include "qwasar_cuda.h"\n'
                   "int main(void) { qw_qmv_part p; qw_ref r = qw_ref_at(NULL, 0); (void)p; (void)r;\n"
                   "  qw_prof_report(stderr, 0); qw_prof_reset(); return qw_gpu_sm_count(); }\n")
    libdir = os.path.join(ROOT, "qwasar_b200")
    cmd = ["gcc", "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-I" + os.path.dirname(REF_HEADER),
           "-I" + os.path.join(ROOT, "include"), str(src), "-o", str(tmp_path / "both"), "-L" + libdir, "-lqwasar_cuda",
           "-Wl,-rpath," + libdir]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("args", [[], ["1", "16", "4", "4096", "1"], ["40", "8", "2", "70", "3"], ["200", "16", "4", "0", "1"]],
                         ids=["verify-3-rows", "decode-4k", "chunk-40", "prefill-200"])
def test_node_from_c_matches_oracle(attn_node, args):
    r = subprocess.run([attn_node] + args, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr


@pytest.fixture(scope="module")
def two_gpu_node(tmp_path_factory):
    import qwasar_b200  # noqa: F401
    from oracle import oracle as orc
    orc.Oracle()
    exe = str(tmp_path_factory.mktemp("c2") / "two_gpu_node")
    libdir, ordir = os.path.join(ROOT, "qwasar_b200"), os.path.join(ROOT, "oracle", "_build")
    cmd = ["gcc", "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-O1", "-I" + os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "c", "two_gpu_node.c"), "-o", exe, "-L" + libdir, "-lqwasar_cuda", "-L" + ordir, "-lqworacle", "-lm",
           "-Wl,-rpath," + libdir, "-Wl,-rpath," + ordir]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_multi_gpu_host_compiles_as_c99(two_gpu_node):
    """tests/c/two_gpu_node.c -- one C99 thread driving several GPUs through the header -- builds
    -pedantic -Werror and, where fewer devices exist than it asks for, says so and exits 0."""
    r = subprocess.run([two_gpu_node], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("args", [["2", "3000", "16", "2"], ["2", "100", "24", "4"], ["4", "5000", "16", "2"]], ids=["2-gpus", "2-gpus-short", "4-gpus"])
def test_one_c_thread_drives_several_gpus(two_gpu_node, args):
    """A sequence split by position over the GPUs of one process: per-device arenas, the partials
    exchanged by peer stores (qw_op_attn_exchange), every device ends with the oracle's output."""
    import torch
    if torch.cuda.device_count() < int(args[0]):
        pytest.skip(f"needs {args[0]} GPUs")
    r = subprocess.run([two_gpu_node] + args, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr
