"""The reference's engine loader and CPU forward built on Linux (oracle/Makefile: the reference's
own qwasar.c, qwasar_flash_cpu.c, ... with two stand-in headers for the macOS-only includes and a
host-memory backend), run on the reference's toy checkpoint and held to its oracle.json at the
bounds of the reference's own test (tests/test_flashnext.c:226-262)."""
import json
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("QWASAR_REF") or os.path.join(os.path.dirname(ROOT), "reference")   # beside this repository, as oracle/Makefile assumes
FIXTURE = os.path.join(REF, "tests", "fixtures", "flashnext-tiny-q4")
EXE = os.path.join(ROOT, "oracle", "_ref", "flash_toy_cpu")

TOY = os.path.join(ROOT, "oracle", "_ref", "flashnext-tiny-q4")
GPU_EXE = os.path.join(ROOT, "oracle", "_ref", "flash_toy_gpu")

needs_reference = pytest.mark.skipif(not os.path.isdir(FIXTURE), reason="the reference checkout (with its toy fixture) is not on this machine")


@needs_reference
def test_toy_checkpoint_reproduces_its_oracle_on_the_cpu():
    subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "ref"], check=True, stdout=subprocess.DEVNULL)
    r = subprocess.run([EXE, FIXTURE], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    res = json.loads(r.stdout.strip().splitlines()[-1])
    assert res["ok"] and res["tokens"] == 32 and res["attention_layers"] == 2
    assert res["layers_over_1e-3"] == 0 and res["argmax_flips"] == 0 and res["mask_entries_differ"] == 0
    assert res["worst_logit_abs"] < 2e-3


@pytest.mark.gpu
@pytest.mark.skipif(not (os.path.exists(GPU_EXE) and os.path.isdir(TOY)),
                    reason="oracle/_ref holds neither the driver nor the toy checkpoint (built where the reference checkout is)")
def test_reference_graph_code_encodes_the_attention_layer_on_the_cuda_backend():
    """The reference's encode_qsa_layer (qwasar_flash_graph.c:408-511), unmodified, with the engine
    loader and session code around it, on this repository's backend: both attention layers of the toy
    checkpoint, token by token past the selection budget and in multi-row chunks, against the
    reference's CPU layer -- outputs within 5e-3 of the scale, selected positions identical."""
    r = subprocess.run([GPU_EXE, TOY], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    res = json.loads(r.stdout.strip().splitlines()[-1])
    assert res["ok"] and res["attention_layers"] == 2
    assert res["token_by_token"]["mask_entries_differ"] == 0 and res["chunks"]["mask_entries_differ"] == 0
    assert res["token_by_token"]["worst_rel"] <= 5e-3 and res["chunks"]["worst_rel"] <= 5e-3
    assert res["token_by_token"]["steps_past_budget"] > 0 and res["chunks"]["rows_past_budget"] > 0
