"""Runs the conformance driver (oracle/conformance_main.cc): the reference's own operation core
-- register_candidate, prepare_candidate, run_prepared_operation with validate_launch_bindings,
compiled in place from the Cellerator tree -- driving the candidates of
cellerator_b200/host/b200_candidates.cc.  The binary exists only where that tree was available at
build time (it travels with the repository to the GPU machine)."""
import os
import subprocess

import pytest

from conftest import ROOT

BINARY = os.path.join(ROOT, "oracle", "_ref", "b200_conformance")


def _run(*args):
    if not os.path.exists(BINARY):
        pytest.skip("oracle/_ref/b200_conformance not built (needs the reference tree)")
    proc = subprocess.run([BINARY, *args], capture_output=True, text=True, timeout=300)
    print(proc.stdout[-4000:])
    return proc


def test_host_half_of_the_operation_core_seam():
    proc = _run("--host-only")
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "FAIL" not in proc.stdout and "PASS prepare without a device fails loudly" in proc.stdout


@pytest.mark.gpu
def test_reference_operation_core_drives_the_backend_on_the_gpu():
    proc = _run()
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "device: present" in proc.stdout
    for line in ("PASS run_prepared_operation(forward)", "PASS forward result within tolerance of the reference referee",
                 "PASS deterministic candidate: identical digest on a second run",
                 "PASS a launch with another structure epoch is stale", "PASS run_prepared_operation(transpose)",
                 "PASS transpose result within tolerance of the reference referee",
                 "PASS tensor transpose under the deterministic policy: the second run repeats every bit of the first",
                 "PASS tensor transpose under the deterministic policy within the fp32 bound"):
        assert line in proc.stdout, line
    assert "FAIL" not in proc.stdout
