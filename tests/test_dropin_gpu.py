"""The reference's own test program with ONE translation unit exchanged: flash_attn_tc.cu left out, the
drop-in file csrc/dropin/flash_attn_tc_dropin.cu (its launch interface over this library) linked
instead. Its drivers (run_drivers.cu), its cuBLAS full-softmax checker (baseline_attention.cu,
attn_tests.cu:27-60) and its matrix of 13 shapes x 3 seeds x 4 modes (attn_tests.cu:70-87) then run
this repository's attention kernels through flash_attn_tc_forward / _combine, fp32 O, tile counters and
split-KV workspace included. Built by `make -C oracle dropin` where the reference sources are mounted;
skipped when the binary is not there."""
import os
import re
import subprocess

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

EXE = os.path.join(ROOT, "oracle", "_ref", "attn_tests_dropin")


@pytest.mark.timeout(700)
def test_reference_test_program_passes_with_this_librarys_kernels(torch_cuda):
    if not os.path.exists(EXE):
        pytest.skip("oracle/_ref/attn_tests_dropin is not built (needs the reference sources at build time)")
    r = subprocess.run([EXE], capture_output=True, text=True, timeout=600)
    tail = r.stdout[-3000:] + r.stderr[-2000:]
    assert r.returncode == 0, tail
    m = re.search(r"(\d+) passed, (\d+) failed, (\d+) skipped", r.stdout)
    assert m, tail
    assert int(m.group(2)) == 0, tail
    # 13 shapes x 3 seeds x 4 modes go through the tensor-core interface (the rest is the scalar v1 kernel)
    tc_lines, kernel = 0, None
    for line in r.stdout.splitlines():
        k = re.match(r"kernel=(\w+) ", line)
        if k:
            kernel = k.group(1)
        elif kernel == "tc" and line.rstrip().endswith("PASS"):
            tc_lines += 1
    assert tc_lines == 13 * 3 * 4, tc_lines


EXE_DRIVERS = os.path.join(ROOT, "oracle", "_ref", "attn_tests_dropin_drivers")


@pytest.mark.timeout(700)
def test_reference_test_program_passes_with_this_librarys_run_modes(torch_cuda):
    """Both translation units exchanged (make -C oracle dropin_drivers): every tensor-core configuration of the
    reference's run_mode goes through efa_run_mode with fp32 partial sums and output."""
    if not os.path.exists(EXE_DRIVERS):
        pytest.skip("oracle/_ref/attn_tests_dropin_drivers is not built")
    r = subprocess.run([EXE_DRIVERS], capture_output=True, text=True, timeout=600)
    tail = r.stdout[-3000:] + r.stderr[-2000:]
    assert r.returncode == 0, tail
    m = re.search(r"(\d+) passed, (\d+) failed, (\d+) skipped", r.stdout)
    assert m and int(m.group(2)) == 0, tail
    tc_lines, kernel = 0, None
    for line in r.stdout.splitlines():
        k = re.match(r"kernel=(\w+) ", line)
        if k:
            kernel = k.group(1)
        elif kernel == "tc" and line.rstrip().endswith("PASS"):
            tc_lines += 1
    assert tc_lines == 13 * 3 * 4, tc_lines
