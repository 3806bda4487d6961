"""The decoder of the five codebook types served from their file layout (csrc/redcuda_kquants_iq.cuh) is one inline function
compiled for host and device. Here nvcc compiles it for the host and every value of 4096 random blocks per type (special
block scales included: zero, subnormal, negative, the largest finite half) is compared bit for bit with the oracle's
dequantiser, which tests/test_oracle_pin.py pins against the reference. No GPU is needed."""
import os
import shutil
import subprocess

import pytest

import oracle_lib as ol

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="nvcc not on PATH")
def test_codebook_type_decoder_on_the_host(tmp_path):
    ol.own()                                   # builds / loads the oracle library
    exe = str(tmp_path / "kq_iq_host_check")
    src = os.path.join(ROOT, "tests", "kq_iq_host_check.cu")
    inc = os.path.join(ROOT, "dwarfstar_red_lite_b200", "csrc")
    subprocess.run(["nvcc", "-O2", "-std=c++17", "-Wno-deprecated-gpu-targets", "-Xcompiler", "-ffp-contract=off", "-I", inc, "-o", exe, src, "-ldl"],
                   check=True, capture_output=True, text=True)
    data = os.path.join(ROOT, "dwarfstar_red_lite_b200", "data")
    out = subprocess.run([exe, os.path.join(ROOT, "oracle", "libredcuda_oracle.so"), os.path.join(data, "codebooks_iq3family.bin"),
                          os.path.join(data, "codebooks_iq2xs_iq1m.bin")], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    for t in (17, 18, 22, 23, 29):
        assert f"type {t}: 0 of 1048576 values differ" in out.stdout, out.stdout
