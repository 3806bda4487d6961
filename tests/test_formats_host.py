"""CPU check of the planar re-layout and the exact decoders the CUDA kernels use (compiled for the host from the same
header): bit-identical to the oracle for every format, through both the block-wise repack and the per-byte map."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import oracle_lib as ol
from dwarfstar_red_lite_b200 import synth

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def hostlib(tmp_path_factory):
    so = str(tmp_path_factory.mktemp("hostfmt") / "libhostfmt.so")
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-shared", "-fPIC", "-ffp-contract=off", "-o", so, os.path.join(HERE, "host_formats_check.cpp")])
    return C.CDLL(so)


@pytest.mark.parametrize("t", [synth.Q6_K, synth.IQ2_XXS, synth.IQ3_S])
@pytest.mark.parametrize("use_map", [0, 1])
def test_planar_decode_bit_exact(hostlib, t, use_map):
    g2, g3 = ol.codebooks()
    rng = np.random.default_rng(t * 7 + use_map)
    for nrows, ncols in ((3, 256), (5, 768), (4, 2048), (37, 512)):
        rows = synth.quant_matrix(rng, t, nrows, ncols, 1e-3, 4e-3)
        out = np.empty((nrows, ncols), np.float32)
        assert hostlib.host_repack_dequant(C.c_uint32(t), ol.ptr(rows, ol.u8p), C.c_uint32(nrows), C.c_uint32(ncols), ol.ptr(g2, ol.u8p),
                                           ol.ptr(g3, ol.u32p), C.c_int(use_map), ol.ptr(out, ol.f32p)) == 1
        want = ol.dequant_rows(t, rows, ncols)
        assert np.array_equal(out.view(np.uint32), want.view(np.uint32))
