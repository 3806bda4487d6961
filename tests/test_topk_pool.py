"""The reference's expert-pool ABI v1 (native/redmetal_topk.h:11-245) on the CUDA backend: the entry points its portable
expert runtime links (native/redlite_native_metal.c) exist under the same names, keep the counters that runtime reads,
and redmetal_topk_pool_execute agrees with the oracle's routed-expert sum within the bound of the reference's own
top-k parity driver (1e-3 + 1e-4 |cpu|, native/redlite_native_main.c:416)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import oracle_lib as ol
import dwarfstar_red_lite_b200 as rc
from dwarfstar_red_lite_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
u32p, u64p, f32p = C.POINTER(C.c_uint32), C.POINTER(C.c_uint64), C.POINTER(C.c_float)


def _declared():
    text = open(os.path.join(ROOT, "include", "redmetal_topk.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(redmetal_topk_[a-z0-9_]+)\s*\(", text)))


def test_every_pool_symbol_is_exported_and_abi_is_1():
    lib = rc.lib()
    names = _declared()
    assert len(names) >= 22
    assert not [n for n in names if not hasattr(lib, n)]
    lib.redmetal_topk_abi_version.restype = C.c_uint32
    assert lib.redmetal_topk_abi_version() == 1          # the runtime refuses any other value (native/redlite_native_metal.c:63)


def _bind(lib):
    lib.redmetal_topk_pool_create.restype = C.c_void_p
    lib.redmetal_topk_pool_create.argtypes = [C.c_char_p, C.c_uint64, C.c_uint64, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32]
    lib.redmetal_topk_pool_destroy.argtypes = [C.c_void_p]
    for n in ("capacity", "slab_count"):
        getattr(lib, "redmetal_topk_pool_" + n).restype = C.c_uint32
        getattr(lib, "redmetal_topk_pool_" + n).argtypes = [C.c_void_p]
    for n in ("allocated_bytes", "bytes_read", "read_calls"):
        getattr(lib, "redmetal_topk_pool_" + n).restype = C.c_uint64
        getattr(lib, "redmetal_topk_pool_" + n).argtypes = [C.c_void_p]
    lib.redmetal_topk_pool_slot_generation.restype = C.c_uint32
    lib.redmetal_topk_pool_slot_generation.argtypes = [C.c_void_p, C.c_uint32]
    lib.redmetal_topk_pool_slot_inflight.argtypes = [C.c_void_p, C.c_uint32]
    lib.redmetal_topk_pool_load_expert.argtypes = [C.c_void_p, C.c_uint32] + [C.c_uint64] * 6 + [u64p, C.POINTER(C.c_double)]
    lib.redmetal_topk_pool_execute.argtypes = [C.c_void_p, u32p, u64p, u64p, u64p, f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                               f32p, C.c_uint32, f32p, C.c_uint32, C.POINTER(C.c_double)]
    lib.redmetal_topk_pool_release.argtypes = [C.c_void_p, u32p, C.c_uint32]
    lib.redmetal_topk_pool_residency_table_init.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32]
    lib.redmetal_topk_pool_residency_table.restype = C.c_void_p
    lib.redmetal_topk_pool_residency_table.argtypes = [C.c_void_p]
    lib.redmetal_topk_pool_residency_set.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32]
    lib.redmetal_topk_pool_residency_clear.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32]
    lib.redmetal_topk_last_error.restype = C.c_char_p
    return lib


@pytest.mark.gpu
@pytest.mark.parametrize("te", [synth.IQ2_XXS, synth.IQ3_S])
def test_pool_load_execute_release_against_oracle(tmp_path, te):
    rc.set_codebooks()
    lib = _bind(rc.lib())
    dims = synth.MoeDims(hidden=512, n_expert=12, top_k=4, ffn=256, ffn_sh=256, type_gu=te, type_down=te)
    layer = synth.moe_layer(70 + te, dims, expert_scale=0.5)
    gu_b, dn_b = layer.gate[0].nbytes, layer.down[0].nbytes
    # a "model file": the three expert tensors back to back, expert-major as in a GGUF
    path = tmp_path / "experts.bin"
    blob = np.concatenate([layer.gate.reshape(-1), layer.up.reshape(-1), layer.down.reshape(-1)])
    blob.tofile(path)
    off_g, off_u, off_d = 0, layer.gate.nbytes, layer.gate.nbytes + layer.up.nbytes
    slot_bytes = (2 * gu_b + dn_b + 15) // 16 * 16
    pool = lib.redmetal_topk_pool_create(str(path).encode(), slot_bytes * 8, slot_bytes, 4, None, 0, None, 0)
    assert pool, lib.redmetal_topk_last_error()
    try:
        assert lib.redmetal_topk_pool_capacity(pool) == 8 and lib.redmetal_topk_pool_slab_count(pool) == 0
        experts, slots = [9, 2, 11, 5], [3, 0, 7, 4]          # experts land in arbitrary slots
        got_b, ms = C.c_uint64(0), C.c_double(0)
        for e, s in zip(experts, slots):
            assert lib.redmetal_topk_pool_load_expert(pool, s, off_g + e * gu_b, gu_b, off_u + e * gu_b, gu_b, off_d + e * dn_b, dn_b, C.byref(got_b), C.byref(ms)) == 1, \
                lib.redmetal_topk_last_error()
            assert got_b.value == 2 * gu_b + dn_b and lib.redmetal_topk_pool_slot_generation(pool, s) == 1
        assert lib.redmetal_topk_pool_bytes_read(pool) == 4 * (2 * gu_b + dn_b) and lib.redmetal_topk_pool_read_calls(pool) == 12
        assert lib.redmetal_topk_pool_slab_count(pool) == 1 and lib.redmetal_topk_pool_allocated_bytes(pool) == 8 * slot_bytes
        assert lib.redmetal_topk_pool_slot_generation(pool, 1) == 0 and lib.redmetal_topk_pool_slot_inflight(pool, 3) == 0
        rng = np.random.default_rng(4)
        x = rng.normal(0, 1, dims.hidden).astype(np.float32)
        w = rng.uniform(0.05, 0.4, 4).astype(np.float32)
        sl = np.array(slots, np.uint32)
        gb, db = np.full(4, gu_b, np.uint64), np.full(4, dn_b, np.uint64)
        want = ol.routed_experts(layer, np.array(experts, np.uint32), w, x, threads=4)
        for row0, nrow in ((0, dims.hidden), (64, 200)):        # the whole output and a row range
            out = np.zeros(nrow, np.float32)
            ok = lib.redmetal_topk_pool_execute(pool, sl.ctypes.data_as(u32p), gb.ctypes.data_as(u64p), gb.ctypes.data_as(u64p), db.ctypes.data_as(u64p),
                                                w.ctypes.data_as(f32p), 4, te, dims.hidden, dims.ffn, row0, nrow, x.ctypes.data_as(f32p), dims.hidden,
                                                out.ctypes.data_as(f32p), nrow, C.byref(ms))
            assert ok == 1, lib.redmetal_topk_last_error()
            ref = want[row0:row0 + nrow]
            assert np.all(np.abs(out - ref) <= 1e-3 + 1e-4 * np.abs(ref)), float(np.max(np.abs(out - ref)))
        # an empty slot is refused, not read
        bad = np.array([3, 0, 7, 1], np.uint32)
        out = np.zeros(dims.hidden, np.float32)
        assert lib.redmetal_topk_pool_execute(pool, bad.ctypes.data_as(u32p), gb.ctypes.data_as(u64p), gb.ctypes.data_as(u64p), db.ctypes.data_as(u64p),
                                              w.ctypes.data_as(f32p), 4, te, dims.hidden, dims.ffn, 0, dims.hidden, x.ctypes.data_as(f32p), dims.hidden,
                                              out.ctypes.data_as(f32p), dims.hidden, C.byref(ms)) == 0
        assert b"empty" in lib.redmetal_topk_last_error()
        # residency table: addresses of resident slots, zero elsewhere
        import torch
        assert lib.redmetal_topk_pool_residency_table_init(pool, 2, 12) == 1
        assert lib.redmetal_topk_pool_residency_set(pool, 1, 9, 3) == 1

        class _Dev:           # the table as a torch view of the library's device memory
            __cuda_array_interface__ = {"shape": (24,), "typestr": "<i8", "data": (int(lib.redmetal_topk_pool_residency_table(pool)), False), "version": 2}
        tab = torch.as_tensor(_Dev(), device="cuda").cpu().numpy()
        assert tab[12 + 9] != 0 and int(np.count_nonzero(tab)) == 1
        lib.redmetal_topk_pool_residency_clear(pool, 1, 9)
        lib.redmetal_topk_pool_release(pool, sl.ctypes.data_as(u32p), 4)
        assert lib.redmetal_topk_pool_slot_inflight(pool, 3) == 0
    finally:
        lib.redmetal_topk_pool_destroy(pool)
