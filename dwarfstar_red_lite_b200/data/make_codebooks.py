"""Regenerate codebooks.bin from the reference's own tables (run where the reference checker library is built).

The IQ2_XXS and IQ3_S codebooks are data of the GGML formats (the reference derives them from its pinned llama.cpp,
MIT licence: native/redlite_native_iq2_xxs.c:6-22, native/redlite_native_iq3_tables.h). They are not retyped: this
script calls rl_native_iq2_xxs_build_grid and reads the arrays of redlite_native_iq3_tables.h through
oracle/_ref/libredlite_ref.so, then stores them as raw little-endian bytes:

    [0, 2048)      IQ2_XXS grid, 256 entries x 8 magnitudes (uint8)
    [2048, 4096)   IQ3_S grid, 512 entries x 4 packed magnitudes (uint32)

and, for the further types of the same family (IQ3_XXS, IQ2_S, IQ4_XS: native/redlite_native_iq3.c:53-110), a second
file codebooks_iq3family.bin:

    [0, 1024)      IQ3_XXS grid, 256 entries x 4 packed magnitudes (uint32)
    [1024, 9216)   IQ2_S grid, 1024 entries x 8 packed magnitudes (uint64)
    [9216, 9232)   IQ4_NL values, 16 x int8

and, for the two types of the reference's routed-expert checker (IQ2_XS, IQ1_M: native/redlite_native_reference.c:116-176,
grids built by rl_native_quant_tables_init, native/redlite_native_tables.c:229), codebooks_iq2xs_iq1m.bin:

    [0, 4096)      IQ2_XS grid, 512 entries x 8 magnitudes (int8)
    [4096, 20480)  IQ1_M grid, 2048 entries x 8 values in {-1, 0, 1} (int8)

Usage: make -C oracle ref && python dwarfstar_red_lite_b200/data/make_codebooks.py
"""
import ctypes
import os

here = os.path.dirname(os.path.abspath(__file__))
root = os.path.dirname(os.path.dirname(here))
ref = ctypes.CDLL(os.path.join(root, "oracle", "_ref", "libredlite_ref.so"), mode=ctypes.RTLD_LOCAL)

grid = (ctypes.c_uint8 * 2048)()
err = ctypes.create_string_buffer(256)
assert ref.rl_native_iq2_xxs_build_grid(grid, err, 256) == 1, err.value
ref.redcuda_ref_iq3s_grid.restype = ctypes.POINTER(ctypes.c_uint32)
n = ctypes.c_size_t(0)
p = ref.redcuda_ref_iq3s_grid(ctypes.byref(n))
assert n.value == 512
iq3s = bytes(ctypes.cast(p, ctypes.POINTER(ctypes.c_uint8 * 2048)).contents)
with open(os.path.join(here, "codebooks.bin"), "wb") as f:
    f.write(bytes(grid) + iq3s)
print("wrote codebooks.bin", 4096, "bytes")


def table(name, ctype, count):
    fn = getattr(ref, name)
    fn.restype = ctypes.POINTER(ctype)
    n = ctypes.c_size_t(0)
    p = fn(ctypes.byref(n))
    assert n.value == count, (name, n.value)
    return bytes(ctypes.cast(p, ctypes.POINTER(ctypes.c_uint8 * (count * ctypes.sizeof(ctype)))).contents)


fam = table("redcuda_ref_iq3xxs_grid", ctypes.c_uint32, 256) + table("redcuda_ref_iq2s_grid", ctypes.c_uint64, 1024) + table("redcuda_ref_iq4nl_values", ctypes.c_int8, 16)
with open(os.path.join(here, "codebooks_iq3family.bin"), "wb") as f:
    f.write(fam)
print("wrote codebooks_iq3family.bin", len(fam), "bytes")


class Tables(ctypes.Structure):
    _fields_ = [("iq2_xs", ctypes.POINTER(ctypes.c_int8)), ("iq1_m", ctypes.POINTER(ctypes.c_int8))]


tabs = Tables()
assert ref.rl_native_quant_tables_init(ctypes.byref(tabs), err, 256) == 1, err.value
two = bytes(ctypes.cast(tabs.iq2_xs, ctypes.POINTER(ctypes.c_uint8 * 4096)).contents) + bytes(ctypes.cast(tabs.iq1_m, ctypes.POINTER(ctypes.c_uint8 * 16384)).contents)
ref.rl_native_quant_tables_free(ctypes.byref(tabs))
with open(os.path.join(here, "codebooks_iq2xs_iq1m.bin"), "wb") as f:
    f.write(two)
print("wrote codebooks_iq2xs_iq1m.bin", len(two), "bytes")
