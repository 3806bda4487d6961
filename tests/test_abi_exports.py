"""The C-ABI library loads without a GPU and exports every symbol the public headers declare (no compute calls)."""
import os
import re

import dwarfstar_red_lite_b200 as rc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b((?:redcuda|rl_engine)_[a-z0-9_]+)\s*\(", text))


def test_every_declared_symbol_is_exported():
    lib = rc.lib()
    declared = _declared("redcuda.h") | _declared("rl_engine.h")
    assert len(declared) >= 35
    missing = sorted(n for n in declared if not hasattr(lib, n))
    assert not missing, missing
    assert set(rc.redcuda.EXPORTS) <= declared


def test_abi_version_and_loud_failure_without_device():
    lib = rc.lib()
    assert lib.redcuda_abi_version() == 1
    if lib.redcuda_device_count() == 0:
        import numpy as np
        import pytest
        with pytest.raises(rc.RedcudaError):
            rc.quant_matvec(16, np.zeros(66, np.uint8), 1, 256, np.zeros(256, np.float32))


def _prototypes(header):
    """{name: number of parameters} of every function a header declares."""
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    out = {}
    for name, params in re.findall(r"\b((?:redcuda|rl_engine)_[a-z0-9_]+)\s*\(([^()]*)\)\s*;", text):
        params = params.strip()
        out[name] = 0 if params in ("", "void") else params.count(",") + 1
    return out


def test_python_bindings_declare_every_signature():
    """ctypes passes an undeclared Python int as a 32-bit C int, which cuts a pointer in half: every function the Python
    side calls with arguments has its argtypes set, with as many entries as the header's prototype has parameters."""
    from dwarfstar_red_lite_b200 import engine as eng_mod
    lib = eng_mod._bind()
    protos = {**_prototypes("redcuda.h"), **_prototypes("rl_engine.h")}
    called = set(rc.redcuda.EXPORTS) | set(eng_mod.ENGINE_EXPORTS)
    bad = []
    for name in sorted(called):
        assert name in protos, name
        fn = getattr(lib, name)
        if protos[name] and (fn.argtypes is None or len(fn.argtypes) != protos[name]):
            bad.append((name, protos[name], None if fn.argtypes is None else len(fn.argtypes)))
    assert not bad, bad
