"""The committed outputs of the reference's own C (tests/golden/reference_vectors.npz, written by tests/golden/make_golden.py
from oracle/_ref) against (i) the CPU oracle — bit for bit, no reference sources needed — and (ii) the CUDA path through
the C ABI on the same seeded inputs (dequantisation bit-exact, row dots within the GEMV bound, router ids exact, engine
decode within the layer / logit bounds)."""
import importlib.util
import os

import numpy as np
import pytest

import oracle_lib as ol
from dwarfstar_red_lite_b200 import gguf_writer, synth

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
mg = importlib.util.module_from_spec(spec)
spec.loader.exec_module(mg)
GOLD = np.load(os.path.join(HERE, "golden", "reference_vectors.npz"))


@pytest.mark.parametrize("t,ncols", mg.QUANT_CASES)
def test_oracle_dequant_and_dot_equal_reference_outputs(t, ncols):
    rows, x = mg.quant_inputs(t, ncols)
    assert np.array_equal(ol.dequant_rows(t, rows, ncols).view(np.uint32), GOLD[f"deq_{t}_{ncols}"].view(np.uint32))
    assert np.array_equal(ol.rows_dot(t, rows, x), GOLD[f"dot_{t}_{ncols}"])


@pytest.mark.parametrize("t,ncols", mg.XS_CASES)
def test_oracle_routed_checker_types_equal_reference_outputs(t, ncols):
    rows, x = mg.quant_inputs(t, ncols)
    assert np.array_equal(ol.rows_dot(t, rows, x), GOLD[f"dot_{t}_{ncols}"])
    if ncols == 256:
        w = GOLD[f"weights_{t}_{ncols}"]
        deq = ol.dequant_rows(t, rows[:2], ncols)
        assert np.array_equal(deq.astype(np.float64), w)          # the reference's double weights are exactly floats


def test_oracle_router_equals_reference_outputs():
    logits = mg.router_inputs()
    for c in range(logits.shape[0]):
        ids, w, _ = ol.router_select(logits[c], 10)
        assert np.array_equal(ids, GOLD["router_ids"][c])
        assert np.array_equal(w.view(np.uint32), GOLD["router_w"][c].view(np.uint32))


def test_oracle_engine_decode_equals_reference_outputs():
    dims, sm = mg.engine_model()
    om = ol.OracleModel(sm, kv_f16=True)
    for step, tok in enumerate(GOLD["engine_tokens"]):
        lg = om.step(int(tok), threads=2)
        assert np.array_equal(lg.view(np.uint32), GOLD["engine_logits"][step].view(np.uint32)), step
        for l in range(dims.n_layer):
            assert np.array_equal(om.router_ids(l), GOLD["engine_router_ids"][step][l])
            assert np.array_equal(om.layer_out(l).view(np.uint32), GOLD["engine_layer_out"][step][l].view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("t,ncols", mg.XS_CASES)
def test_cuda_routed_checker_types_against_reference_outputs(t, ncols):
    import dwarfstar_red_lite_b200 as rc
    rows, x = mg.quant_inputs(t, ncols)
    deq = rc.quant_dequant_rows(t, rows, ncols).reshape(mg.ROWS, ncols)
    if ncols == 256:
        assert np.array_equal(deq[:2].astype(np.float64), GOLD[f"weights_{t}_{ncols}"])
    dots = rc.quant_matvec(t, rows, mg.ROWS, ncols, x)
    mag = np.abs(deq.astype(np.float64) * x.astype(np.float64)).sum(axis=1) + 1e-30
    assert np.max(np.abs(dots.astype(np.float64) - GOLD[f"dot_{t}_{ncols}"]) / mag) <= 2e-5


@pytest.mark.gpu
@pytest.mark.parametrize("t,ncols", mg.QUANT_CASES)
def test_cuda_dequant_and_matvec_against_reference_outputs(t, ncols):
    import dwarfstar_red_lite_b200 as rc
    rows, x = mg.quant_inputs(t, ncols)
    want = GOLD[f"deq_{t}_{ncols}"]
    got = rc.quant_dequant_rows(t, rows, ncols).reshape(mg.ROWS, ncols)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    dots = rc.quant_matvec(t, rows, mg.ROWS, ncols, x)
    mag = np.abs(want.astype(np.float64) * x.astype(np.float64)).sum(axis=1) + 1e-30
    assert np.max(np.abs(dots.astype(np.float64) - GOLD[f"dot_{t}_{ncols}"]) / mag) <= 2e-5


@pytest.mark.gpu
def test_cuda_router_against_reference_outputs():
    import dwarfstar_red_lite_b200 as rc
    logits = mg.router_inputs()
    ids, w = rc.router_select_softmax_topk(logits, 10)
    assert np.array_equal(ids, GOLD["router_ids"])
    assert np.allclose(w, GOLD["router_w"], rtol=2e-6, atol=1e-9)


@pytest.mark.gpu
def test_cuda_engine_decode_against_reference_outputs(tmp_path, monkeypatch):
    from dwarfstar_red_lite_b200.engine import Engine
    monkeypatch.setenv("RL_KV_F16", "1")
    dims, sm = mg.engine_model()
    path = str(tmp_path / "tiny.gguf")
    gguf_writer.write_gguf(path, sm)
    eng = Engine(path, context=dims.context)
    try:
        for step, tok in enumerate(GOLD["engine_tokens"]):
            lg = eng.step(int(tok))
            ref_l = GOLD["engine_logits"][step]
            for l in range(dims.n_layer):
                assert np.array_equal(eng.router_ids(l), GOLD["engine_router_ids"][step][l]), (step, l)
                a, b = eng.layer_out(l), GOLD["engine_layer_out"][step][l]
                assert np.max(np.abs(a - b)) <= 1e-3 * np.max(np.abs(b)), (step, l)
            assert np.max(np.abs(lg - ref_l)) <= 1e-3 * np.max(np.abs(ref_l)) + 1e-6
            assert int(np.argmax(lg)) == int(np.argmax(ref_l))
    finally:
        eng.close()
