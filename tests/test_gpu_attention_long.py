"""Decode and chunked-prefill attention at long sequence lengths against the CPU oracle, with the protocol of the
reference's kernel self-test (lengths 1, 200, 256, 257, 1024, 1500 against a double-precision GQA,
native/redmetal_engine_selftest.m:213-215): the lengths straddle the points where the split-K decode kernel changes its
slicing. The model is small everywhere except in the attention layer, which has the full head shape (16 query heads,
2 K/V heads, head_dim 256, partial NeoX RoPE over 64 dims), and the context is 2048 positions."""
import os

import numpy as np
import pytest

import oracle_lib as ol
from dwarfstar_red_lite_b200 import gguf_writer, synth
from dwarfstar_red_lite_b200.engine import Engine

pytestmark = pytest.mark.gpu

LENGTHS = (1, 200, 256, 257, 1024, 1500)
REL_OUT = 1e-3


def _compare(eng, om, dims, gl, ml, tag):
    for l in range(dims.n_layer):
        assert np.array_equal(eng.router_ids(l), om.router_ids(l)), (tag, l)
        a, b = eng.layer_out(l), om.layer_out(l)
        assert np.max(np.abs(a - b)) <= REL_OUT * np.max(np.abs(b)), (tag, l, float(np.max(np.abs(a - b)) / np.max(np.abs(b))))
    assert np.max(np.abs(gl - ml)) <= REL_OUT * np.max(np.abs(ml)) + 1e-6, tag
    assert int(np.argmax(gl)) == int(np.argmax(ml)), tag


@pytest.mark.parametrize("kv_f16", [1, 0])
def test_attention_at_long_context(tmp_path, kv_f16, monkeypatch):
    monkeypatch.setenv("RL_KV_F16", str(kv_f16))
    dims = synth.tiny_model_dims(n_layer=4, n_head=16, n_head_kv=2, head_dim=256, rope_dims=64, context=2048)
    sm = synth.model(91 + kv_f16, dims)
    path = str(tmp_path / "long.gguf")
    gguf_writer.write_gguf(path, sm)
    threads = os.cpu_count() or 1
    om = ol.OracleModel(sm, kv_f16=bool(kv_f16), context=dims.context)
    eng = Engine(path, context=dims.context)
    try:
        prompt = np.random.default_rng(17).integers(0, dims.vocab, max(LENGTHS) + 1).astype(np.uint32)
        done, ml_last = 0, None
        for R in LENGTHS:
            # the oracle walks the prompt once; at every length R it has consumed prompt[:R] (ml_last: logits after token R - 1)
            while done < R:
                ml_last = om.step(int(prompt[done]), threads=threads)
                done += 1
            # GPU: the first R tokens by chunked prefill from an empty state (batched attention over the chunk's rows) ...
            eng.reset()
            gl = eng.prefill(prompt[:R])
            assert eng.position == R
            _compare(eng, om, dims, gl, ml_last, ("prefill", R))
            # ... then one decode step at position R (split-K decode attention over R + 1 positions)
            ml = ml_last = om.step(int(prompt[R]), threads=threads)
            done += 1
            gl = eng.step(int(prompt[R]))
            _compare(eng, om, dims, gl, ml, ("decode", R))
    finally:
        eng.close()
