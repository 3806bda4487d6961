"""Full-depth engine parity on the GPU: a 48-layer model with the full head shapes and widths (hidden 2048, DeltaNet
16/32 heads of 128, GQA 16/2 heads of 256, IQ2_XXS experts of 512x2048, Q6_K dense matrices) and a small expert count
and vocabulary, so that the CPU oracle steps it in a few seconds per token. Rounding differences between fp32 GPU sums
and the oracle's double sums grow from layer to layer in a random-init model; this is where they are largest.

Criteria are the reference's (native/redlite_native_engine_cli.c:691-741): router ids identical in every layer, layer
outputs within 1e-3 of their range, logits within the parity bound, greedy tokens equal. One relaxation, written out in
_ids_equal_or_near_tie: the SAME ten experts may come in another order where the oracle's own logits of the two swapped
experts differ by less than 1e-4 (fp32 sums against double sums: at depth 40 the logits carry ~4e-5 of noise); such a
swap changes neither the experts nor their weights beyond that noise. At most 4 of the 3072 selections may do so."""
import os

import numpy as np
import pytest

import oracle_lib as ol
from dwarfstar_red_lite_b200 import gguf_writer, synth
from dwarfstar_red_lite_b200.engine import Engine

pytestmark = pytest.mark.gpu

REL_OUT = 1e-3
N_PROMPT, N_GREEDY = 64, 64


NEAR_TIE = 1e-4


def _ids_equal_or_near_tie(gpu_ids, cpu_ids, cpu_logits):
    """0 = identical, 1 = the same experts with neighbours swapped at a near tie of the oracle's logits, 2 = different."""
    if np.array_equal(gpu_ids, cpu_ids):
        return 0
    if sorted(gpu_ids.tolist()) != sorted(cpu_ids.tolist()):
        return 2
    pos = [k for k in range(len(cpu_ids)) if gpu_ids[k] != cpu_ids[k]]
    for k in pos:
        j = k + 1 if k + 1 in pos and gpu_ids[k] == cpu_ids[k + 1] and gpu_ids[k + 1] == cpu_ids[k] else k - 1
        if j not in pos or gpu_ids[k] != cpu_ids[j] or abs(float(cpu_logits[cpu_ids[k]]) - float(cpu_logits[cpu_ids[j]])) > NEAR_TIE:
            return 2
    return 1


def _layer_errs(eng, om, n_layer):
    errs, bad_ids, swaps = [], [], 0
    for l in range(n_layer):
        a, b = eng.layer_out(l), om.layer_out(l)
        errs.append(float(np.max(np.abs(a - b)) / np.max(np.abs(b))))
        kind = _ids_equal_or_near_tie(eng.router_ids(l), om.router_ids(l), om.router_logits(l))
        if kind == 2:
            bad_ids.append(l)
        swaps += kind == 1
    return errs, bad_ids, swaps


def test_deep48_prefill_chunk_then_greedy(tmp_path, monkeypatch):
    monkeypatch.setenv("RL_KV_F16", "1")
    dims = synth.ModelDims(n_layer=48, vocab=2048, n_expert=32, top_k=10, context=N_PROMPT + N_GREEDY + 32)
    sm = synth.model(48, dims)
    path = str(tmp_path / "deep.gguf")
    gguf_writer.write_gguf(path, sm)
    threads = os.cpu_count() or 1
    om = ol.OracleModel(sm, kv_f16=True, context=dims.context)
    eng = Engine(path, context=dims.context, prefill_batch=N_PROMPT)
    try:
        assert eng.info.n_layer == 48 and eng.prefill_batch == N_PROMPT
        prompt = np.random.default_rng(49).integers(0, dims.vocab, N_PROMPT).astype(np.uint32)
        # ---- the prompt as ONE chunk on the GPU (batched projections, DeltaNet scan, batched attention, grouped experts)
        gl = eng.prefill(prompt)
        for t in prompt:
            ml = om.step(int(t), threads=threads)
        errs, bad, swaps = _layer_errs(eng, om, dims.n_layer)
        assert not bad and not swaps, ("router ids differ after the prefill chunk", bad, swaps)
        assert max(errs) <= REL_OUT, ("prefill layer error", int(np.argmax(errs)), max(errs))
        assert np.max(np.abs(gl - ml)) <= 0.005 * max(1.0, float(ml.max() - ml.min())) + 0.05
        assert int(np.argmax(gl)) == int(np.argmax(ml))
        # ---- free-running greedy decode on the GPU from the prefilled state
        first = int(np.argmax(ml))
        got, _ = eng.generate_greedy(first, N_GREEDY)
        # ---- the same tokens step by step on both sides (the GPU replays from a fresh prefill)
        eng.reset()
        eng.prefill(prompt, want_logits=False)
        tok, want, worst, swaps = first, [], 0.0, 0
        for step in range(N_GREEDY):
            gl = eng.step(tok)
            ml = om.step(tok, threads=threads)
            errs, bad, sw = _layer_errs(eng, om, dims.n_layer)
            assert not bad, ("router ids differ", step, bad)
            swaps += sw
            assert max(errs) <= REL_OUT, ("decode layer error", step, int(np.argmax(errs)), max(errs))
            worst = max(worst, max(errs))
            assert np.max(np.abs(gl - ml)) <= 0.005 * max(1.0, float(ml.max() - ml.min())) + 0.05
            assert int(np.argmax(gl)) == int(np.argmax(ml)), ("argmax differs", step, float(np.sort(ml)[-1] - np.sort(ml)[-2]), float(np.max(np.abs(gl - ml))))
            tok = int(np.argmax(ml))
            want.append(tok)
        assert list(got) == want, "free-running greedy tokens differ from the oracle's"
        assert swaps <= 4, swaps
        print(f"deep48: {N_GREEDY} greedy tokens equal, {N_GREEDY * dims.n_layer - swaps} of {N_GREEDY * dims.n_layer} router selections identical "
              f"({swaps} near-tie order swaps), worst layer error {worst:.2e}")
    finally:
        eng.close()
