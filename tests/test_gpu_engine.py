"""Engine parity on the GPU: rl_engine_step / rl_engine_generate_greedy of the CUDA backend against the CPU oracle on
the same synthetic GGUF model, with the reference's own criteria (native/redlite_native_engine_cli.c:691-741): router
ids of every layer identical, per-layer outputs and logits within bound, greedy tokens equal."""
import os

import numpy as np
import pytest

import oracle_lib as ol
from dwarfstar_red_lite_b200 import gguf_writer, synth
from dwarfstar_red_lite_b200.engine import Engine

pytestmark = pytest.mark.gpu

REL_OUT = 1e-3


def _compare_step(eng, om, dims, tok, step):
    gl = eng.step(tok)
    ml = om.step(tok, threads=os.cpu_count() or 1)
    for l in range(dims.n_layer):
        assert np.array_equal(eng.router_ids(l), om.router_ids(l)), (step, l, eng.router_ids(l), om.router_ids(l))
        a, b = eng.layer_out(l), om.layer_out(l)
        assert np.max(np.abs(a - b)) <= REL_OUT * np.max(np.abs(b)), (step, l, float(np.max(np.abs(a - b)) / np.max(np.abs(b))))
    rng_ = float(ml.max() - ml.min())
    assert np.max(np.abs(gl - ml)) <= 0.005 * max(1.0, rng_) + 0.05      # logits bound of the reference's parity tool
    assert np.max(np.abs(gl - ml)) <= REL_OUT * np.max(np.abs(ml)) + 1e-6
    assert int(np.argmax(gl)) == int(np.argmax(ml))
    return int(np.argmax(ml))


@pytest.mark.parametrize("te", [synth.IQ2_XXS, synth.IQ3_S])
@pytest.mark.parametrize("kv_f16", [1, 0])
def test_tiny_model_stepwise(tmp_path, te, kv_f16, monkeypatch):
    monkeypatch.setenv("RL_KV_F16", str(kv_f16))
    dims = synth.tiny_model_dims(type_experts=te, n_layer=8)
    sm = synth.model(21 + te, dims)
    path = str(tmp_path / "tiny.gguf")
    gguf_writer.write_gguf(path, sm)
    eng = Engine(path, context=dims.context)
    om = ol.OracleModel(sm, kv_f16=bool(kv_f16))
    try:
        assert eng.info.n_recurrent == 6 and eng.info.n_attention == 2
        # embedding row: bit-exact dequantisation
        emb = eng.embed_token(5)
        want = ol.dequant_rows(dims.type_dense, sm.tensors["token_embd.weight"][2][5], dims.hidden)[0]
        assert np.array_equal(emb.view(np.uint32), want.view(np.uint32))
        tok = 3
        for step in range(12):
            tok = _compare_step(eng, om, dims, tok, step)
        # reset returns to an empty state: the first step repeats bit-for-bit
        first = None
        for rep in range(2):
            eng.reset()
            l = eng.step(3)
            if first is None:
                first = l.copy()
            else:
                assert np.array_equal(first, l)
    finally:
        eng.close()


@pytest.mark.parametrize("td", [synth.Q4_K, synth.Q8_0, synth.Q5_K, synth.Q2_K])
def test_tiny_model_with_file_layout_dense_types(tmp_path, td, monkeypatch):
    """Dense matrices (embedding, projections, LM head) in further GGUF types, kept in file layout: decode steps and a
    chunked prefill against the oracle. The routed and shared experts stay in the types their kernels are built for."""
    monkeypatch.setenv("RL_KV_F16", "1")
    dims = synth.tiny_model_dims(type_dense=td, type_shared=synth.Q6_K, n_layer=4)
    sm = synth.model(300 + td, dims)
    path = str(tmp_path / "tiny.gguf")
    gguf_writer.write_gguf(path, sm)
    eng = Engine(path, context=dims.context, prefill_batch=8)
    om = ol.OracleModel(sm, kv_f16=True)
    try:
        emb = eng.embed_token(5)
        want = ol.dequant_rows(td, sm.tensors["token_embd.weight"][2][5], dims.hidden)[0]
        assert np.array_equal(emb.view(np.uint32), want.view(np.uint32))
        tok = 3
        for step in range(5):
            tok = _compare_step(eng, om, dims, tok, step)
        prompt = np.random.default_rng(6).integers(0, dims.vocab, 11).astype(np.uint32)
        gl = eng.prefill(prompt)
        for t in prompt:
            ml = om.step(int(t), threads=os.cpu_count() or 1)
        _compare_last(eng, om, dims, gl, ml, ("file layout", td))
    finally:
        eng.close()


def test_tiny_model_greedy_60_tokens(tmp_path, monkeypatch):
    monkeypatch.setenv("RL_KV_F16", "1")
    dims = synth.tiny_model_dims(n_layer=8)
    sm = synth.model(33, dims)
    path = str(tmp_path / "tiny.gguf")
    gguf_writer.write_gguf(path, sm)
    eng = Engine(path, context=dims.context)
    om = ol.OracleModel(sm, kv_f16=True)
    try:
        n = 60
        got, _ = eng.generate_greedy(7, n)
        tok, want = 7, []
        for _ in range(n):
            tok = int(np.argmax(om.step(tok, threads=os.cpu_count() or 1)))
            want.append(tok)
        assert list(got) == want
        assert eng.position == n
    finally:
        eng.close()


def test_midsize_model_full_head_shapes(tmp_path, monkeypatch):
    """Full-size heads and widths (hidden 2048, DeltaNet 16/32 heads of 128, GQA 16/2 heads of 256, IQ2_XXS experts of
    512x2048), fewer layers / experts / vocabulary so that the oracle stays in seconds."""
    monkeypatch.setenv("RL_KV_F16", "1")
    dims = synth.ModelDims(n_layer=4, vocab=2048, n_expert=32, top_k=10, context=48)
    sm = synth.model(55, dims)
    path = str(tmp_path / "mid.gguf")
    gguf_writer.write_gguf(path, sm)
    eng = Engine(path, context=dims.context)
    om = ol.OracleModel(sm, kv_f16=True, context=dims.context)
    try:
        tok = 11
        for step in range(6):
            tok = _compare_step(eng, om, dims, tok, step)
    finally:
        eng.close()


def _compare_last(eng, om, dims, gl, ml, tag):
    for l in range(dims.n_layer):
        assert np.array_equal(eng.router_ids(l), om.router_ids(l)), (tag, l, eng.router_ids(l), om.router_ids(l))
        a, b = eng.layer_out(l), om.layer_out(l)
        assert np.max(np.abs(a - b)) <= REL_OUT * np.max(np.abs(b)), (tag, l, float(np.max(np.abs(a - b)) / np.max(np.abs(b))))
    assert np.max(np.abs(gl - ml)) <= REL_OUT * np.max(np.abs(ml)) + 1e-6, tag
    assert int(np.argmax(gl)) == int(np.argmax(ml)), tag


@pytest.mark.parametrize("chunk", [1, 2, 5, 8, 64])
def test_tiny_model_chunked_prefill(tmp_path, chunk, monkeypatch):
    """rl_engine_prefill in chunks (ragged last chunk, chunk larger than the prompt, two calls in a row) leaves the same
    mirrors, logits and state as the oracle's token-by-token pass; decode steps after it agree as well."""
    monkeypatch.setenv("RL_KV_F16", "0")
    dims = synth.tiny_model_dims(n_layer=8)
    sm = synth.model(77, dims)
    path = str(tmp_path / "tiny.gguf")
    gguf_writer.write_gguf(path, sm)
    eng = Engine(path, context=dims.context, prefill_batch=chunk)
    om = ol.OracleModel(sm, kv_f16=False)
    try:
        assert eng.prefill_batch == chunk
        prompt = np.random.default_rng(5).integers(0, dims.vocab, 21).astype(np.uint32)
        gl = eng.prefill(prompt[:13])
        for t in prompt[:13]:
            ml = om.step(int(t), threads=os.cpu_count() or 1)
        assert eng.position == 13
        _compare_last(eng, om, dims, gl, ml, ("first call", chunk))
        gl = eng.prefill(prompt[13:])                      # continues from position 13
        for t in prompt[13:]:
            ml = om.step(int(t), threads=os.cpu_count() or 1)
        assert eng.position == 21
        _compare_last(eng, om, dims, gl, ml, ("second call", chunk))
        tok = int(np.argmax(ml))
        for step in range(4):
            tok = _compare_step(eng, om, dims, tok, step)
        got, _ = eng.generate_greedy(tok, 5)
        want = []
        for _ in range(5):
            tok = int(np.argmax(om.step(tok, threads=os.cpu_count() or 1)))
            want.append(tok)
        assert list(got) == want
    finally:
        eng.close()


@pytest.mark.parametrize("router_tc", [None, "8"])
def test_midsize_model_chunked_prefill(tmp_path, router_tc, monkeypatch):
    """Full-size head shapes: the chunk takes the tensor-core projections (Q6_K dense matrices, >= 3 tokens), the in-register
    DeltaNet scan over 128-wide states and the batched GQA attention. router_tc: the opt-in form of the router logits on
    the tcgen05 GEMM (fp32 weight rows through the same digit decoder), here from 8 tokens on."""
    monkeypatch.setenv("RL_KV_F16", "1")
    if router_tc:
        monkeypatch.setenv("RC_ROUTER_TC_MIN", router_tc)
    dims = synth.ModelDims(n_layer=4, vocab=2048, n_expert=32, top_k=10, context=48)
    sm = synth.model(56, dims)
    path = str(tmp_path / "mid.gguf")
    gguf_writer.write_gguf(path, sm)
    eng = Engine(path, context=dims.context, prefill_batch=16)
    om = ol.OracleModel(sm, kv_f16=True, context=dims.context)
    try:
        prompt = np.random.default_rng(9).integers(0, dims.vocab, 37).astype(np.uint32)
        gl = eng.prefill(prompt)
        for t in prompt:
            ml = om.step(int(t), threads=os.cpu_count() or 1)
        _compare_last(eng, om, dims, gl, ml, "mid")
        tok = int(np.argmax(ml))
        for step in range(3):
            tok = _compare_step(eng, om, dims, tok, step)
        with pytest.raises(Exception):
            eng.prefill(np.zeros(dims.context, np.uint32))      # does not fit what is left of the context
    finally:
        eng.close()


@pytest.mark.parametrize("scan", ["grouped", "warp"])
@pytest.mark.parametrize("which", ["tiny", "mid"])
def test_chunked_prefill_with_alternative_deltanet_scans(tmp_path, which, scan, monkeypatch):
    """The two scan kernels kept beside the default one. RC_DN_SCAN=grouped: the delta rule four tokens at a time (one round
    of reductions per group) must leave the same outputs and state as the oracle's token-by-token pass; prompt lengths that
    are not multiples of four leave a tail for the token-by-token kernel. RC_DN_SCAN=warp: one state row per warp."""
    monkeypatch.setenv("RL_KV_F16", "1")
    monkeypatch.setenv("RC_DN_SCAN", scan)
    if which == "tiny":
        dims = synth.tiny_model_dims(n_layer=8)
    else:
        dims = synth.ModelDims(n_layer=4, vocab=2048, n_expert=32, top_k=10, context=48)
    sm = synth.model(91, dims)
    path = str(tmp_path / "m.gguf")
    gguf_writer.write_gguf(path, sm)
    eng = Engine(path, context=dims.context, prefill_batch=16)
    om = ol.OracleModel(sm, kv_f16=True, context=dims.context)
    try:
        prompt = np.random.default_rng(10).integers(0, dims.vocab, 27).astype(np.uint32)     # 16 + 11: groups plus a tail of 3
        gl = eng.prefill(prompt)
        for t in prompt:
            ml = om.step(int(t), threads=os.cpu_count() or 1)
        _compare_last(eng, om, dims, gl, ml, which)
        tok = int(np.argmax(ml))
        for step in range(3):
            tok = _compare_step(eng, om, dims, tok, step)
    finally:
        eng.close()


def test_resident_engine_reports_no_expert_traffic(tmp_path, monkeypatch):
    """Every expert is resident in HBM, so what the reference's expert LRU counts (native/redlite_native_cache.c:160-323,
    surfaced through rl_engine_step_stats, native/redlite_native_engine.h:62-87) stays at zero after open: no loads, no
    misses, no SSD reads, and every slot of every layer is resident."""
    monkeypatch.setenv("RL_KV_F16", "1")
    dims = synth.tiny_model_dims(n_layer=4)
    sm = synth.model(12, dims)
    path = str(tmp_path / "tiny.gguf")
    gguf_writer.write_gguf(path, sm)
    eng = Engine(path, context=dims.context)
    try:
        ok, ms = eng.experts_preloaded()
        assert ok and ms > 0.0
        assert eng.full_residency_mib() >= 1
        tok = 1
        for _ in range(8):
            tok = int(np.argmax(eng.step(tok)))
            st = eng.last_stats
            assert st.expert_loads == 0 and st.cache_misses == 0 and st.ssd_reads == 0 and st.ssd_bytes == 0
            assert st.resident_slots == st.slot_capacity == dims.n_layer * dims.n_expert
    finally:
        eng.close()


def test_engine_errors(tmp_path):
    with pytest.raises(Exception):
        Engine(str(tmp_path / "missing.gguf"))
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGUF" + b"\0" * 64)
    with pytest.raises(Exception):
        Engine(str(bad))
