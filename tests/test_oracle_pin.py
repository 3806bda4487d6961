"""Pins the restated CPU oracle (oracle/redcuda_oracle.c): known-answer vectors of the reference's own offline tests,
and — where the reference's portable C has been compiled (oracle/_ref) — bit-for-bit agreement with it on seeded
inputs, up to a whole stateful decode of a small synthetic model through rl_engine_step on the CPU backend."""
import ctypes as C
import os

import numpy as np
import pytest

import oracle_lib as ol
from dwarfstar_red_lite_b200 import gguf_writer, synth

REF = ol.ref()
needs_ref = pytest.mark.skipif(REF is None, reason="reference checker library not built here")


def _f16(v):
    return np.array([v], np.float16).view(np.uint8)


# ---- known-answer vectors (reference: native/redlite_native_shared_exec_offline_test.c:18-55, quant_cpu.c:364-393,
# ---- native/redlite_native_router_offline_test.c:8-30, native/redlite_native_deltanet_state_cli.c:110-141)
def test_kat_q6k_all_minus32():
    blk = np.zeros(210, np.uint8)
    blk[192:208] = 1
    blk[208:210] = _f16(1.0)
    y = ol.dequant_rows(synth.Q6_K, blk, 256)[0]
    assert np.all(y == -32.0)
    assert ol.rows_dot(synth.Q6_K, blk, np.ones(256, np.float32))[0] == -8192.0


def test_kat_q6k_subnormal_scale():
    # the smallest fp16 subnormal (2^-24) must convert exactly
    assert ol.own().ro_f16_to_f32(1) == 2.0 ** -24
    blk = np.zeros(210, np.uint8)
    blk[192:208] = 1
    blk[208] = 1
    y = ol.dequant_rows(synth.Q6_K, blk, 256)[0]
    assert np.all(y == np.float32(-32.0 * 2.0 ** -24))


def test_kat_iq2xxs_zero_block():
    # d = 1, grid index 0 (all magnitudes 8), no signs, scale nibble 0 -> db = 0.125, every value 1.0, dot with ones = 256
    blk = np.zeros(66, np.uint8)
    blk[0:2] = _f16(1.0)
    y = ol.dequant_rows(synth.IQ2_XXS, blk, 256)[0]
    assert np.all(y == 1.0)
    assert ol.rows_dot(synth.IQ2_XXS, blk, np.ones(256, np.float32))[0] == 256.0


def test_kat_codebook_spot_values():
    g2, g3 = ol.codebooks()
    assert set(np.unique(g2)) == {0x08, 0x19, 0x2b}
    assert np.all(g2[:8] == 8)
    assert g3[0] == 0x01010101 and g3[511] == 0x0f0f0101       # iq3.c:398-402


def test_kat_router():
    ids, w, _ = ol.router_select(np.array([0, 1, 2, 3], np.float32), 2)
    assert list(ids) == [3, 2]
    assert abs(w[0] - 0.7310585786) < 1e-6 and abs(w[1] - 0.2689414214) < 1e-6
    ids, _, _ = ol.router_select(np.array([1, 1, 0, 0], np.float32), 2)
    assert list(ids) == [0, 1]                                  # ties -> lower index


def test_kat_deltanet_state_s2():
    # S = 2, one head: state zero, k = (1, 0), v = (0.5, -0.25), beta = 0.5, q = (1, 0), no decay:
    # delta = (0.25, -0.125); state[j][i] += k[i]*delta[j]; out = state q / sqrt(2)
    S = 2
    p = dict(d_conv=2, d_state=S, n_group=1, dt_rank=1, d_inner=S, channels=3 * S, rms_eps=1e-6,
             conv_kernel=np.tile(np.array([0.0, 1.0], np.float32), (3 * S, 1)), dt_bias=np.zeros(1, np.float32),
             ssm_a=np.zeros(1, np.float32), ssm_norm=np.ones(S, np.float32))
    # conv output = SiLU(new sample); choose pre-activations whose SiLU gives the wanted q, k, v
    def inv_silu(y):
        lo, hi = -1.0, 20.0
        f = lambda t: t / (1 + np.exp(-t))
        if y < 0:
            lo, hi = -1.2, 0.0   # decreasing branch avoided: use the increasing part on [-1.278, 0]
            for _ in range(200):
                mid = (lo + hi) / 2
                if f(mid) < y: lo = mid
                else: hi = mid
            return (lo + hi) / 2
        for _ in range(200):
            mid = (lo + hi) / 2
            if f(mid) < y: lo = mid
            else: hi = mid
        return (lo + hi) / 2
    qkv = np.array([inv_silu(1.0), 0.0, inv_silu(1.0), 0.0, inv_silu(0.5), inv_silu(-0.25)], np.float32)
    conv = np.zeros((3 * S, 1), np.float32)
    rec = np.zeros((1, S, S), np.float32)
    ba = np.array([0.0, 0.0], np.float32)      # beta = sigmoid(0) = 0.5; gate = softplus(0)*0 = 0 -> decay 1
    z = np.full(S, 30.0, np.float32)           # SiLU(z) ~ z
    ol.deltanet_mid(p, qkv, z, ba, conv, rec)
    assert np.allclose(rec[0, :, 0], [0.25, -0.125], atol=1e-6) and np.allclose(rec[0, :, 1], 0.0, atol=1e-7)
    assert np.allclose(conv[:, 0], qkv)


# ---- bit-for-bit against the reference library
@needs_ref
@pytest.mark.parametrize("t", [synth.Q6_K, synth.IQ2_XXS, synth.IQ3_S, synth.F32, synth.F16, synth.Q8_0, synth.Q2_K, synth.Q4_K, synth.Q5_K,
                               synth.IQ3_XXS, synth.IQ2_S, synth.IQ4_XS])
def test_dequant_and_dot_match_reference(t):
    rng = np.random.default_rng(100 + t)
    g2, _ = ol.codebooks()
    for ncols in (256, 768, 2048):
        if t in (synth.F32, synth.F16):
            w = rng.normal(0, 1, size=(5, ncols)).astype(np.float32 if t == synth.F32 else np.float16)
            rows = w.view(np.uint8).reshape(5, -1)
        else:
            rows = synth.quant_matrix(rng, t, 5, ncols, 1e-3, 4e-3)
        x = rng.normal(0, 1, ncols).astype(np.float32)
        mine = ol.dequant_rows(t, rows, ncols)
        dots = ol.rows_dot(t, rows, x)
        for r in range(5):
            out = np.empty(ncols, np.float32)
            assert REF.rl_quant_dequant_row(C.c_uint32(t), ol.ptr(rows[r], ol.u8p), C.c_uint32(ncols), ol.ptr(g2, ol.u8p), ol.ptr(out, ol.f32p)) == 1
            assert np.array_equal(out.view(np.uint32), mine[r].view(np.uint32))
            d = C.c_double()
            assert REF.rl_quant_row_dot(C.c_uint32(t), ol.ptr(rows[r], ol.u8p), ol.ptr(x, ol.f32p), C.c_uint32(ncols), ol.ptr(g2, ol.u8p), C.byref(d)) == 1
            assert d.value == dots[r]


@needs_ref
@pytest.mark.parametrize("t", [synth.IQ2_XS, synth.IQ1_M])
def test_routed_checker_types_match_reference(t):
    """IQ2_XS and IQ1_M exist in the reference only as the row dot of its routed-expert checker
    (rl_native_quant_row_dot, native/redlite_native_reference.c:182-195): dots bit for bit, and every dequantised value
    against the dot with a unit vector (the only way that function shows a single weight)."""
    rng = np.random.default_rng(400 + t)
    xs, m1 = ol.codebooks_xs()
    grid = xs if t == synth.IQ2_XS else m1
    REF.rl_native_quant_row_dot.argtypes = [C.c_void_p, C.c_size_t, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_size_t, C.POINTER(C.c_double), C.c_char_p, C.c_size_t]
    err = C.create_string_buffer(256)

    def ref_dot(row, x, ncols):
        d = C.c_double()
        assert REF.rl_native_quant_row_dot(row.ctypes.data, row.size, t, x.ctypes.data, ncols, grid.ctypes.data, grid.size, C.byref(d), err, 256) == 1, err.value
        return d.value

    for ncols in (256, 768, 2048):
        rows = synth.quant_matrix(rng, t, 5, ncols, 1e-2, 6e-2)
        x = rng.normal(0, 1, ncols).astype(np.float32)
        dots = ol.rows_dot(t, rows, x)
        for r in range(5):
            assert ref_dot(np.ascontiguousarray(rows[r]), x, ncols) == dots[r]
    rows = synth.quant_matrix(rng, t, 3, 256, 1e-2, 6e-2)
    mine = ol.dequant_rows(t, rows, 256)
    for r in range(3):
        row = np.ascontiguousarray(rows[r])
        for i in range(256):
            e = np.zeros(256, np.float32)
            e[i] = 1.0
            w = ref_dot(row, e, 256)
            assert np.float32(w) == mine[r, i] and float(mine[r, i]) == w      # the double weight is exactly a float


@needs_ref
def test_f16_and_round_half_match_reference():
    lib = ol.own()
    for h in list(range(0, 2048)) + list(range(0x7b00, 0x7c02)) + [0x8001, 0xfbff, 0x3c00, 0xbc00]:
        a, b = lib.ro_f16_to_f32(h), REF.rl_quant_f16_to_f32(h)
        assert (a == b) or (a != a and b != b)
    # round_half against numpy's float16 rounding (the reference function is static)
    rng = np.random.default_rng(5)
    v = np.concatenate([rng.normal(0, 1, 2000), rng.normal(0, 1e-6, 500), rng.normal(0, 3e4, 500)]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = v.astype(np.float16).astype(np.float32)
    got = np.array([lib.ro_round_half(C.c_float(float(f))) for f in v], np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@needs_ref
def test_router_select_matches_reference():
    rng = np.random.default_rng(7)
    for case in range(64):
        n, k = 512, 10
        logits = rng.normal(0, 2, n).astype(np.float32)
        if case % 4 == 0:   # exact ties, as the reference's kernel self-test does
            logits[rng.integers(0, n, 24)] = logits[3]
        ids, w, probs = ol.router_select(logits, k)
        rid, rw, rp = np.empty(k, np.uint32), np.empty(k, np.float32), np.empty(n, np.float32)
        err = C.create_string_buffer(256)
        assert REF.rl_native_router_select_softmax_topk(ol.ptr(logits, ol.f32p), C.c_uint32(n), C.c_uint32(k), ol.ptr(rid, ol.u32p),
                                                        ol.ptr(rw, ol.f32p), ol.ptr(rp, ol.f32p), err, C.c_size_t(256)) == 1
        assert np.array_equal(ids, rid) and np.array_equal(w.view(np.uint32), rw.view(np.uint32)) and np.array_equal(probs.view(np.uint32), rp.view(np.uint32))


@needs_ref
@pytest.mark.parametrize("kv_f16", [True])
def test_model_step_matches_reference_engine(tmp_path, kv_f16):
    """Whole stateful decode: the restated step over in-memory tensors == rl_engine_step(CPU) over the same model
    written as GGUF, IQ3_S experts (a routed type the unmodified reference accepts). Layer outputs, router ids and
    logits must agree to the last bit for several tokens (DeltaNet state, conv window and KV cache carried over)."""
    os.environ["RL_KV_F16"] = "1"
    dims = synth.tiny_model_dims(type_experts=synth.IQ3_S)
    sm = synth.model(11, dims)
    path = str(tmp_path / "tiny.gguf")
    gguf_writer.write_gguf(path, sm)
    eng = ol.RefEngine(path, dims.context, threads=2)
    om = ol.OracleModel(sm, kv_f16=True)
    try:
        tok = 3
        for step in range(6):
            rl = eng.step(tok, dims.vocab)
            ml = om.step(tok, threads=2)
            for l in range(dims.n_layer):
                assert np.array_equal(eng.router_ids(l, dims.top_k), om.router_ids(l)), (step, l)
                assert np.array_equal(eng.layer_out(l, dims.hidden).view(np.uint32), om.layer_out(l).view(np.uint32)), (step, l)
            assert np.array_equal(rl.view(np.uint32), ml.view(np.uint32))
            tok = int(np.argmax(ml))
    finally:
        eng.close()
