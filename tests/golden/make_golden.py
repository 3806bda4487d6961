"""Writes tests/golden/reference_vectors.npz: outputs of the reference's own C (oracle/_ref/libredlite_ref.so, compiled
unchanged from the reference sources by `make -C oracle ref`) on seeded inputs. The fixtures make the pin of the oracle —
and the GPU parity of the same cases — independent of the reference sources being present at test time.

    python tests/golden/make_golden.py

Inputs are regenerated from the seeds by the tests (dwarfstar_red_lite_b200/synth.py), only the reference outputs are stored.
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

import oracle_lib as ol  # noqa: E402
from dwarfstar_red_lite_b200 import gguf_writer, synth  # noqa: E402

QUANT_CASES = [(synth.Q6_K, 256), (synth.Q6_K, 2048), (synth.IQ2_XXS, 256), (synth.IQ2_XXS, 2048), (synth.IQ3_S, 768), (synth.IQ3_S, 2048),
               # the further types that stay in file layout (stage entry points)
               (synth.Q8_0, 256), (synth.Q2_K, 768), (synth.Q4_K, 2048), (synth.Q5_K, 256), (synth.IQ3_XXS, 768), (synth.IQ2_S, 256), (synth.IQ4_XS, 2048)]
# IQ2_XS / IQ1_M: the reference has them only as the row dot of its routed-expert checker (rl_native_quant_row_dot)
XS_CASES = [(synth.IQ2_XS, 256), (synth.IQ2_XS, 2048), (synth.IQ1_M, 256), (synth.IQ1_M, 768)]
ROWS = 6


def quant_inputs(t, ncols):
    rng = np.random.default_rng(7000 + 13 * t + ncols)
    rows = synth.quant_matrix(rng, t, ROWS, ncols, 1e-3, 4e-3)
    x = rng.normal(0, 1, ncols).astype(np.float32)
    return rows, x


def router_inputs():
    rng = np.random.default_rng(7100)
    logits = rng.normal(0, 2, size=(24, 512)).astype(np.float32)
    for case in range(0, 24, 4):
        logits[case, rng.integers(0, 512, 24)] = logits[case, 3]       # exact ties
    logits[1, :] = 0.25
    return logits


def engine_model():
    dims = synth.tiny_model_dims(type_experts=synth.IQ3_S)
    return dims, synth.model(7200, dims)


def main():
    ref = ol.ref()
    if ref is None:
        raise SystemExit("oracle/_ref/libredlite_ref.so is missing: run `make -C oracle ref` where the reference sources are mounted")
    g2, _ = ol.codebooks()
    out = {}
    for t, ncols in QUANT_CASES:
        rows, x = quant_inputs(t, ncols)
        deq = np.empty((ROWS, ncols), np.float32)
        dots = np.empty(ROWS, np.float64)
        for r in range(ROWS):
            assert ref.rl_quant_dequant_row(C.c_uint32(t), ol.ptr(rows[r], ol.u8p), C.c_uint32(ncols), ol.ptr(g2, ol.u8p), ol.ptr(deq[r], ol.f32p)) == 1
            d = C.c_double()
            assert ref.rl_quant_row_dot(C.c_uint32(t), ol.ptr(rows[r], ol.u8p), ol.ptr(x, ol.f32p), C.c_uint32(ncols), ol.ptr(g2, ol.u8p), C.byref(d)) == 1
            dots[r] = d.value
        out[f"deq_{t}_{ncols}"] = deq
        out[f"dot_{t}_{ncols}"] = dots
    xs, m1 = ol.codebooks_xs()
    ref.rl_native_quant_row_dot.argtypes = [C.c_void_p, C.c_size_t, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_size_t, C.POINTER(C.c_double), C.c_char_p, C.c_size_t]
    msg = C.create_string_buffer(256)
    for t, ncols in XS_CASES:
        rows, x = quant_inputs(t, ncols)
        grid = xs if t == synth.IQ2_XS else m1

        def dot(row, vec):
            d = C.c_double()
            assert ref.rl_native_quant_row_dot(row.ctypes.data, row.size, t, vec.ctypes.data, ncols, grid.ctypes.data, grid.size, C.byref(d), msg, 256) == 1, msg.value
            return d.value

        dots = np.array([dot(np.ascontiguousarray(rows[r]), x) for r in range(ROWS)], np.float64)
        out[f"dot_{t}_{ncols}"] = dots
        if ncols == 256:      # every single weight of the first two rows, through dots with unit vectors
            w = np.empty((2, ncols), np.float64)
            for r in range(2):
                row = np.ascontiguousarray(rows[r])
                for i in range(ncols):
                    e = np.zeros(ncols, np.float32)
                    e[i] = 1.0
                    w[r, i] = dot(row, e)
            out[f"weights_{t}_{ncols}"] = w
    logits = router_inputs()
    k = 10
    ids = np.empty((logits.shape[0], k), np.uint32)
    w = np.empty((logits.shape[0], k), np.float32)
    err = C.create_string_buffer(256)
    for c in range(logits.shape[0]):
        probs = np.empty(512, np.float32)
        assert ref.rl_native_router_select_softmax_topk(ol.ptr(logits[c], ol.f32p), C.c_uint32(512), C.c_uint32(k), ol.ptr(ids[c], ol.u32p),
                                                        ol.ptr(w[c], ol.f32p), ol.ptr(probs, ol.f32p), err, C.c_size_t(256)) == 1
    out["router_ids"], out["router_w"] = ids, w
    # stateful decode of a tiny GGUF model through the reference engine's CPU backend (IQ3_S experts, fp16 KV)
    os.environ["RL_KV_F16"] = "1"
    dims, sm = engine_model()
    path = "/tmp/redcuda_golden_tiny.gguf"
    gguf_writer.write_gguf(path, sm)
    eng = ol.RefEngine(path, dims.context, threads=2)
    toks, logit_rows, layer_rows, id_rows = [], [], [], []
    tok = 3
    for _ in range(6):
        lg = eng.step(tok, dims.vocab)
        toks.append(tok)
        logit_rows.append(lg.copy())
        layer_rows.append(np.stack([eng.layer_out(l, dims.hidden) for l in range(dims.n_layer)]))
        id_rows.append(np.stack([eng.router_ids(l, dims.top_k) for l in range(dims.n_layer)]))
        tok = int(np.argmax(lg))
    eng.close()
    os.remove(path)
    out["engine_tokens"] = np.array(toks, np.uint32)
    out["engine_logits"] = np.stack(logit_rows)
    out["engine_layer_out"] = np.stack(layer_rows)
    out["engine_router_ids"] = np.stack(id_rows).astype(np.uint32)
    dst = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
