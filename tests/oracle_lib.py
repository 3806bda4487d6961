"""ctypes access to the two CPU checkers (test infrastructure; the product never imports this).

  own()  oracle/libredcuda_oracle.so   — the restated oracle, built from oracle/redcuda_oracle.c on demand
  ref()  oracle/_ref/libredlite_ref.so — the reference's own portable C compiled unchanged; present where it was
         built from the reference tree (it travels as a prebuilt file), else None
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
MAX_TOPK = 64

u8p, f32p, f64p, u32p = C.POINTER(C.c_uint8), C.POINTER(C.c_float), C.POINTER(C.c_double), C.POINTER(C.c_uint32)


def ptr(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def codebooks() -> tuple[np.ndarray, np.ndarray]:
    raw = np.fromfile(os.path.join(ROOT, "dwarfstar_red_lite_b200", "data", "codebooks.bin"), dtype=np.uint8)
    assert raw.size == 4096
    return raw[:2048].copy(), raw[2048:].view(np.uint32).copy()


def codebooks_ext() -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """IQ3_XXS grid (256 x uint32), IQ2_S grid (1024 x uint64), IQ4_NL values (16 x int8)."""
    raw = np.fromfile(os.path.join(ROOT, "dwarfstar_red_lite_b200", "data", "codebooks_iq3family.bin"), dtype=np.uint8)
    assert raw.size == 9232
    return raw[:1024].view(np.uint32).copy(), raw[1024:9216].view(np.uint64).copy(), raw[9216:].view(np.int8).copy()


def codebooks_xs() -> tuple[np.ndarray, np.ndarray]:
    """IQ2_XS grid (512 x 8 int8), IQ1_M grid (2048 x 8 int8)."""
    raw = np.fromfile(os.path.join(ROOT, "dwarfstar_red_lite_b200", "data", "codebooks_iq2xs_iq1m.bin"), dtype=np.int8)
    assert raw.size == 20480
    return raw[:4096].copy(), raw[4096:].copy()


class MoeLayerC(C.Structure):
    _fields_ = [("hidden", C.c_uint32), ("n_expert", C.c_uint32), ("top_k", C.c_uint32), ("ffn", C.c_uint32), ("ffn_sh", C.c_uint32),
                ("type_gu", C.c_uint32), ("type_down", C.c_uint32), ("type_sh", C.c_uint32),
                ("router", f32p), ("gate_all", u8p), ("up_all", u8p), ("down_all", u8p),
                ("sh_gate_inp", f32p), ("sh_gate", u8p), ("sh_up", u8p), ("sh_down", u8p)]


class DeltaParamsC(C.Structure):
    _fields_ = [("d_conv", C.c_uint32), ("d_state", C.c_uint32), ("n_group", C.c_uint32), ("dt_rank", C.c_uint32),
                ("d_inner", C.c_uint32), ("channels", C.c_uint32), ("rms_eps", C.c_float),
                ("conv_kernel", f32p), ("dt_bias", f32p), ("ssm_a", f32p), ("ssm_norm", f32p)]


class TensorC(C.Structure):
    _fields_ = [("type", C.c_uint32), ("nrows", C.c_uint32), ("ncols", C.c_uint32), ("data", u8p)]


_LAYER_SLOTS = ["attn_norm", "post_norm", "qkv", "z", "ba", "conv", "dt", "a", "ssm_norm", "ssm_out",
                "q", "k", "v", "q_norm", "k_norm", "o", "router", "sh_gate_inp", "sh_gate", "sh_up", "sh_down",
                "gate_exps", "up_exps", "down_exps"]


class LayerC(C.Structure):
    _fields_ = [("recurrent", C.c_int)] + [(n, TensorC) for n in _LAYER_SLOTS]


class ModelC(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ["n_layer", "hidden", "vocab", "n_expert", "top_k", "context", "d_conv", "d_inner",
                                          "d_state", "n_group", "dt_rank", "channels", "n_head", "n_head_kv", "head_dim", "rope_dims"]] + \
               [("rope_freq_base", C.c_float), ("rms_eps", C.c_float), ("kv_f16", C.c_int),
                ("tok_embd", TensorC), ("output_norm", TensorC), ("output", TensorC), ("layers", C.POINTER(LayerC))]


_own = None


def own():
    global _own
    if _own is not None:
        return _own
    so = os.path.join(ORACLE_DIR, "libredcuda_oracle.so")
    src = os.path.join(ORACLE_DIR, "redcuda_oracle.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", ORACLE_DIR, "own"], stdout=subprocess.DEVNULL)
    lib = C.CDLL(so, mode=C.RTLD_LOCAL)
    lib.ro_f16_to_f32.restype = C.c_float
    lib.ro_f16_to_f32.argtypes = [C.c_uint16]
    lib.ro_round_half.restype = C.c_float
    lib.ro_round_half.argtypes = [C.c_float]
    lib.ro_row_bytes.restype = C.c_size_t
    lib.ro_row_bytes.argtypes = [C.c_uint32, C.c_uint32]
    lib.ro_state_create.restype = C.c_void_p
    lib.ro_state_create.argtypes = [C.POINTER(ModelC)]
    lib.ro_state_free.argtypes = [C.c_void_p]
    lib.ro_state_reset.argtypes = [C.c_void_p]
    lib.ro_state_layer_out.restype = f32p
    lib.ro_state_layer_out.argtypes = [C.c_void_p, C.c_uint32]
    lib.ro_state_router_ids.restype = u32p
    lib.ro_state_router_ids.argtypes = [C.c_void_p, C.c_uint32]
    lib.ro_state_final_norm.restype = f32p
    lib.ro_state_final_norm.argtypes = [C.c_void_p]
    lib.ro_state_router_logits.restype = f32p
    lib.ro_state_router_logits.argtypes = [C.c_void_p, C.c_uint32]
    lib.ro_state_rec.restype = f32p
    lib.ro_state_rec.argtypes = [C.c_void_p, C.c_uint32]
    lib.ro_state_conv.restype = f32p
    lib.ro_state_conv.argtypes = [C.c_void_p, C.c_uint32]
    lib.ro_model_step.argtypes = [C.POINTER(ModelC), C.c_void_p, C.c_uint32, f32p, C.c_int]
    g2, g3 = codebooks()
    x3, s2, n4 = codebooks_ext()
    xs, m1 = codebooks_xs()
    lib._keep = (g2, g3, x3, s2, n4, xs, m1)
    assert lib.ro_set_codebooks_xs(xs.ctypes.data_as(C.c_void_p), m1.ctypes.data_as(C.c_void_p)) == 1
    assert lib.ro_set_codebooks(ptr(g2, u8p), ptr(g3, u32p)) == 1
    assert lib.ro_set_codebooks_ext(x3.ctypes.data_as(C.c_void_p), s2.ctypes.data_as(C.c_void_p), n4.ctypes.data_as(C.c_void_p)) == 1
    _own = lib
    return lib


_ref = False


def ref():
    """The reference library, or None where it has not been built."""
    global _ref
    if _ref is not False:
        return _ref
    so = os.path.join(ORACLE_DIR, "_ref", "libredlite_ref.so")
    root = os.environ.get("REF_ROOT", "")
    if not os.path.exists(so) and root and os.path.isdir(os.path.join(root, "native")):
        subprocess.call(["make", "-C", ORACLE_DIR, "ref", f"REF_ROOT={root}"], stdout=subprocess.DEVNULL)
    if not os.path.exists(so):
        _ref = None
        return None
    lib = C.CDLL(so, mode=C.RTLD_LOCAL)
    lib.rl_quant_f16_to_f32.restype = C.c_float
    lib.rl_quant_f16_to_f32.argtypes = [C.c_uint16]
    lib.rl_engine_open.restype = C.c_void_p
    lib.rl_engine_close.argtypes = [C.c_void_p]
    lib.rl_engine_last_layer_output.restype = f32p
    lib.rl_engine_last_layer_output.argtypes = [C.c_void_p, C.c_int, C.c_uint32]
    lib.rl_engine_last_router_ids.restype = u32p
    lib.rl_engine_last_router_ids.argtypes = [C.c_void_p, C.c_int, C.c_uint32]
    lib.rl_engine_last_final_norm.restype = f32p
    lib.rl_engine_last_final_norm.argtypes = [C.c_void_p, C.c_int]
    _ref = lib
    return lib


# ---------------------------------------------------------------------------------------------- own-oracle helpers
def dequant_rows(t: int, rows: np.ndarray, ncols: int) -> np.ndarray:
    lib = own()
    rows = np.ascontiguousarray(rows, dtype=np.uint8).reshape(-1, lib.ro_row_bytes(t, ncols))
    out = np.empty((rows.shape[0], ncols), np.float32)
    for r in range(rows.shape[0]):
        assert lib.ro_dequant_row(C.c_uint32(t), ptr(rows[r], u8p), C.c_uint32(ncols), ptr(out[r], f32p)) == 1
    return out


def rows_dot(t: int, rows: np.ndarray, x: np.ndarray) -> np.ndarray:
    """double dot of every row with x (float32 vector)."""
    lib = own()
    ncols = x.size
    rows = np.ascontiguousarray(rows, dtype=np.uint8).reshape(-1, lib.ro_row_bytes(t, ncols))
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(rows.shape[0], np.float64)
    d = C.c_double()
    for r in range(rows.shape[0]):
        assert lib.ro_row_dot(C.c_uint32(t), ptr(rows[r], u8p), ptr(x, f32p), C.c_uint32(ncols), C.byref(d)) == 1
        out[r] = d.value
    return out


def matvec(t: int, w: np.ndarray, nrows: int, ncols: int, x: np.ndarray, threads: int = 1) -> np.ndarray:
    lib = own()
    w = np.ascontiguousarray(w).view(np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(nrows, np.float32)
    assert lib.ro_matvec(C.c_uint32(t), ptr(w, u8p), C.c_uint32(nrows), C.c_uint32(ncols), ptr(x, f32p), ptr(out, f32p), C.c_int(threads)) == 1
    return out


def router_logits(w: np.ndarray, x: np.ndarray) -> np.ndarray:
    lib = own()
    w = np.ascontiguousarray(w, np.float32)
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(w.shape[0], np.float32)
    lib.ro_router_logits(ptr(w, f32p), ptr(x, f32p), C.c_uint32(w.shape[0]), C.c_uint32(w.shape[1]), ptr(out, f32p))
    return out


def router_select(logits: np.ndarray, top_k: int):
    lib = own()
    logits = np.ascontiguousarray(logits, np.float32)
    ids = np.empty(top_k, np.uint32)
    w = np.empty(top_k, np.float32)
    probs = np.empty(logits.size, np.float32)
    ok = lib.ro_router_select(ptr(logits, f32p), C.c_uint32(logits.size), C.c_uint32(top_k), ptr(ids, u32p), ptr(w, f32p), ptr(probs, f32p))
    assert ok == 1
    return ids, w, probs


def moe_layer_c(layer) -> tuple[MoeLayerC, list]:
    """MoeLayerC view of a synth.MoeLayer; the second value keeps the arrays alive."""
    d = layer.dims
    keep = [np.ascontiguousarray(a) for a in (layer.router, layer.gate, layer.up, layer.down, layer.sh_gate_inp,
                                              layer.sh_gate, layer.sh_up, layer.sh_down)]
    L = MoeLayerC(d.hidden, d.n_expert, d.top_k, d.ffn, d.ffn_sh, d.type_gu, d.type_down, d.type_sh,
                  ptr(keep[0], f32p), ptr(keep[1], u8p), ptr(keep[2], u8p), ptr(keep[3], u8p),
                  ptr(keep[4], f32p), ptr(keep[5], u8p), ptr(keep[6], u8p), ptr(keep[7], u8p))
    return L, keep


def moe_ffn(layer, x: np.ndarray, threads: int = 1, logits_in: np.ndarray | None = None, view=None):
    """-> (out f32[hidden], ids u32[k], weights f32[k], logits f32[n_expert]); view = a cached moe_layer_c(layer)"""
    lib = own()
    L, keep = view if view is not None else moe_layer_c(layer)
    d = layer.dims
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(d.hidden, np.float32)
    ids = np.empty(d.top_k, np.uint32)
    w = np.empty(d.top_k, np.float32)
    logits = np.empty(d.n_expert, np.float32)
    li = None if logits_in is None else np.ascontiguousarray(logits_in, np.float32)
    ok = lib.ro_moe_ffn2(C.byref(L), ptr(x, f32p), None if li is None else ptr(li, f32p), ptr(out, f32p), ptr(ids, u32p), ptr(w, f32p),
                         ptr(logits, f32p), C.c_int(threads))
    assert ok == 1
    return out, ids, w, logits


def routed_experts(layer, ids: np.ndarray, weights: np.ndarray, x: np.ndarray, threads: int = 1) -> np.ndarray:
    lib = own()
    d = layer.dims
    keep = [np.ascontiguousarray(a) for a in (layer.gate, layer.up, layer.down)]
    ids = np.ascontiguousarray(ids, np.uint32)
    weights = np.ascontiguousarray(weights, np.float32)
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(d.hidden, np.float64)
    ok = lib.ro_routed_experts(C.c_uint32(d.type_gu), C.c_uint32(d.type_down), ptr(keep[0], u8p), ptr(keep[1], u8p), ptr(keep[2], u8p),
                               ptr(ids, u32p), ptr(weights, f32p), C.c_uint32(ids.size), C.c_uint32(d.hidden), C.c_uint32(d.ffn),
                               ptr(x, f32p), ptr(out, f64p), C.c_int(threads))
    assert ok == 1
    return out


def deltanet_mid(p: dict, qkv, z, ba, conv_state, rec_state):
    """p: d_conv,d_state,n_group,dt_rank,d_inner,channels,rms_eps + arrays conv_kernel, dt_bias, ssm_a, ssm_norm.
    conv_state and rec_state (float32, C-contiguous) are updated in place. Returns ng f32[d_inner]."""
    lib = own()
    arrs = {k: np.ascontiguousarray(p[k], np.float32) for k in ("conv_kernel", "dt_bias", "ssm_a", "ssm_norm")}
    P = DeltaParamsC(p["d_conv"], p["d_state"], p["n_group"], p["dt_rank"], p["d_inner"], p["channels"], p["rms_eps"],
                     ptr(arrs["conv_kernel"], f32p), ptr(arrs["dt_bias"], f32p), ptr(arrs["ssm_a"], f32p), ptr(arrs["ssm_norm"], f32p))
    qkv, z, ba = (np.ascontiguousarray(a, np.float32) for a in (qkv, z, ba))
    assert conv_state.dtype == np.float32 and conv_state.flags.c_contiguous and rec_state.dtype == np.float32 and rec_state.flags.c_contiguous
    out = np.empty(p["d_inner"], np.float32)
    ok = lib.ro_deltanet_mid(C.byref(P), ptr(qkv, f32p), ptr(z, f32p), ptr(ba, f32p), ptr(conv_state, f32p), ptr(rec_state, f32p), ptr(out, f32p))
    assert ok == 1
    return out


# ---------------------------------------------------------------------------------------------- whole model
_GGUF_TO_SLOT = {
    "attn_norm.weight": "attn_norm", "post_attention_norm.weight": "post_norm", "attn_qkv.weight": "qkv", "attn_gate.weight": "z",
    "ssm_ba.weight": "ba", "ssm_conv1d.weight": "conv", "ssm_dt.bias": "dt", "ssm_a": "a", "ssm_norm.weight": "ssm_norm",
    "ssm_out.weight": "ssm_out", "attn_q.weight": "q", "attn_k.weight": "k", "attn_v.weight": "v", "attn_q_norm.weight": "q_norm",
    "attn_k_norm.weight": "k_norm", "attn_output.weight": "o", "ffn_gate_inp.weight": "router", "ffn_gate_inp_shexp.weight": "sh_gate_inp",
    "ffn_gate_shexp.weight": "sh_gate", "ffn_up_shexp.weight": "sh_up", "ffn_down_shexp.weight": "sh_down",
    "ffn_gate_exps.weight": "gate_exps", "ffn_up_exps.weight": "up_exps", "ffn_down_exps.weight": "down_exps",
}


def _tensor_c(entry) -> TensorC:
    t, shape, arr = entry
    ncols = shape[0]
    nrows = shape[1] if len(shape) > 1 else 1
    return TensorC(t, nrows, ncols, arr.ctypes.data_as(u8p))


class OracleModel:
    """The restated oracle's view of a synth.SynthModel, with its own decode state."""

    def __init__(self, sm, kv_f16: bool = True, context: int | None = None):
        self.lib = own()
        self.sm = sm
        d = sm.dims
        self.layers = (LayerC * d.n_layer)()
        for l in range(d.n_layer):
            L = self.layers[l]
            L.recurrent = 0 if d.is_attention(l) else 1
            for gname, slot in _GGUF_TO_SLOT.items():
                e = sm.tensors.get(f"blk.{l}.{gname}")
                if e is not None:
                    setattr(L, slot, _tensor_c(e))
        self.m = ModelC(d.n_layer, d.hidden, d.vocab, d.n_expert, d.top_k, context or d.context, d.d_conv, d.d_inner, d.d_state,
                        d.n_group, d.dt_rank, d.channels, d.n_head, d.n_head_kv, d.head_dim, d.rope_dims,
                        d.rope_freq_base, d.rms_eps, 1 if kv_f16 else 0,
                        _tensor_c(sm.tensors["token_embd.weight"]), _tensor_c(sm.tensors["output_norm.weight"]),
                        _tensor_c(sm.tensors["output.weight"]), self.layers)
        self.state = self.lib.ro_state_create(C.byref(self.m))
        assert self.state

    def __del__(self):
        if getattr(self, "state", None):
            self.lib.ro_state_free(self.state)
            self.state = None

    def reset(self):
        self.lib.ro_state_reset(self.state)

    def step(self, token: int, want_logits: bool = True, threads: int = 1):
        d = self.sm.dims
        logits = np.empty(d.vocab, np.float32) if want_logits else None
        ok = self.lib.ro_model_step(C.byref(self.m), self.state, C.c_uint32(token), ptr(logits, f32p) if want_logits else None, C.c_int(threads))
        assert ok == 1
        return logits

    def layer_out(self, l: int) -> np.ndarray:
        return np.ctypeslib.as_array(self.lib.ro_state_layer_out(self.state, l), (self.sm.dims.hidden,)).copy()

    def router_ids(self, l: int) -> np.ndarray:
        return np.ctypeslib.as_array(self.lib.ro_state_router_ids(self.state, l), (self.sm.dims.top_k,)).copy()

    def final_norm(self) -> np.ndarray:
        return np.ctypeslib.as_array(self.lib.ro_state_final_norm(self.state), (self.sm.dims.hidden,)).copy()

    def router_logits(self, l: int) -> np.ndarray:
        return np.ctypeslib.as_array(self.lib.ro_state_router_logits(self.state, l), (self.sm.dims.n_expert,)).copy()


# ---------------------------------------------------------------------------------------------- reference engine
class RlEngineConfig(C.Structure):
    _fields_ = [("context", C.c_uint32), ("cache_mib", C.c_uint64), ("top_k", C.c_uint32), ("enable_cpu", C.c_int),
                ("enable_gpu", C.c_int), ("cpu_threads", C.c_int), ("prefill_batch", C.c_uint32), ("mtp_path", C.c_char_p)]


class RlStepStats(C.Structure):
    _fields_ = [(n, C.c_double) for n in ["embed_ms", "layers_ms", "recurrent_ms", "attention_ms", "router_ms", "routed_ms", "shared_ms",
                                          "output_ms", "total_ms", "routed_load_ms", "routed_gpu_ms", "gpu_ms"]] + \
               [(n, C.c_uint64) for n in ["expert_loads", "cache_hits", "cache_misses", "ssd_bytes", "ssd_reads"]] + \
               [(n, C.c_uint32) for n in ["resident_slots", "slot_capacity", "expert_plans"]] + \
               [(n, C.c_double) for n in ["prep_lru_ms", "prep_load_ms", "prep_commit_ms", "expert_wait_ms", "prefetch_ms"]] + \
               [("speculative", C.c_uint32), ("speculative_fallback", C.c_uint32)]


class RefEngine:
    """rl_engine_open / rl_engine_step of the unmodified reference on its CPU backend, over a GGUF file."""

    def __init__(self, path: str, context: int, threads: int = 1):
        self.lib = ref()
        assert self.lib is not None
        cfg = RlEngineConfig(context, 4096, 0, 1, 0, threads, 0, None)
        err = C.create_string_buffer(512)
        self.e = self.lib.rl_engine_open(path.encode(), C.byref(cfg), err, C.c_size_t(512))
        if not self.e:
            raise RuntimeError("rl_engine_open: " + err.value.decode())

    def close(self):
        if self.e:
            self.lib.rl_engine_close(self.e)
            self.e = None

    def step(self, token: int, vocab: int):
        logits = np.empty(vocab, np.float32)
        stats = RlStepStats()
        err = C.create_string_buffer(512)
        ok = self.lib.rl_engine_step(C.c_void_p(self.e), C.c_int(0), C.c_uint32(token), ptr(logits, f32p), C.byref(stats), err, C.c_size_t(512))
        if ok != 1:
            raise RuntimeError("rl_engine_step: " + err.value.decode())
        return logits

    def layer_out(self, l: int, hidden: int) -> np.ndarray:
        return np.ctypeslib.as_array(self.lib.rl_engine_last_layer_output(self.e, 0, l), (hidden,)).copy()

    def router_ids(self, l: int, k: int) -> np.ndarray:
        return np.ctypeslib.as_array(self.lib.rl_engine_last_router_ids(self.e, 0, l), (k,)).copy()
