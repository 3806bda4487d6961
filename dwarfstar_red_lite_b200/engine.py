"""ctypes mirror of include/rl_engine.h: the persistent decode engine (rl_engine_open / rl_engine_step / ... of the
reference, native/redlite_native_engine.h:89-209) served by the CUDA backend."""
from __future__ import annotations

import ctypes as C

import numpy as np

from .redcuda import RedcudaError, _ensure_books, lib

RL_BACKEND_GPU = 1
MAX_TOPK = 64
f32p, u32p = C.POINTER(C.c_float), C.POINTER(C.c_uint32)


class RlEngineConfig(C.Structure):
    _fields_ = [("context", C.c_uint32), ("cache_mib", C.c_uint64), ("top_k", C.c_uint32), ("enable_cpu", C.c_int),
                ("enable_gpu", C.c_int), ("cpu_threads", C.c_int), ("prefill_batch", C.c_uint32), ("mtp_path", C.c_char_p)]


class RlEngineInfo(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ["n_layer", "n_recurrent", "n_attention", "hidden", "vocab", "n_expert", "top_k", "context",
                                          "d_conv", "d_inner", "d_state", "n_group", "dt_rank", "channels", "head_v",
                                          "n_head", "n_head_kv", "head_dim", "rope_dims"]] + \
               [("rope_freq_base", C.c_float), ("rms_eps", C.c_float), ("dense_bytes", C.c_uint64), ("state_bytes", C.c_uint64)]


class RlStepStats(C.Structure):
    _fields_ = [(n, C.c_double) for n in ["embed_ms", "layers_ms", "recurrent_ms", "attention_ms", "router_ms", "routed_ms", "shared_ms",
                                          "output_ms", "total_ms", "routed_load_ms", "routed_gpu_ms", "gpu_ms"]] + \
               [(n, C.c_uint64) for n in ["expert_loads", "cache_hits", "cache_misses", "ssd_bytes", "ssd_reads"]] + \
               [(n, C.c_uint32) for n in ["resident_slots", "slot_capacity", "expert_plans"]] + \
               [(n, C.c_double) for n in ["prep_lru_ms", "prep_load_ms", "prep_commit_ms", "expert_wait_ms", "prefetch_ms"]] + \
               [("speculative", C.c_uint32), ("speculative_fallback", C.c_uint32)]


ENGINE_EXPORTS = ["rl_engine_config_default", "rl_engine_open", "rl_engine_close", "rl_engine_info_get", "rl_engine_reset", "rl_engine_position",
                  "rl_engine_bench_set_position", "rl_engine_step", "rl_engine_prefill", "rl_engine_last_embedding", "rl_engine_last_layer_output",
                  "rl_engine_last_final_norm", "rl_engine_last_router_ids", "rl_engine_experts_preloaded", "rl_engine_full_residency_mib",
                  "rl_engine_embed_token", "rl_engine_generate_greedy", "rl_engine_step_bytes", "rl_engine_prefill_batch"]


def _bind():
    L = lib()
    if getattr(L, "_engine_bound", False):
        return L
    L.rl_engine_config_default.argtypes = [C.POINTER(RlEngineConfig)]
    L.rl_engine_open.restype = C.c_void_p
    L.rl_engine_open.argtypes = [C.c_char_p, C.POINTER(RlEngineConfig), C.c_char_p, C.c_size_t]
    L.rl_engine_close.argtypes = [C.c_void_p]
    L.rl_engine_info_get.restype = C.POINTER(RlEngineInfo)
    L.rl_engine_info_get.argtypes = [C.c_void_p]
    L.rl_engine_reset.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.c_size_t]
    L.rl_engine_position.restype = C.c_uint32
    L.rl_engine_position.argtypes = [C.c_void_p, C.c_int]
    L.rl_engine_bench_set_position.argtypes = [C.c_void_p, C.c_int, C.c_uint32, C.c_char_p, C.c_size_t]
    L.rl_engine_step.argtypes = [C.c_void_p, C.c_int, C.c_uint32, C.c_void_p, C.POINTER(RlStepStats), C.c_char_p, C.c_size_t]
    L.rl_engine_prefill.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_uint32, C.c_void_p, C.POINTER(RlStepStats), C.c_char_p, C.c_size_t]
    L.rl_engine_generate_greedy.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.POINTER(RlStepStats), C.c_char_p, C.c_size_t]
    L.rl_engine_last_embedding.restype = f32p
    L.rl_engine_last_embedding.argtypes = [C.c_void_p, C.c_int]
    L.rl_engine_last_layer_output.restype = f32p
    L.rl_engine_last_layer_output.argtypes = [C.c_void_p, C.c_int, C.c_uint32]
    L.rl_engine_last_final_norm.restype = f32p
    L.rl_engine_last_final_norm.argtypes = [C.c_void_p, C.c_int]
    L.rl_engine_last_router_ids.restype = u32p
    L.rl_engine_last_router_ids.argtypes = [C.c_void_p, C.c_int, C.c_uint32]
    L.rl_engine_experts_preloaded.argtypes = [C.c_void_p, C.POINTER(C.c_double)]
    L.rl_engine_full_residency_mib.restype = C.c_uint64
    L.rl_engine_full_residency_mib.argtypes = [C.c_void_p]
    L.rl_engine_embed_token.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_char_p, C.c_size_t]
    L.rl_engine_prefill_batch.restype = C.c_uint32
    L.rl_engine_prefill_batch.argtypes = [C.c_void_p]
    L.rl_engine_step_bytes.restype = C.c_uint64
    L.rl_engine_step_bytes.argtypes = [C.c_void_p]
    L._engine_bound = True
    return L


class Engine:
    """rl_engine on the CUDA backend over a GGUF file."""

    def __init__(self, path: str, context: int = 4096, top_k: int = 0, prefill_batch: int = 0, ep_rank: int = 0, ep_world: int = 1):
        """ep_rank / ep_world: under expert parallelism the engine holds the experts [rank * E / world, (rank + 1) * E / world)
        of every layer; attach_ep() must follow before the first prefill or step."""
        _ensure_books()
        self.L = _bind()
        if self.L.redcuda_engine_shard(ep_rank, ep_world) != 1:
            raise RedcudaError(self.L.redcuda_last_error().decode(errors="replace"))
        cfg = RlEngineConfig()
        self.L.rl_engine_config_default(C.byref(cfg))
        cfg.context, cfg.top_k, cfg.enable_cpu, cfg.enable_gpu, cfg.prefill_batch = context, top_k, 0, 1, prefill_batch
        self._err = C.create_string_buffer(1024)
        self._e = self.L.rl_engine_open(path.encode(), C.byref(cfg), self._err, 1024)
        self.L.redcuda_engine_shard(0, 1)          # the setting is per open call
        if not self._e:
            raise RedcudaError("rl_engine_open: " + self._err.value.decode(errors="replace"))
        self.info = self.L.rl_engine_info_get(self._e).contents
        self._ep = None

    def attach_ep(self, ctx):
        """ctx: an ep.EpContext created with tokens >= prefill_batch; kept alive by this object"""
        if self.L.redcuda_engine_attach_ep(self._e, ctx.handle) != 1:
            raise RedcudaError(self.L.redcuda_last_error().decode(errors="replace"))
        self._ep = ctx

    def close(self):
        if getattr(self, "_e", None):
            self.L.rl_engine_close(self._e)
            self._e = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ok(self, rc, what):
        if rc != 1:
            raise RedcudaError(f"{what}: " + self._err.value.decode(errors="replace"))

    def reset(self):
        self._ok(self.L.rl_engine_reset(self._e, RL_BACKEND_GPU, self._err, 1024), "rl_engine_reset")

    @property
    def position(self) -> int:
        return int(self.L.rl_engine_position(self._e, RL_BACKEND_GPU))

    def set_position(self, pos: int):
        self._ok(self.L.rl_engine_bench_set_position(self._e, RL_BACKEND_GPU, pos, self._err, 1024), "rl_engine_bench_set_position")

    def step(self, token: int, want_logits: bool = True, logits: np.ndarray | None = None):
        if want_logits and logits is None:
            logits = np.empty(self.info.vocab, np.float32)
        stats = RlStepStats()
        self._ok(self.L.rl_engine_step(self._e, RL_BACKEND_GPU, token, logits.ctypes.data if want_logits else None, C.byref(stats), self._err, 1024), "rl_engine_step")
        self.last_stats = stats
        return logits

    def prefill(self, tokens, want_logits: bool = True):
        t = np.ascontiguousarray(tokens, np.uint32)
        logits = np.empty(self.info.vocab, np.float32) if want_logits else None
        stats = RlStepStats()
        self._ok(self.L.rl_engine_prefill(self._e, RL_BACKEND_GPU, t.ctypes.data, t.size, logits.ctypes.data if want_logits else None, C.byref(stats),
                                          self._err, 1024), "rl_engine_prefill")
        return logits

    def generate_greedy(self, token: int, n_new: int):
        out = np.empty(n_new, np.uint32)
        stats = RlStepStats()
        self._ok(self.L.rl_engine_generate_greedy(self._e, token, n_new, out.ctypes.data, C.byref(stats), self._err, 1024), "rl_engine_generate_greedy")
        return out, stats.total_ms

    def layer_out(self, l: int) -> np.ndarray:
        return np.ctypeslib.as_array(self.L.rl_engine_last_layer_output(self._e, RL_BACKEND_GPU, l), (self.info.hidden,)).copy()

    def router_ids(self, l: int) -> np.ndarray:
        return np.ctypeslib.as_array(self.L.rl_engine_last_router_ids(self._e, RL_BACKEND_GPU, l), (self.info.top_k,)).copy()

    def final_norm(self) -> np.ndarray:
        return np.ctypeslib.as_array(self.L.rl_engine_last_final_norm(self._e, RL_BACKEND_GPU), (self.info.hidden,)).copy()

    def embedding(self) -> np.ndarray:
        return np.ctypeslib.as_array(self.L.rl_engine_last_embedding(self._e, RL_BACKEND_GPU), (self.info.hidden,)).copy()

    def embed_token(self, token: int) -> np.ndarray:
        out = np.empty(self.info.hidden, np.float32)
        self._ok(self.L.rl_engine_embed_token(self._e, token, out.ctypes.data, self._err, 1024), "rl_engine_embed_token")
        return out

    @property
    def prefill_batch(self) -> int:
        return int(self.L.rl_engine_prefill_batch(self._e))

    def experts_preloaded(self) -> tuple[bool, float]:
        """(every routed expert is resident, milliseconds the load took at open)"""
        ms = C.c_double(0.0)
        return self.L.rl_engine_experts_preloaded(self._e, C.byref(ms)) == 1, float(ms.value)

    def step_bytes(self) -> int:
        return int(self.L.rl_engine_step_bytes(self._e))

    def full_residency_mib(self) -> int:
        return int(self.L.rl_engine_full_residency_mib(self._e))
