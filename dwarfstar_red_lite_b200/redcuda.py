"""ctypes mirror of include/redcuda.h — the call a Python user makes; same names and argument meaning as the C ABI,
which in turn follow the reference's CPU functions (rl_quant_dequant_row, rl_quant_row_dot,
rl_native_router_select_softmax_topk, the ffn() and deltanet_branch() of native/redlite_native_engine_cpu.c)."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("REDCUDA_LIB") or os.path.join(HERE, "libredcuda.so")    # REDCUDA_LIB: an alternative build (A/B runs)

u8p, f32p, u32p = C.POINTER(C.c_uint8), C.POINTER(C.c_float), C.POINTER(C.c_uint32)

EXPORTS = [
    "redcuda_abi_version", "redcuda_last_error", "redcuda_device_count", "redcuda_set_device", "redcuda_set_codebooks", "redcuda_set_codebooks_ext", "redcuda_set_codebooks_xs",
    "redcuda_quant_dequant_rows", "redcuda_nib_dequant_rows", "redcuda_quant_matvec", "redcuda_quant_matmul_tc", "redcuda_router_select_softmax_topk", "redcuda_deltanet_step",
    "redcuda_deltanet_step_noalloc",
    "redcuda_moe_create", "redcuda_moe_destroy", "redcuda_moe_resident_bytes", "redcuda_moe_forward",
    "redcuda_moe_forward_device", "redcuda_moe_route_device", "redcuda_moe_experts_device", "redcuda_moe_shared_device",
    "redcuda_moe_combine_device", "redcuda_moe_partial_device",
    "redcuda_launch_count", "redcuda_profile_enable", "redcuda_profile_report",
    "redcuda_ep_unique_id", "redcuda_ep_ipc_handle", "redcuda_ep_attach_peers", "redcuda_ep_detach_peers", "redcuda_ep_create", "redcuda_ep_destroy", "redcuda_ep_layer_forward", "redcuda_ep_layer_forward_n", "redcuda_ep_last_ids_device", "redcuda_ep_step", "redcuda_engine_shard", "redcuda_engine_attach_ep",
    # engine ABI (include/rl_engine.h)
    "rl_engine_config_default", "rl_engine_open", "rl_engine_close", "rl_engine_info_get", "rl_engine_reset", "rl_engine_position",
    "rl_engine_bench_set_position", "rl_engine_step", "rl_engine_prefill", "rl_engine_last_embedding", "rl_engine_last_layer_output",
    "rl_engine_last_final_norm", "rl_engine_last_router_ids", "rl_engine_experts_preloaded", "rl_engine_full_residency_mib",
    "rl_engine_embed_token", "rl_engine_generate_greedy", "rl_engine_step_bytes", "rl_engine_prefill_batch",
]


class RedcudaError(RuntimeError):
    pass


class DeltanetParams(C.Structure):
    _fields_ = [("d_conv", C.c_uint32), ("d_state", C.c_uint32), ("n_group", C.c_uint32), ("dt_rank", C.c_uint32),
                ("d_inner", C.c_uint32), ("channels", C.c_uint32), ("rms_eps", C.c_float),
                ("conv_kernel", f32p), ("dt_bias", f32p), ("ssm_a", f32p), ("ssm_norm", f32p)]


class MoeDesc(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ["hidden", "n_expert", "top_k", "ffn", "ffn_sh", "type_gu", "type_down", "type_sh",
                                          "expert_begin", "expert_count", "max_tokens", "weights_on_device"]] + \
               [("router", C.c_void_p), ("gate_exps", C.c_void_p), ("up_exps", C.c_void_p), ("down_exps", C.c_void_p),
                ("sh_gate_inp", C.c_void_p), ("sh_gate", C.c_void_p), ("sh_up", C.c_void_p), ("sh_down", C.c_void_p), ("expert_stride", C.c_uint32)]


_lib = None
_books_devices: set[int] = set()


def lib():
    """The loaded C-ABI library. Raises when it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RedcudaError(f"{LIB_PATH} is missing: build it with `python -m dwarfstar_red_lite_b200.build` (no CPU fallback exists)")
    L = C.CDLL(LIB_PATH)
    L.redcuda_last_error.restype = C.c_char_p
    L.redcuda_abi_version.restype = C.c_uint32
    L.redcuda_launch_count.restype = C.c_uint64
    L.redcuda_moe_create.restype = C.c_void_p
    L.redcuda_moe_create.argtypes = [C.POINTER(MoeDesc)]
    L.redcuda_moe_destroy.argtypes = [C.c_void_p]
    L.redcuda_moe_resident_bytes.restype = C.c_uint64
    L.redcuda_moe_resident_bytes.argtypes = [C.c_void_p]
    L.redcuda_moe_forward.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.redcuda_moe_forward_device.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.redcuda_moe_route_device.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.redcuda_moe_experts_device.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.redcuda_moe_shared_device.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p]
    L.redcuda_moe_combine_device.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.redcuda_moe_partial_device.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
    L.redcuda_quant_dequant_rows.argtypes = [C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p]
    L.redcuda_nib_dequant_rows.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p]
    L.redcuda_quant_matvec.argtypes = [C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p]
    L.redcuda_quant_matmul_tc.argtypes = [C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p]
    L.redcuda_router_select_softmax_topk.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p]
    L.redcuda_deltanet_step.argtypes = [C.POINTER(DeltanetParams), C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.redcuda_deltanet_step_noalloc.argtypes = [C.POINTER(DeltanetParams), C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.redcuda_ep_unique_id.argtypes = [C.c_void_p]
    L.redcuda_ep_ipc_handle.argtypes = [C.c_void_p, C.c_void_p]
    L.redcuda_ep_attach_peers.argtypes = [C.c_void_p, C.c_void_p]
    L.redcuda_ep_detach_peers.argtypes = [C.c_void_p]
    L.redcuda_ep_create.restype = C.c_void_p
    L.redcuda_ep_create.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32]
    L.redcuda_ep_destroy.argtypes = [C.c_void_p]
    L.redcuda_ep_layer_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.redcuda_ep_layer_forward_n.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.redcuda_ep_last_ids_device.restype = C.c_void_p
    L.redcuda_ep_last_ids_device.argtypes = [C.c_void_p]
    L.redcuda_engine_shard.argtypes = [C.c_int, C.c_int]
    L.redcuda_engine_attach_ep.argtypes = [C.c_void_p, C.c_void_p]
    L.redcuda_ep_step.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.redcuda_profile_enable.argtypes = [C.c_int]
    L.redcuda_profile_report.argtypes = [C.c_char_p, C.c_size_t]
    L.redcuda_set_device.argtypes = [C.c_int]
    L.redcuda_set_codebooks.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32]
    L.redcuda_set_codebooks_ext.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32]
    L.redcuda_set_codebooks_xs.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32]
    _lib = L
    return L


def profile_enable(on: bool):
    lib().redcuda_profile_enable(C.c_int(1 if on else 0))


def profile_report() -> dict:
    """{kernel name: (launches, total_ms)} since profile_enable(True)."""
    buf = C.create_string_buffer(8192)
    lib().redcuda_profile_report(buf, C.c_size_t(8192))
    out = {}
    for line in buf.value.decode().splitlines():
        name, n, ms = line.split()
        out[name] = (int(n), float(ms))
    return out


def _check(ok: int):
    if ok != 1:
        raise RedcudaError(lib().redcuda_last_error().decode(errors="replace"))


def default_codebooks() -> tuple[np.ndarray, np.ndarray]:
    raw = np.fromfile(os.path.join(HERE, "data", "codebooks.bin"), dtype=np.uint8)
    return raw[:2048].copy(), raw[2048:].view(np.uint32).copy()


def default_codebooks_ext() -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """IQ3_XXS grid (256 x uint32), IQ2_S grid (1024 x uint64), IQ4_NL values (16 x int8) from data/codebooks_iq3family.bin."""
    raw = np.fromfile(os.path.join(HERE, "data", "codebooks_iq3family.bin"), dtype=np.uint8)
    return raw[:1024].view(np.uint32).copy(), raw[1024:9216].view(np.uint64).copy(), raw[9216:9232].view(np.int8).copy()


def set_codebooks_ext(iq3xxs_grid: np.ndarray | None = None, iq2s_grid: np.ndarray | None = None, iq4nl_values: np.ndarray | None = None):
    """Hand the tables of IQ3_XXS / IQ2_S / IQ4_XS to the current device (defaults: data/codebooks_iq3family.bin)."""
    if iq3xxs_grid is None or iq2s_grid is None or iq4nl_values is None:
        iq3xxs_grid, iq2s_grid, iq4nl_values = default_codebooks_ext()
    a = np.ascontiguousarray(iq3xxs_grid, np.uint32)
    b = np.ascontiguousarray(iq2s_grid, np.uint64)
    c = np.ascontiguousarray(iq4nl_values, np.int8)
    _check(lib().redcuda_set_codebooks_ext(a.ctypes.data, a.size, b.ctypes.data, b.size, c.ctypes.data, c.size))


def set_codebooks_xs(iq2xs_grid: np.ndarray | None = None, iq1m_grid: np.ndarray | None = None):
    """Hand the IQ2_XS / IQ1_M grids to the current device (defaults: data/codebooks_iq2xs_iq1m.bin)."""
    if iq2xs_grid is None or iq1m_grid is None:
        raw = np.fromfile(os.path.join(HERE, "data", "codebooks_iq2xs_iq1m.bin"), dtype=np.int8)
        iq2xs_grid, iq1m_grid = raw[:4096].copy(), raw[4096:20480].copy()
    a = np.ascontiguousarray(iq2xs_grid, np.int8)
    b = np.ascontiguousarray(iq1m_grid, np.int8)
    _check(lib().redcuda_set_codebooks_xs(a.ctypes.data, a.size, b.ctypes.data, b.size))


def set_codebooks(iq2xxs_grid: np.ndarray | None = None, iq3s_grid: np.ndarray | None = None, device: int | None = None):
    """Hand the IQ2_XXS / IQ3_S codebooks to the current device (defaults: data/codebooks.bin); with the defaults the tables
    of IQ3_XXS / IQ2_S / IQ4_XS and the IQ2_XS / IQ1_M grids go along."""
    ext = iq2xxs_grid is None or iq3s_grid is None
    if iq2xxs_grid is None or iq3s_grid is None:
        iq2xxs_grid, iq3s_grid = default_codebooks()
    g2 = np.ascontiguousarray(iq2xxs_grid, np.uint8)
    g3 = np.ascontiguousarray(iq3s_grid, np.uint32)
    if device is not None:
        _check(lib().redcuda_set_device(C.c_int(device)))
    _check(lib().redcuda_set_codebooks(g2.ctypes.data, g2.size, g3.ctypes.data, g3.size))
    if ext:
        set_codebooks_ext()
        set_codebooks_xs()
    _books_devices.add(-1 if device is None else device)


def _ensure_books():
    if not _books_devices:
        set_codebooks()


def quant_dequant_rows(ggml_type: int, rows: np.ndarray, ncols: int) -> np.ndarray:
    _ensure_books()
    rows = np.ascontiguousarray(rows).view(np.uint8)
    nrows = rows.size // max(1, _row_bytes(ggml_type, ncols))
    out = np.empty((nrows, ncols), np.float32)
    _check(lib().redcuda_quant_dequant_rows(ggml_type, rows.ctypes.data, nrows, ncols, out.ctypes.data))
    return out


def nib_dequant_rows(rows: np.ndarray, ncols: int) -> np.ndarray:
    """IQ2_XXS rows dequantised through the nibble layout of the routed experts (must equal quant_dequant_rows(16, ...))."""
    _ensure_books()
    rows = np.ascontiguousarray(rows).view(np.uint8)
    nrows = rows.size // _row_bytes(16, ncols)
    out = np.empty((nrows, ncols), np.float32)
    _check(lib().redcuda_nib_dequant_rows(rows.ctypes.data, nrows, ncols, out.ctypes.data))
    return out


def _row_bytes(t: int, ncols: int) -> int:
    from .synth import row_bytes
    return row_bytes(t, ncols)


def quant_matvec(ggml_type: int, w: np.ndarray, nrows: int, ncols: int, x: np.ndarray) -> np.ndarray:
    """out[t][r] = dot(W[r], x[t]); x is [ncols] or [ntok, ncols]."""
    _ensure_books()
    w = np.ascontiguousarray(w).view(np.uint8)
    x2 = np.ascontiguousarray(x, np.float32).reshape(-1, ncols)
    out = np.empty((x2.shape[0], nrows), np.float32)
    _check(lib().redcuda_quant_matvec(ggml_type, w.ctypes.data, nrows, ncols, x2.ctypes.data, x2.shape[0], out.ctypes.data))
    return out if np.ndim(x) > 1 else out[0]


def quant_matmul_tc(ggml_type: int, w: np.ndarray, nrows: int, ncols: int, x: np.ndarray) -> np.ndarray:
    """quant_matvec for a chunk of tokens on the tcgen05 tensor cores; x is [ntok, ncols]."""
    _ensure_books()
    w = np.ascontiguousarray(w).view(np.uint8)
    x2 = np.ascontiguousarray(x, np.float32).reshape(-1, ncols)
    out = np.empty((x2.shape[0], nrows), np.float32)
    _check(lib().redcuda_quant_matmul_tc(ggml_type, w.ctypes.data, nrows, ncols, x2.ctypes.data, x2.shape[0], out.ctypes.data))
    return out


def router_select_softmax_topk(logits: np.ndarray, top_k: int, want_probs: bool = False):
    l2 = np.ascontiguousarray(logits, np.float32)
    l2 = l2.reshape(-1, l2.shape[-1])
    ntok, n = l2.shape
    ids = np.empty((ntok, top_k), np.uint32)
    w = np.empty((ntok, top_k), np.float32)
    probs = np.empty((ntok, n), np.float32) if want_probs else None
    _check(lib().redcuda_router_select_softmax_topk(l2.ctypes.data, ntok, n, top_k, ids.ctypes.data, w.ctypes.data,
                                                    probs.ctypes.data if want_probs else None))
    return (ids, w, probs) if want_probs else (ids, w)


def deltanet_step(p: dict, qkv: np.ndarray, z: np.ndarray, ba: np.ndarray, conv_state: np.ndarray, rec_state: np.ndarray) -> np.ndarray:
    """Batched DeltaNet step; qkv [B, channels], z [B, d_inner], ba [B, 2*dt_rank]; states updated in place."""
    arrs = {k: np.ascontiguousarray(p[k], np.float32) for k in ("conv_kernel", "dt_bias", "ssm_a", "ssm_norm")}
    P = DeltanetParams(p["d_conv"], p["d_state"], p["n_group"], p["dt_rank"], p["d_inner"], p["channels"], p["rms_eps"],
                       arrs["conv_kernel"].ctypes.data_as(f32p), arrs["dt_bias"].ctypes.data_as(f32p),
                       arrs["ssm_a"].ctypes.data_as(f32p), arrs["ssm_norm"].ctypes.data_as(f32p))
    qkv, z, ba = (np.ascontiguousarray(a, np.float32) for a in (qkv, z, ba))
    B = qkv.reshape(-1, p["channels"]).shape[0]
    for s in (conv_state, rec_state):
        if s.dtype != np.float32 or not s.flags.c_contiguous:
            raise ValueError("states must be C-contiguous float32 arrays (they are updated in place)")
    out = np.empty((B, p["d_inner"]), np.float32)
    _check(lib().redcuda_deltanet_step(C.byref(P), B, qkv.ctypes.data, z.ctypes.data, ba.ctypes.data, conv_state.ctypes.data,
                                       rec_state.ctypes.data, out.ctypes.data))
    return out


class MoeLayer:
    """One resident MoE layer (router + every routed expert + shared expert in HBM)."""

    def __init__(self, layer=None, max_tokens: int = 64, expert_begin: int = 0, expert_count: int | None = None, device_tensors: dict | None = None,
                 dims=None, expert_stride: int = 1):
        """layer: a synth.MoeLayer with host arrays; or device_tensors: dict of torch CUDA uint8/float32 tensors with the
        same field names (raw GGUF bytes on the device), with dims given."""
        _ensure_books()
        self._h = None
        d = dims if dims is not None else layer.dims
        self.dims = d
        self.max_tokens = max_tokens
        st = max(1, expert_stride)
        ec = (d.n_expert - expert_begin + st - 1) // st if expert_count is None else expert_count
        names = ["router", "gate", "up", "down", "sh_gate_inp", "sh_gate", "sh_up", "sh_down"]
        if device_tensors is not None:
            ptrs = [device_tensors[n].data_ptr() for n in names]
            on_dev = 1
            keep = device_tensors
        else:
            keep = [np.ascontiguousarray(getattr(layer, n)) for n in names]
            # an expert shard takes the slice of the expert-major arrays
            gu, dn = keep[1].reshape(d.n_expert, -1), keep[3].reshape(d.n_expert, -1)
            sel = slice(expert_begin, expert_begin + (ec - 1) * st + 1, st)
            keep[1] = np.ascontiguousarray(gu[sel])
            keep[2] = np.ascontiguousarray(keep[2].reshape(d.n_expert, -1)[sel])
            keep[3] = np.ascontiguousarray(dn[sel])
            ptrs = [a.ctypes.data for a in keep]
            on_dev = 0
        desc = MoeDesc(d.hidden, d.n_expert, d.top_k, d.ffn, d.ffn_sh, d.type_gu, d.type_down, d.type_sh, expert_begin, ec, max_tokens, on_dev, *ptrs, st)
        h = lib().redcuda_moe_create(C.byref(desc))
        del keep
        if not h:
            raise RedcudaError(lib().redcuda_last_error().decode(errors="replace"))
        self._h = h

    def close(self):
        if self._h:
            lib().redcuda_moe_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    def resident_bytes(self) -> int:
        return int(lib().redcuda_moe_resident_bytes(self._h))

    def forward(self, x: np.ndarray, logits_in: np.ndarray | None = None, out: np.ndarray | None = None, want_routing: bool = False):
        """Host call (the end-to-end path): x [ntok, hidden] float32 (pinned or pageable) -> out [ntok, hidden]."""
        d = self.dims
        x2 = np.ascontiguousarray(x, np.float32).reshape(-1, d.hidden)
        ntok = x2.shape[0]
        if out is None:
            out = np.empty((ntok, d.hidden), np.float32)
        li = None if logits_in is None else np.ascontiguousarray(logits_in, np.float32)
        ids = np.empty((ntok, d.top_k), np.uint32) if want_routing else None
        w = np.empty((ntok, d.top_k), np.float32) if want_routing else None
        lo = np.empty((ntok, d.n_expert), np.float32) if want_routing else None
        _check(lib().redcuda_moe_forward(self._h, ntok, x2.ctypes.data, None if li is None else li.ctypes.data, out.ctypes.data,
                                         None if ids is None else ids.ctypes.data, None if w is None else w.ctypes.data,
                                         None if lo is None else lo.ctypes.data))
        return (out, ids, w, lo) if want_routing else out

    def forward_device(self, ntok: int, x_ptr: int, out_ptr: int, stream: int, logits_ptr: int = 0, resid_ptr: int = 0):
        _check(lib().redcuda_moe_forward_device(self._h, ntok, x_ptr, logits_ptr or None, resid_ptr or None, out_ptr, stream or None))

    def route_device(self, ntok: int, x_ptr: int, ids_ptr: int, weights_ptr: int, stream: int, logits_ptr: int = 0):
        _check(lib().redcuda_moe_route_device(self._h, ntok, x_ptr or None, logits_ptr or None, ids_ptr, weights_ptr, stream or None))

    def experts_device(self, npairs: int, pair_x_ptr: int, pair_expert_ptr: int, pair_out_ptr: int, stream: int):
        _check(lib().redcuda_moe_experts_device(self._h, npairs, pair_x_ptr, pair_expert_ptr, pair_out_ptr, stream or None))

    def combine_device(self, ntok: int, pair_out_ptr: int, pair_row_ptr: int, weights_ptr: int, add_ptr: int, resid_ptr: int, out_ptr: int, stream: int):
        _check(lib().redcuda_moe_combine_device(self._h, ntok, pair_out_ptr, pair_row_ptr or None, weights_ptr, add_ptr or None, resid_ptr or None,
                                                out_ptr, stream or None))

    def partial_device(self, ntok: int, x_ptr: int, x_stride: int, ids_ptr: int, weights_ptr: int, meta_stride: int, out_ptr: int, stream: int):
        """out[t] = sum over token t's pairs whose expert lives on this shard of weight * expert(x[t])"""
        _check(lib().redcuda_moe_partial_device(self._h, ntok, x_ptr, x_stride, ids_ptr, weights_ptr, meta_stride, out_ptr, stream or None))

    def shared_device(self, ntok: int, x_ptr: int, out_ptr: int, stream: int):
        _check(lib().redcuda_moe_shared_device(self._h, ntok, x_ptr, out_ptr, stream or None))
