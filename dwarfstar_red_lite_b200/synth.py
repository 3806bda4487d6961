"""Seeded synthetic inputs for the decode hot path: GGML quant blocks, one MoE layer, a whole model, Zipf routing.

No checkpoint or dataset is read anywhere; every tensor is built from a seed with the block layouts the reference
decodes (IQ2_XXS 66 B / 256 values: native/redlite_native_quant_cpu.c:166-191; Q6_K 210 B: :130-153; IQ3_S 110 B:
native/redlite_native_iq3.c:82-91). The fixture recipe "random bytes everywhere, then a realistic fp16 block
scale" is the one of the reference's kernel self-test (native/redmetal_engine_selftest.m:64-76).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

F32, F16, Q6_K, IQ2_XXS, IQ3_S = 0, 1, 14, 16, 21
Q8_0, Q2_K, Q4_K, Q5_K = 8, 10, 12, 13          # further GGUF types served by the stage entry points (dequantise, matvec)
IQ3_XXS, IQ2_S, IQ4_XS = 18, 22, 23             # and three more of the IQ3 family (codebook types), stage entry points only
IQ2_XS, IQ1_M = 17, 29                          # the two types of the reference's routed-expert checker, stage entry points only
BLOCK_BYTES = {Q6_K: 210, IQ2_XXS: 66, IQ3_S: 110, Q8_0: 34, Q2_K: 84, Q4_K: 144, Q5_K: 176, IQ3_XXS: 98, IQ2_S: 82, IQ4_XS: 136, IQ2_XS: 74, IQ1_M: 56}
BLOCK_VALUES = {Q8_0: 32}                        # every other block holds 256 values
D_OFFSET = {Q6_K: 208, IQ2_XXS: 0, IQ3_S: 0, Q8_0: 0, Q2_K: 80, Q4_K: 0, Q5_K: 0, IQ3_XXS: 0, IQ2_S: 0, IQ4_XS: 0, IQ2_XS: 0}
DMIN_OFFSET = {Q2_K: 82, Q4_K: 2, Q5_K: 2}       # second fp16 scale (of the block minimum)
DMIN_FACTOR = {Q2_K: 1.5, Q4_K: 7.5, Q5_K: 15.5}  # dmin ~ d x the mean code, so that d*sc*q - dmin*mn is centred on zero


def row_bytes(ggml_type: int, ncols: int) -> int:
    if ggml_type == F32:
        return ncols * 4
    if ggml_type == F16:
        return ncols * 2
    bv = BLOCK_VALUES.get(ggml_type, 256)
    if ncols % bv:
        raise ValueError(f"quantised rows of type {ggml_type} hold a multiple of {bv} values")
    return ncols // bv * BLOCK_BYTES[ggml_type]


def quant_matrix(rng: np.random.Generator, ggml_type: int, nrows: int, ncols: int, d_lo: float, d_hi: float,
                 sub_scale_range: tuple[int, int] | None = None) -> np.ndarray:
    """uint8 [nrows, row_bytes]: random payload bytes, fp16 block scale d ~ U(d_lo, d_hi).

    For Q6_K the 16 int8 sub-block scales are drawn from sub_scale_range (default the full int8 range)."""
    bv = BLOCK_VALUES.get(ggml_type, 256)
    nb = nrows * (ncols // bv)
    bb = BLOCK_BYTES[ggml_type]
    blocks = np.frombuffer(rng.bytes(nb * bb), dtype=np.uint8).reshape(nb, bb).copy()     # random payload bytes (fast path of the generator)
    d = rng.uniform(d_lo, d_hi, size=nb).astype(np.float16)
    if ggml_type == IQ1_M:
        # the block scale is spread over the top nibbles of the four 16-bit scale words at bytes 48..55
        bits = d.view(np.uint16).astype(np.uint32)
        for k in range(4):
            blocks[:, 49 + 2 * k] = (blocks[:, 49 + 2 * k] & 0x0F) | (((bits >> (4 * k)) & 0xF) << 4).astype(np.uint8)
        return blocks.reshape(nrows, (ncols // bv) * bb)
    off = D_OFFSET[ggml_type]
    blocks[:, off:off + 2] = d.view(np.uint8).reshape(nb, 2)
    if ggml_type in DMIN_OFFSET:
        off = DMIN_OFFSET[ggml_type]
        f = DMIN_FACTOR[ggml_type]
        blocks[:, off:off + 2] = rng.uniform(d_lo * f, d_hi * f, size=nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    if ggml_type == Q6_K and sub_scale_range is not None:
        lo, hi = sub_scale_range
        blocks[:, 192:208] = rng.integers(lo, hi + 1, size=(nb, 16)).astype(np.int8).view(np.uint8)
    return blocks.reshape(nrows, (ncols // bv) * bb)


@dataclass
class MoeDims:
    hidden: int = 2048
    n_expert: int = 512
    top_k: int = 10
    ffn: int = 512
    ffn_sh: int = 512
    type_gu: int = IQ2_XXS
    type_down: int = IQ2_XXS
    type_sh: int = Q6_K


@dataclass
class MoeLayer:
    dims: MoeDims
    router: np.ndarray        # f32 [n_expert, hidden]
    gate: np.ndarray          # u8 [n_expert, ffn * row_bytes(hidden)]
    up: np.ndarray
    down: np.ndarray          # u8 [n_expert, hidden * row_bytes(ffn)]
    sh_gate_inp: np.ndarray   # f32 [hidden]
    sh_gate: np.ndarray       # u8 [ffn_sh, row_bytes(hidden)]
    sh_up: np.ndarray
    sh_down: np.ndarray       # u8 [hidden, row_bytes(ffn_sh)]


def expert_d_range(ggml_type: int, scale: float = 1.0) -> tuple[float, float]:
    """fp16 block-scale range of the routed experts: U(1e-3, 4e-3) for IQ2_XXS as the workload states; the IQ3_S range
    gives weights of a similar magnitude."""
    if ggml_type == IQ2_XXS:
        return 1e-3 * scale, 4e-3 * scale
    if ggml_type == IQ3_S:
        return 5e-4 * scale, 2e-3 * scale
    if ggml_type == Q6_K:
        return 2e-5 * scale, 6e-5 * scale
    if ggml_type == Q8_0:
        return 1.5e-4 * scale, 4e-4 * scale
    if ggml_type == Q4_K:
        return 5e-5 * scale, 1.5e-4 * scale
    if ggml_type == Q5_K:
        return 2.5e-5 * scale, 7e-5 * scale
    if ggml_type == Q2_K:
        return 1e-3 * scale, 3e-3 * scale
    raise ValueError(ggml_type)


def moe_layer(seed: int, dims: MoeDims | None = None, expert_scale: float = 1.0, shared_scale: float = 1.0) -> MoeLayer:
    """One routed-MoE FFN layer: router ~N(0,0.02), routed experts, Q6_K shared expert, sigmoid gate vector ~N(0,0.02)."""
    dims = dims or MoeDims()
    rng = np.random.default_rng(seed)
    h, e, f, fs = dims.hidden, dims.n_expert, dims.ffn, dims.ffn_sh
    router = rng.normal(0.0, 0.02, size=(e, h)).astype(np.float32)
    glo, ghi = expert_d_range(dims.type_gu, expert_scale)
    dlo, dhi = expert_d_range(dims.type_down, expert_scale)
    gate = quant_matrix(rng, dims.type_gu, e * f, h, glo, ghi).reshape(e, -1)
    up = quant_matrix(rng, dims.type_gu, e * f, h, glo, ghi).reshape(e, -1)
    down = quant_matrix(rng, dims.type_down, e * h, f, dlo, dhi).reshape(e, -1)
    slo, shi = expert_d_range(dims.type_sh, shared_scale)
    sub = (-64, 63) if dims.type_sh == Q6_K else None
    sh_gate = quant_matrix(rng, dims.type_sh, fs, h, slo, shi, sub)
    sh_up = quant_matrix(rng, dims.type_sh, fs, h, slo, shi, sub)
    sh_down = quant_matrix(rng, dims.type_sh, h, fs, slo, shi, sub)
    sh_gate_inp = rng.normal(0.0, 0.02, size=h).astype(np.float32)
    return MoeLayer(dims, router, gate, up, down, sh_gate_inp, sh_gate, sh_up, sh_down)


def zipf_routing_logits(seed: int, n_tokens: int, n_expert: int = 512, top_k: int = 10, alpha: float = 1.1) -> np.ndarray:
    """Router logits DRAWN so that per-expert token counts follow Zipf(alpha): every token picks top_k distinct experts
    from the Zipf pmf (expert id = popularity rank); the picked logits sit well above the rest, with pairwise margins
    far above float rounding so that the selection has no ties."""
    rng = np.random.default_rng(seed)
    pmf = 1.0 / np.arange(1, n_expert + 1, dtype=np.float64) ** alpha
    pmf /= pmf.sum()
    logits = rng.normal(0.0, 1.0, size=(n_tokens, n_expert)).astype(np.float32)
    for t in range(n_tokens):
        picked = rng.choice(n_expert, size=top_k, replace=False, p=pmf)
        # strictly decreasing, margin >= 0.05 between selected experts, >= 4 above the unselected bulk
        logits[t, picked] = (8.0 + 0.05 * np.arange(top_k, 0, -1) + rng.uniform(0, 0.04, size=top_k)).astype(np.float32)
    return logits


@dataclass
class ModelDims:
    n_layer: int = 48
    hidden: int = 2048
    vocab: int = 151936
    n_expert: int = 512
    top_k: int = 10
    ffn: int = 512
    ffn_sh: int = 512
    d_conv: int = 4
    d_state: int = 128
    n_group: int = 16
    dt_rank: int = 32
    d_inner: int = 4096
    n_head: int = 16
    n_head_kv: int = 2
    head_dim: int = 256
    rope_dims: int = 64
    rope_freq_base: float = 10000000.0
    rms_eps: float = 1e-6
    full_attention_interval: int = 4
    context: int = 4096
    type_dense: int = Q6_K
    type_shared: int = 0          # type of the shared expert's matrices; 0 = as type_dense
    type_experts: int = IQ2_XXS

    @property
    def channels(self) -> int:
        return 2 * self.d_state * self.n_group + self.d_inner

    def is_attention(self, layer: int) -> bool:
        return (layer + 1) % self.full_attention_interval == 0


def tiny_model_dims(**kw) -> ModelDims:
    """A model small enough for the CPU oracle to decode in seconds, with every structural feature of the big one."""
    base = dict(n_layer=4, hidden=256, vocab=512, n_expert=16, top_k=4, ffn=256, ffn_sh=256, d_conv=4, d_state=64,
                n_group=2, dt_rank=4, d_inner=256, n_head=4, n_head_kv=2, head_dim=64, rope_dims=32,
                full_attention_interval=4, context=64)
    base.update(kw)
    return ModelDims(**base)


@dataclass
class SynthModel:
    dims: ModelDims
    tensors: dict = field(default_factory=dict)   # name -> (ggml_type, shape tuple in GGUF order, np.ndarray payload)


def _dense(rng, t, nrows, ncols, scale=1.0):
    if t == F32:
        return rng.normal(0.0, 0.02 * scale, size=(nrows, ncols)).astype(np.float32)
    lo, hi = expert_d_range(t, scale)
    return quant_matrix(rng, t, nrows, ncols, lo, hi, (-64, 63) if t == Q6_K else None)


def iter_model_tensors(seed: int, dims: ModelDims, expert_scale: float = 0.2):
    """Yields (name, ggml_type, GGUF shape, payload) tensor by tensor, generating each layer only when it is reached, so
    that a 22 GB model can be streamed to a file without being held in memory. Whole random-init Qwen3-Next-shaped model
    under the tensor names the reference audits (native/redlite_native_engine.c:117-183); GGUF shapes list the row
    length first."""
    rng = np.random.default_rng(seed)
    h, td, te = dims.hidden, dims.type_dense, dims.type_experts

    def put(name, t, shape, arr):
        return (name, t, tuple(int(s) for s in shape), np.ascontiguousarray(arr))

    def norm_w(n):
        return (1.0 + rng.normal(0.0, 0.02, size=n)).astype(np.float32)

    yield put("token_embd.weight", td, (h, dims.vocab), _dense(rng, td, dims.vocab, h, 40.0))
    yield put("output_norm.weight", F32, (h,), norm_w(h))
    yield put("output.weight", td, (h, dims.vocab), _dense(rng, td, dims.vocab, h))
    for l in range(dims.n_layer):
        p = f"blk.{l}."
        lr = np.random.default_rng([seed, l + 1])
        yield put(p + "attn_norm.weight", F32, (h,), norm_w(h))
        yield put(p + "post_attention_norm.weight", F32, (h,), norm_w(h))
        if dims.is_attention(l):
            qc, kvc = dims.n_head * dims.head_dim, dims.n_head_kv * dims.head_dim
            yield put(p + "attn_q.weight", td, (h, 2 * qc), _dense(lr, td, 2 * qc, h))
            yield put(p + "attn_k.weight", td, (h, kvc), _dense(lr, td, kvc, h))
            yield put(p + "attn_v.weight", td, (h, kvc), _dense(lr, td, kvc, h))
            yield put(p + "attn_q_norm.weight", F32, (dims.head_dim,), (1.0 + lr.normal(0, 0.02, dims.head_dim)).astype(np.float32))
            yield put(p + "attn_k_norm.weight", F32, (dims.head_dim,), (1.0 + lr.normal(0, 0.02, dims.head_dim)).astype(np.float32))
            yield put(p + "attn_output.weight", td, (qc, h), _dense(lr, td, h, qc))
        else:
            yield put(p + "attn_qkv.weight", td, (h, dims.channels), _dense(lr, td, dims.channels, h))
            yield put(p + "attn_gate.weight", td, (h, dims.d_inner), _dense(lr, td, dims.d_inner, h))
            yield put(p + "ssm_ba.weight", td, (h, 2 * dims.dt_rank), _dense(lr, td, 2 * dims.dt_rank, h))
            yield put(p + "ssm_conv1d.weight", F32, (dims.d_conv, dims.channels),
                lr.normal(0.0, 0.5, size=(dims.channels, dims.d_conv)).astype(np.float32))
            yield put(p + "ssm_dt.bias", F32, (dims.dt_rank,), lr.normal(0.0, 0.5, size=dims.dt_rank).astype(np.float32))
            yield put(p + "ssm_a", F32, (dims.dt_rank,), (-np.exp(lr.normal(0.0, 0.5, size=dims.dt_rank))).astype(np.float32))
            yield put(p + "ssm_norm.weight", F32, (dims.d_state,), (1.0 + lr.normal(0, 0.1, dims.d_state)).astype(np.float32))
            yield put(p + "ssm_out.weight", td, (dims.d_inner, h), _dense(lr, td, h, dims.d_inner))
        ts = dims.type_shared or td
        md = MoeDims(h, dims.n_expert, dims.top_k, dims.ffn, dims.ffn_sh, te, te, ts)
        ml = moe_layer(int(lr.integers(1 << 31)), md, expert_scale=expert_scale)
        yield put(p + "ffn_gate_inp.weight", F32, (h, dims.n_expert), ml.router)
        yield put(p + "ffn_gate_inp_shexp.weight", F32, (h,), ml.sh_gate_inp)
        yield put(p + "ffn_gate_shexp.weight", ts, (h, dims.ffn_sh), ml.sh_gate)
        yield put(p + "ffn_up_shexp.weight", ts, (h, dims.ffn_sh), ml.sh_up)
        yield put(p + "ffn_down_shexp.weight", ts, (dims.ffn_sh, h), ml.sh_down)
        yield put(p + "ffn_gate_exps.weight", te, (h, dims.ffn, dims.n_expert), ml.gate)
        yield put(p + "ffn_up_exps.weight", te, (h, dims.ffn, dims.n_expert), ml.up)
        yield put(p + "ffn_down_exps.weight", te, (dims.ffn, h, dims.n_expert), ml.down)


def model(seed: int, dims: ModelDims, expert_scale: float = 0.2) -> SynthModel:
    """The whole synthetic model in memory (small models: tests)."""
    m = SynthModel(dims)
    for name, t, shape, arr in iter_model_tensors(seed, dims, expert_scale):
        m.tensors[name] = (t, shape, arr)
    return m


def tensor_spec(dims: ModelDims) -> list:
    """(name, ggml_type, GGUF shape) of every tensor in the order iter_model_tensors yields them, without any data."""
    h, td, te = dims.hidden, dims.type_dense, dims.type_experts
    spec = [("token_embd.weight", td, (h, dims.vocab)), ("output_norm.weight", F32, (h,)), ("output.weight", td, (h, dims.vocab))]
    for l in range(dims.n_layer):
        p = f"blk.{l}."
        spec += [(p + "attn_norm.weight", F32, (h,)), (p + "post_attention_norm.weight", F32, (h,))]
        if dims.is_attention(l):
            qc, kvc = dims.n_head * dims.head_dim, dims.n_head_kv * dims.head_dim
            spec += [(p + "attn_q.weight", td, (h, 2 * qc)), (p + "attn_k.weight", td, (h, kvc)), (p + "attn_v.weight", td, (h, kvc)),
                     (p + "attn_q_norm.weight", F32, (dims.head_dim,)), (p + "attn_k_norm.weight", F32, (dims.head_dim,)),
                     (p + "attn_output.weight", td, (qc, h))]
        else:
            spec += [(p + "attn_qkv.weight", td, (h, dims.channels)), (p + "attn_gate.weight", td, (h, dims.d_inner)),
                     (p + "ssm_ba.weight", td, (h, 2 * dims.dt_rank)), (p + "ssm_conv1d.weight", F32, (dims.d_conv, dims.channels)),
                     (p + "ssm_dt.bias", F32, (dims.dt_rank,)), (p + "ssm_a", F32, (dims.dt_rank,)), (p + "ssm_norm.weight", F32, (dims.d_state,)),
                     (p + "ssm_out.weight", td, (dims.d_inner, h))]
        spec += [(p + "ffn_gate_inp.weight", F32, (h, dims.n_expert)), (p + "ffn_gate_inp_shexp.weight", F32, (h,)),
                 (p + "ffn_gate_shexp.weight", dims.type_shared or td, (h, dims.ffn_sh)), (p + "ffn_up_shexp.weight", dims.type_shared or td, (h, dims.ffn_sh)),
                 (p + "ffn_down_shexp.weight", dims.type_shared or td, (dims.ffn_sh, h)), (p + "ffn_gate_exps.weight", te, (h, dims.ffn, dims.n_expert)),
                 (p + "ffn_up_exps.weight", te, (h, dims.ffn, dims.n_expert)), (p + "ffn_down_exps.weight", te, (dims.ffn, h, dims.n_expert))]
    return spec


def tensor_nbytes(ggml_type: int, shape) -> int:
    n = row_bytes(ggml_type, shape[0])
    for s in shape[1:]:
        n *= s
    return n
