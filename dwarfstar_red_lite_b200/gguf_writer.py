"""Minimal GGUF v3 writer for the synthetic Qwen3-Next-shaped models of synth.py.

Writes exactly what the reference's readers require to open a file with the CPU backend
(native/redlite_native_gguf_dir.c:190-270 metadata keys, :320-384 directory geometry;
native/redlite_native_engine.c:198-291 checks): architecture "qwen3next", the qwen3next.* scalars, a
tokenizer.ggml.tokens string array whose length is the vocabulary, and a tensor directory whose offsets are
relative to the aligned end of the directory.
"""
from __future__ import annotations

import struct

import numpy as np

from .synth import ModelDims, SynthModel, iter_model_tensors, tensor_nbytes, tensor_spec

_U32, _F32, _STR, _ARR = 4, 6, 8, 9
ALIGNMENT = 32


def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def _kv_u32(k: str, v: int) -> bytes:
    return _s(k.encode()) + struct.pack("<II", _U32, v)


def _kv_f32(k: str, v: float) -> bytes:
    return _s(k.encode()) + struct.pack("<If", _F32, v)


def _kv_str(k: str, v: str) -> bytes:
    return _s(k.encode()) + struct.pack("<I", _STR) + _s(v.encode())


def metadata(d: ModelDims) -> list[bytes]:
    kv = [
        _kv_str("general.architecture", "qwen3next"),
        _kv_u32("general.alignment", ALIGNMENT),
        _kv_u32("qwen3next.block_count", d.n_layer),
        _kv_u32("qwen3next.embedding_length", d.hidden),
        _kv_u32("qwen3next.feed_forward_length", d.ffn),
        _kv_u32("qwen3next.attention.head_count", d.n_head),
        _kv_u32("qwen3next.attention.head_count_kv", d.n_head_kv),
        _kv_u32("qwen3next.attention.key_length", d.head_dim),
        _kv_u32("qwen3next.attention.value_length", d.head_dim),
        _kv_u32("qwen3next.rope.dimension_count", d.rope_dims),
        _kv_u32("qwen3next.expert_count", d.n_expert),
        _kv_u32("qwen3next.expert_used_count", d.top_k),
        _kv_u32("qwen3next.expert_feed_forward_length", d.ffn),
        _kv_u32("qwen3next.expert_shared_feed_forward_length", d.ffn_sh),
        _kv_u32("qwen3next.ssm.conv_kernel", d.d_conv),
        _kv_u32("qwen3next.ssm.state_size", d.d_state),
        _kv_u32("qwen3next.ssm.group_count", d.n_group),
        _kv_u32("qwen3next.ssm.time_step_rank", d.dt_rank),
        _kv_u32("qwen3next.ssm.inner_size", d.d_inner),
        _kv_u32("qwen3next.context_length", d.context),
        _kv_u32("qwen3next.full_attention_interval", d.full_attention_interval),
        _kv_f32("qwen3next.attention.layer_norm_rms_epsilon", d.rms_eps),
        _kv_f32("qwen3next.rope.freq_base", d.rope_freq_base),
    ]
    toks = b"".join(_s(b"t%d" % i) for i in range(d.vocab))
    kv.append(_s(b"tokenizer.ggml.tokens") + struct.pack("<IIQ", _ARR, _STR, d.vocab) + toks)
    return kv


def write_gguf(path: str, model: SynthModel) -> int:
    """Write the model; returns the file size in bytes."""
    kv = metadata(model.dims)
    names = list(model.tensors)
    directory, offset = [], 0
    for n in names:
        t, shape, arr = model.tensors[n]
        nbytes = arr.nbytes
        directory.append(_s(n.encode()) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", s) for s in shape) +
                         struct.pack("<IQ", t, offset))
        offset += nbytes
        offset += (-offset) % ALIGNMENT
    with open(path, "wb") as f:
        f.write(b"GGUF" + struct.pack("<IQQ", 3, len(names), len(kv)))
        for b in kv:
            f.write(b)
        for b in directory:
            f.write(b)
        pos = f.tell()
        f.write(b"\0" * ((-pos) % ALIGNMENT))
        for n in names:
            arr = model.tensors[n][2]
            f.write(np.ascontiguousarray(arr).reshape(-1).view(np.uint8).data)
            f.write(b"\0" * ((-arr.nbytes) % ALIGNMENT))
        return f.tell()


def write_gguf_streaming(path: str, seed: int, dims: ModelDims, expert_scale: float = 0.2) -> int:
    """Same file as write_gguf(path, synth.model(seed, dims, expert_scale)), written tensor by tensor as it is generated
    (peak memory: one layer). Returns the file size."""
    kv = metadata(dims)
    spec = tensor_spec(dims)
    directory, offset = [], 0
    for name, t, shape in spec:
        directory.append(_s(name.encode()) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", s) for s in shape) + struct.pack("<IQ", t, offset))
        offset += tensor_nbytes(t, shape)
        offset += (-offset) % ALIGNMENT
    with open(path, "wb") as f:
        f.write(b"GGUF" + struct.pack("<IQQ", 3, len(spec), len(kv)))
        for b in kv:
            f.write(b)
        for b in directory:
            f.write(b)
        f.write(b"\0" * ((-f.tell()) % ALIGNMENT))
        for (name, t, shape), (gname, gt, gshape, arr) in zip(spec, iter_model_tensors(seed, dims, expert_scale)):
            if (name, t, tuple(shape)) != (gname, gt, tuple(gshape)) or arr.nbytes != tensor_nbytes(t, shape):
                raise RuntimeError(f"tensor spec and generator disagree at {name} / {gname}")
            f.write(np.ascontiguousarray(arr).reshape(-1).view(np.uint8).data)
            f.write(b"\0" * ((-arr.nbytes) % ALIGNMENT))
        return f.tell()


def load_gguf(path: str, dims: ModelDims) -> SynthModel:
    """Memory-mapped view of a file written by this module (tensor payloads are np.memmap slices, nothing is copied)."""
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    pos = 4
    version, n_tensors, n_kv = struct.unpack_from("<IQQ", mm, pos)
    pos += 20
    scalar = {0: 1, 1: 1, 2: 2, 3: 2, 4: 4, 5: 4, 6: 4, 7: 1, 10: 8, 11: 8, 12: 8}

    def rd_str(p):
        n, = struct.unpack_from("<Q", mm, p)
        return bytes(mm[p + 8:p + 8 + n]).decode(), p + 8 + n

    for _ in range(n_kv):
        _, pos = rd_str(pos)
        t, = struct.unpack_from("<I", mm, pos)
        pos += 4
        if t == 8:
            _, pos = rd_str(pos)
        elif t == 9:
            sub, cnt = struct.unpack_from("<IQ", mm, pos)
            pos += 12
            if sub == 8:
                for _ in range(cnt):
                    n, = struct.unpack_from("<Q", mm, pos)
                    pos += 8 + n
            else:
                pos += cnt * scalar[sub]
        else:
            pos += scalar[t]
    entries = []
    for _ in range(n_tensors):
        name, pos = rd_str(pos)
        nd, = struct.unpack_from("<I", mm, pos)
        pos += 4
        shape = struct.unpack_from("<" + "Q" * nd, mm, pos)
        pos += 8 * nd
        t, off = struct.unpack_from("<IQ", mm, pos)
        pos += 12
        entries.append((name, t, tuple(int(v) for v in shape), off))
    base = pos + (-pos) % ALIGNMENT
    m = SynthModel(dims)
    for name, t, shape, off in entries:
        nb = tensor_nbytes(t, shape)
        raw = mm[base + off:base + off + nb]
        arr = raw.view(np.float32) if t == 0 else raw
        m.tensors[name] = (t, shape, arr)
    return m
