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

from .synth import ModelDims, SynthModel

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
