"""Seeded synthetic MoE layers generated directly in HBM (torch is used as an allocator and RNG only), with the same
block recipe as synth.py: random payload bytes, fp16 block scale from the stated range."""
from __future__ import annotations

import torch

from .synth import BLOCK_BYTES, D_OFFSET, Q6_K, MoeDims, expert_d_range


def quant_matrix(gen: torch.Generator, t: int, nrows: int, ncols: int, d_lo: float, d_hi: float, device, sub_scale=None) -> torch.Tensor:
    nb, bb = nrows * (ncols // 256), BLOCK_BYTES[t]
    blocks = torch.randint(0, 256, (nb, bb), dtype=torch.uint8, device=device, generator=gen)
    d = (torch.rand(nb, device=device, generator=gen) * (d_hi - d_lo) + d_lo).to(torch.float16)
    off = D_OFFSET[t]
    blocks[:, off:off + 2] = d.view(torch.uint8).reshape(nb, 2)
    if t == Q6_K and sub_scale is not None:
        lo, hi = sub_scale
        blocks[:, 192:208] = torch.randint(lo, hi + 1, (nb, 16), dtype=torch.int8, device=device, generator=gen).view(torch.uint8)
    return blocks.reshape(-1)


def moe_layer_tensors(seed: int, dims: MoeDims, device, expert_begin: int = 0, expert_count: int | None = None) -> dict:
    """Raw GGUF bytes of one MoE layer on `device`. Under expert parallelism every rank draws the replicated tensors
    from the same seed and only its own experts' matrices (seeded per expert shard)."""
    ec = dims.n_expert - expert_begin if expert_count is None else expert_count
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    h, f, fs = dims.hidden, dims.ffn, dims.ffn_sh
    out = {"router": (torch.randn(dims.n_expert, h, device=device, generator=g) * 0.02).contiguous(),
           "sh_gate_inp": (torch.randn(h, device=device, generator=g) * 0.02).contiguous()}
    slo, shi = expert_d_range(dims.type_sh)
    sub = (-64, 63) if dims.type_sh == Q6_K else None
    out["sh_gate"] = quant_matrix(g, dims.type_sh, fs, h, slo, shi, device, sub)
    out["sh_up"] = quant_matrix(g, dims.type_sh, fs, h, slo, shi, device, sub)
    out["sh_down"] = quant_matrix(g, dims.type_sh, h, fs, slo, shi, device, sub)
    ge = torch.Generator(device=device)
    ge.manual_seed(seed * 1000003 + expert_begin)
    glo, ghi = expert_d_range(dims.type_gu)
    dlo, dhi = expert_d_range(dims.type_down)
    out["gate"] = quant_matrix(ge, dims.type_gu, ec * f, h, glo, ghi, device)
    out["up"] = quant_matrix(ge, dims.type_gu, ec * f, h, glo, ghi, device)
    out["down"] = quant_matrix(ge, dims.type_down, ec * h, f, dlo, dhi, device)
    return out
