"""The allocation-free DeltaNet entry point (redcuda_deltanet_step_noalloc) against the allocating one.

Some users of the library cannot let a call allocate device memory: a decode loop with a latency budget (the CUDA
allocator stalls the device), or a process whose GPU memory is managed by someone else. For them the library carries a
fixed scratch array; this test drives the entry point through the C ABI with device buffers it allocates itself (torch
only provides the memory), twice in a row so that the second call runs on whatever the first one left in the shared
scratch, and requires the same outputs and states as redcuda_deltanet_step — and, so that the chain does not end at
another entry point of the same library, as the CPU oracle within the stage tolerances of the reference
(native/redlite_native_deltanet_state_cli.c:267-269). Kept in a file of its own that pytest collects last."""
import ctypes as C

import numpy as np
import pytest

import dwarfstar_red_lite_b200 as rc
import oracle_lib as ol
from dwarfstar_red_lite_b200.redcuda import DeltanetParams, f32p

pytestmark = pytest.mark.gpu


def _inputs(seed, B, S=128, groups=16, rank=32, d_conv=4):
    rng = np.random.default_rng(seed)
    d_inner, channels = rank * S, 2 * S * groups + rank * S
    p = dict(d_conv=d_conv, d_state=S, n_group=groups, dt_rank=rank, d_inner=d_inner, channels=channels, rms_eps=1e-6,
             conv_kernel=rng.normal(0, 0.5, size=(channels, d_conv)).astype(np.float32), dt_bias=rng.normal(0, 0.3, rank).astype(np.float32),
             ssm_a=-np.exp(rng.normal(0, 0.3, rank)).astype(np.float32), ssm_norm=(1 + rng.normal(0, 0.1, S)).astype(np.float32))
    arrs = dict(qkv=rng.normal(0, 1, size=(B, channels)), z=rng.normal(0, 1, size=(B, d_inner)), ba=rng.normal(0, 1, size=(B, 2 * rank)),
                conv=rng.normal(0, 1, size=(B, channels, d_conv - 1)), rec=rng.normal(0, 0.05, size=(B, rank, S, S)))
    return p, {k: v.astype(np.float32) for k, v in arrs.items()}


@pytest.mark.parametrize("B", [1, 8, 10])      # 10 sequences of this shape is the most the built-in scratch holds
def test_noalloc_matches_allocating_entry_point_twice(B):
    import torch
    lib = rc.lib()
    p, a = _inputs(90 + B, B)
    dev = torch.device("cuda", 0)
    pd = {k: torch.from_numpy(np.ascontiguousarray(p[k])).to(dev) for k in ("conv_kernel", "dt_bias", "ssm_a", "ssm_norm")}
    P = DeltanetParams(p["d_conv"], p["d_state"], p["n_group"], p["dt_rank"], p["d_inner"], p["channels"], p["rms_eps"],
                       C.cast(pd["conv_kernel"].data_ptr(), f32p), C.cast(pd["dt_bias"].data_ptr(), f32p),
                       C.cast(pd["ssm_a"].data_ptr(), f32p), C.cast(pd["ssm_norm"].data_ptr(), f32p))
    conv_ref, rec_ref = a["conv"].copy(), a["rec"].copy()
    conv_cpu, rec_cpu = a["conv"].copy(), a["rec"].copy()
    conv_d, rec_d = torch.from_numpy(a["conv"].copy()).to(dev), torch.from_numpy(a["rec"].copy()).to(dev)
    z_d, ba_d = torch.from_numpy(a["z"]).to(dev), torch.from_numpy(a["ba"]).to(dev)
    out_d = torch.empty(B, p["d_inner"], device=dev)
    for call in range(2):                       # the second call meets the first call's leftovers in the shared scratch
        qkv = np.roll(a["qkv"], call * 7, axis=1).copy()
        want = rc.deltanet_step(p, qkv, a["z"], a["ba"], conv_ref, rec_ref)
        qkv_d = torch.from_numpy(qkv).to(dev)
        torch.cuda.synchronize()
        ok = lib.redcuda_deltanet_step_noalloc(C.byref(P), B, qkv_d.data_ptr(), z_d.data_ptr(), ba_d.data_ptr(), conv_d.data_ptr(), rec_d.data_ptr(),
                                               out_d.data_ptr(), None)
        assert ok == 1, lib.redcuda_last_error().decode()
        torch.cuda.synchronize()
        assert np.array_equal(out_d.cpu().numpy(), want), call          # same kernels, same order: bit-identical
        assert np.array_equal(rec_d.cpu().numpy(), rec_ref) and np.array_equal(conv_d.cpu().numpy(), conv_ref)
        got, rec_got = out_d.cpu().numpy(), rec_d.cpu().numpy()
        for b in range(min(B, 2)):              # the CPU oracle on the first sequences: output 1e-3 of its range, state 3e-6 + 3e-5 |ref|
            cpu = ol.deltanet_mid(p, qkv[b], a["z"][b], a["ba"][b], conv_cpu[b], rec_cpu[b])
            assert np.max(np.abs(got[b] - cpu)) <= 1e-3 * np.max(np.abs(cpu)), (call, b)
            assert np.all(np.abs(rec_got[b] - rec_cpu[b]) <= 3e-6 + 3e-5 * np.abs(rec_cpu[b])), (call, b)


def test_noalloc_rejects_oversized_batch():
    import torch
    lib = rc.lib()
    p, a = _inputs(3, 1)
    dev = torch.device("cuda", 0)
    dummy = torch.zeros(16, device=dev)
    P = DeltanetParams(p["d_conv"], p["d_state"], p["n_group"], p["dt_rank"], p["d_inner"], p["channels"], p["rms_eps"],
                       C.cast(dummy.data_ptr(), f32p), C.cast(dummy.data_ptr(), f32p), C.cast(dummy.data_ptr(), f32p), C.cast(dummy.data_ptr(), f32p))
    ptr = dummy.data_ptr()
    for batch in (11, 64):                      # one sequence beyond the limit of this shape, and far beyond it
        ok = lib.redcuda_deltanet_step_noalloc(C.byref(P), batch, ptr, ptr, ptr, ptr, ptr, ptr, None)
        assert ok == 0
        msg = lib.redcuda_last_error().decode()
        assert "scratch" in msg and str(batch) in msg
