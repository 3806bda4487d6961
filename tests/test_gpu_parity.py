"""GPU parity tests proper: every case calls the CUDA library through its C ABI (ctypes mirror) and compares with the
CPU oracle on the same seeded inputs. Integer / index work must match exactly; floating point within the stated
tolerance (fp32 accumulation on the GPU against the oracle's double)."""
import numpy as np
import pytest

import oracle_lib as ol
import dwarfstar_red_lite_b200 as rc
from dwarfstar_red_lite_b200 import synth

pytestmark = pytest.mark.gpu

# kernel self-test protocol of the reference (native/redmetal_engine_selftest.m:103-117, 317-321):
# 37 rows x {256, 768, 2048, 4096} columns, error relative to sum |w*x| at most 2e-5
SELFTEST_COLS = (256, 768, 2048, 4096)
SELFTEST_ROWS = 37
REL_SUMABS = 2e-5
REL_OUT = 1e-3            # layer outputs: max |gpu - ref| <= REL_OUT * max |ref|


def _rows(rng, t, nrows, ncols):
    if t == synth.F32:
        return rng.uniform(-1, 1, size=(nrows, ncols)).astype(np.float32).view(np.uint8).reshape(nrows, -1)
    if t == synth.F16:
        return rng.uniform(-1, 1, size=(nrows, ncols)).astype(np.float16).view(np.uint8).reshape(nrows, -1)
    lo, hi = {synth.Q6_K: (1e-3, 5e-3), synth.IQ2_XXS: (1e-2, 6e-2), synth.IQ3_S: (2e-3, 1.2e-2), synth.Q8_0: (1e-3, 8e-3), synth.Q2_K: (2e-2, 8e-2),
              synth.Q4_K: (1e-3, 5e-3), synth.Q5_K: (1e-3, 5e-3), synth.IQ3_XXS: (2e-3, 1.2e-2), synth.IQ2_S: (1e-2, 6e-2), synth.IQ4_XS: (1e-3, 5e-3),
              synth.IQ2_XS: (1e-2, 6e-2), synth.IQ1_M: (2e-2, 1e-1)}[t]
    return synth.quant_matrix(rng, t, nrows, ncols, lo, hi)


@pytest.mark.parametrize("t", [synth.Q6_K, synth.IQ2_XXS, synth.IQ3_S, synth.F16, synth.Q8_0, synth.Q2_K, synth.Q4_K, synth.Q5_K,
                               synth.IQ3_XXS, synth.IQ2_S, synth.IQ4_XS, synth.IQ2_XS, synth.IQ1_M])
def test_dequant_bit_exact(t):
    rng = np.random.default_rng(1000 + t)
    for ncols in SELFTEST_COLS:
        rows = _rows(rng, t, SELFTEST_ROWS, ncols)
        got = rc.quant_dequant_rows(t, rows, ncols)
        want = ol.dequant_rows(t, rows, ncols)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (t, ncols)


@pytest.mark.parametrize("nrows,ncols", [(16, 256), (48, 512), (32, 2048)])
def test_nibble_layout_keeps_every_value(nrows, ncols):
    """The routed experts are re-coded at load (4-bit magnitude/sign codes, byte scales); decoding that layout must give
    the oracle's dequantised values bit for bit, subnormal and extreme block scales included."""
    rng = np.random.default_rng(300 + ncols)
    rows = _rows(rng, synth.IQ2_XXS, nrows, ncols).copy()
    rb = rows.reshape(nrows, ncols // 256, 66)
    rb[0, 0, 0:2] = np.frombuffer(np.float16(6e-8).tobytes(), np.uint8)       # fp16-subnormal d
    rb[1, 0, 0:2] = np.frombuffer(np.float16(-3.5).tobytes(), np.uint8)       # negative d
    rb[2, 0, 62:66] = 0xFF                                                    # scale 15, every sign bit set
    rb[3, 0, 62:66] = 0x00
    got = rc.nib_dequant_rows(rows, ncols)
    want = ol.dequant_rows(synth.IQ2_XXS, rows, ncols)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequant_subnormal_block_scale():
    # Q6_K block whose fp16 d is the smallest subnormal (reference KAT, native/redlite_native_shared_exec_offline_test.c:32-44)
    blk = np.zeros((1, 210), np.uint8)
    blk[0, 192:208] = 1
    blk[0, 208] = 1
    got = rc.quant_dequant_rows(synth.Q6_K, blk, 256)
    assert np.all(got == np.float32(-32.0 * 2.0 ** -24))


@pytest.mark.parametrize("t", [synth.Q6_K, synth.IQ2_XXS, synth.IQ3_S, synth.F32, synth.F16, synth.Q8_0, synth.Q2_K, synth.Q4_K, synth.Q5_K,
                               synth.IQ3_XXS, synth.IQ2_S, synth.IQ4_XS, synth.IQ2_XS, synth.IQ1_M])
@pytest.mark.parametrize("ntok", [1, 3, 9])
def test_matvec_selftest_protocol(t, ntok):
    rng = np.random.default_rng(2000 + t + ntok)
    worst = 0.0
    for ncols in SELFTEST_COLS:
        rows = _rows(rng, t, SELFTEST_ROWS, ncols)
        x = rng.uniform(-1, 1, size=(ntok, ncols)).astype(np.float32)
        got = rc.quant_matvec(t, rows, SELFTEST_ROWS, ncols, x)
        deq = ol.dequant_rows(t, rows, ncols).astype(np.float64)
        for tk in range(ntok):
            ref = ol.rows_dot(t, rows, x[tk])
            mag = np.abs(deq * x[tk].astype(np.float64)).sum(axis=1) + 1e-12
            err = np.abs(got[tk].astype(np.float64) - ref) / mag
            worst = max(worst, float(err.max()))
    assert worst <= REL_SUMABS, worst


def test_matvec_large_rows_and_kats():
    # many rows (grid larger than one wave) and the all-ones known answers
    blk = np.zeros((1, 66), np.uint8)
    blk[0, 0:2] = np.array([1.0], np.float16).view(np.uint8)
    assert rc.quant_matvec(synth.IQ2_XXS, blk, 1, 256, np.ones(256, np.float32))[0] == 256.0
    q6 = np.zeros((1, 210), np.uint8)
    q6[0, 192:208] = 1
    q6[0, 208:210] = np.array([1.0], np.float16).view(np.uint8)
    assert rc.quant_matvec(synth.Q6_K, q6, 1, 256, np.ones(256, np.float32))[0] == -8192.0
    rng = np.random.default_rng(5)
    rows = _rows(rng, synth.Q6_K, 5000, 512)
    x = rng.normal(0, 1, 512).astype(np.float32)
    got = rc.quant_matvec(synth.Q6_K, rows, 5000, 512, x)
    ref = ol.matvec(synth.Q6_K, rows, 5000, 512, x, threads=8)
    assert np.max(np.abs(got - ref)) <= 1e-4 * np.max(np.abs(ref))


@pytest.mark.parametrize("t", [synth.Q6_K, synth.IQ2_XXS, synth.IQ3_S])
@pytest.mark.parametrize("ntok,nrows,ncols", [(5, 64, 256), (40, 200, 512), (128, 384, 2048), (200, 130, 768)])
def test_matmul_tensor_core(t, ntok, nrows, ncols):
    """tcgen05 chunk GEMM against the oracle's row dots: ragged row tiles (64, 130, 200 rows), ragged and multiple token
    tiles (5, 40, 200 tokens), every quantised format; activations of mixed magnitude exercise the per-token scaling."""
    rng = np.random.default_rng(4000 + t + ntok)
    rows = _rows(rng, t, nrows, ncols)
    x = (rng.normal(0, 1, size=(ntok, ncols)) * np.exp(rng.uniform(-6, 6, size=(ntok, 1)))).astype(np.float32)
    x[ntok // 2] = 0.0
    got = rc.quant_matmul_tc(t, rows, nrows, ncols, x)
    deq = ol.dequant_rows(t, rows, ncols).astype(np.float64)
    worst = 0.0
    for tk in range(ntok):
        ref = ol.rows_dot(t, rows, x[tk])
        mag = np.abs(deq * x[tk].astype(np.float64)).sum(axis=1) + 1e-30
        worst = max(worst, float((np.abs(got[tk].astype(np.float64) - ref) / mag).max()))
    assert np.all(got[ntok // 2] == 0.0)
    assert worst <= REL_SUMABS, worst


def test_router_topk_exact_incl_ties():
    rng = np.random.default_rng(7)
    n, k = 512, 10
    logits = rng.normal(0, 2, size=(64, n)).astype(np.float32)
    for case in range(0, 64, 4):    # exact ties, as the reference's kernel self-test does (redmetal_engine_selftest.m:185-196)
        logits[case, rng.integers(0, n, 24)] = logits[case, 3]
    logits[1, :] = 0.25            # everything tied -> ids 0..k-1
    ids, w, probs = rc.router_select_softmax_topk(logits, k, want_probs=True)
    for c in range(64):
        rid, rw, rp = ol.router_select(logits[c], k)
        assert np.array_equal(ids[c], rid), c
        assert np.allclose(w[c], rw, rtol=2e-6, atol=1e-9)
        assert np.allclose(probs[c], rp, rtol=2e-6, atol=1e-12)
    assert list(ids[1]) == list(range(k))
    # reference KATs (native/redlite_native_router_offline_test.c:8-30)
    ids, w = rc.router_select_softmax_topk(np.array([[0, 1, 2, 3]], np.float32), 2)
    assert list(ids[0]) == [3, 2] and abs(w[0, 0] - 0.7310585786) < 1e-6
    ids, _ = rc.router_select_softmax_topk(np.array([[1, 1, 0, 0]], np.float32), 2)
    assert list(ids[0]) == [0, 1]


def test_non_finite_router_logits_are_an_error_not_an_address():
    """NaN logits give no maximum, so no expert id: the reference fails with "invalid router softmax denominator"
    (native/redlite_native_router_exec.c:135). Here the kernels clamp the id they could not form (nothing is read
    out of bounds) and the synchronous entry points report the failure; the next call works again."""
    logits = np.random.default_rng(2).normal(0, 1, size=(3, 64)).astype(np.float32)
    logits[1, :] = np.nan
    with pytest.raises(rc.RedcudaError, match="router softmax"):
        rc.router_select_softmax_topk(logits, 4)
    ids, _ = rc.router_select_softmax_topk(logits[:1], 4)
    assert np.array_equal(ids[0], ol.router_select(logits[0], 4)[0])
    dims = synth.MoeDims(hidden=512, n_expert=32, top_k=4, ffn=256, ffn_sh=256)
    layer = synth.moe_layer(5, dims, expert_scale=0.5)
    x = np.random.default_rng(3).normal(0, 1, size=(2, dims.hidden)).astype(np.float32)
    bad = np.full((2, dims.n_expert), np.nan, np.float32)
    m = rc.MoeLayer(layer, max_tokens=2)
    try:
        with pytest.raises(rc.RedcudaError, match="router softmax"):
            m.forward(x, logits_in=bad)
        out = m.forward(x)                       # the layer is usable afterwards
        ro = ol.moe_ffn(layer, x[0], threads=4)[0]
        assert np.max(np.abs(out[0] - ro)) <= REL_OUT * np.max(np.abs(ro))
    finally:
        m.close()


def _check_moe(layer, x, logits_in=None, threads=8, rows=None, expect_kernel=None):
    d = layer.dims
    m = rc.MoeLayer(layer, max_tokens=x.shape[0])
    try:
        if expect_kernel:           # one pass with per-kernel timing on (single stream) to see which kernels ran
            rc.redcuda.profile_enable(True)
            m.forward(x, logits_in=logits_in)
            names = rc.redcuda.profile_report()
            rc.redcuda.profile_enable(False)
            assert expect_kernel in names, sorted(names)
        out, ids, w, logits = m.forward(x, logits_in=logits_in, want_routing=True)
    finally:
        m.close()
    view = ol.moe_layer_c(layer)
    for t in (range(x.shape[0]) if rows is None else rows):
        ro, rid, rw, rl = ol.moe_ffn(layer, x[t], threads=threads, logits_in=None if logits_in is None else logits_in[t], view=view)
        if logits_in is None:
            assert np.array_equal(logits[t].view(np.uint32), rl.view(np.uint32)), "router logits differ"
        assert np.array_equal(ids[t], rid), (t, ids[t], rid)
        assert np.allclose(w[t], rw, rtol=1e-5)
        err = np.max(np.abs(out[t] - ro)) / max(np.max(np.abs(ro)), 1e-30)
        assert err <= REL_OUT, (t, err)
    return out


@pytest.mark.parametrize("te", [synth.IQ2_XXS, synth.IQ3_S])
@pytest.mark.parametrize("ntok", [1, 7])
def test_moe_layer_small(te, ntok):
    dims = synth.MoeDims(hidden=512, n_expert=32, top_k=4, ffn=256, ffn_sh=256, type_gu=te, type_down=te)
    layer = synth.moe_layer(21 + te, dims, expert_scale=0.5)
    x = np.random.default_rng(3).normal(0, 1, size=(ntok, dims.hidden)).astype(np.float32)
    _check_moe(layer, x)


@pytest.fixture(scope="module")
def full_layer():
    return synth.moe_layer(1234)          # 512 experts, hidden 2048, ffn 512, IQ2_XXS experts, Q6_K shared expert


def test_moe_layer_config0_batch1(full_layer):
    x = np.random.default_rng(9).normal(0, 1, size=(1, 2048)).astype(np.float32)
    _check_moe(full_layer, x)


def test_moe_layer_config1_ragged_zipf(full_layer):
    # 64 sequences, router logits drawn so that per-expert token counts follow Zipf(1.1)
    x = np.random.default_rng(10).normal(0, 1, size=(64, 2048)).astype(np.float32)
    logits = synth.zipf_routing_logits(77, 64)
    _check_moe(full_layer, x, logits_in=logits)


def test_moe_chunk_on_tcgen05_small(monkeypatch):
    """A chunk large enough for the tcgen05 expert kernel (>= 16 pairs per expert): 8 experts, 160 tokens, so that experts
    get more than one 64-pair work item and ragged last items."""
    monkeypatch.setenv("RC_MOE_TC_MIN", "16")
    dims = synth.MoeDims(hidden=512, n_expert=8, top_k=2, ffn=256, ffn_sh=256)
    layer = synth.moe_layer(31, dims, expert_scale=0.5)
    x = np.random.default_rng(4).normal(0, 1, size=(160, dims.hidden)).astype(np.float32)
    _check_moe(layer, x, expect_kernel="moe_gateup_tc")


def test_router_logits_of_a_large_batch_are_the_double_sums():
    """300 tokens x 96 experts: the fp64 GEMM with 32 x 64 block tiles (ragged in both directions) must give the logits of
    the oracle's double-precision row dots bit for bit, and so the same selection."""
    dims = synth.MoeDims(hidden=512, n_expert=96, top_k=4, ffn=256, ffn_sh=256)
    layer = synth.moe_layer(57, dims, expert_scale=0.5)
    x = np.random.default_rng(8).normal(0, 1, size=(300, dims.hidden)).astype(np.float32)
    _check_moe(layer, x, rows=list(range(0, 300, 7)) + [299], expect_kernel="moe_router_logits")


def test_moe_chunk_on_tcgen05_full_size(full_layer, monkeypatch):
    """1024 tokens through the full-size layer with Zipf-skewed routing: the popular experts see hundreds of pairs (many
    work items each), the tail ones a handful. Every 16th token is compared with the oracle."""
    monkeypatch.setenv("RC_MOE_TC_MIN", "16")
    x = np.random.default_rng(12).normal(0, 1, size=(1024, 2048)).astype(np.float32)
    logits = synth.zipf_routing_logits(79, 1024)
    _check_moe(full_layer, x, logits_in=logits, rows=range(0, 1024, 16), expect_kernel="moe_down_tc")


def test_moe_linearity_of_routed_part(full_layer):
    # size-independent property at full size: with the routing fixed by drawn logits, the expert FFN is positively
    # homogeneous only through SiLU, so check determinism and token-order invariance instead: permuting the batch
    # permutes the outputs bit-for-bit (grouping by expert must not leak between tokens)
    rng = np.random.default_rng(11)
    x = rng.normal(0, 1, size=(32, 2048)).astype(np.float32)
    logits = synth.zipf_routing_logits(78, 32)
    m = rc.MoeLayer(full_layer, max_tokens=32)
    try:
        a = m.forward(x, logits_in=logits)
        perm = rng.permutation(32)
        b = m.forward(x[perm], logits_in=logits[perm])
        a2 = m.forward(x, logits_in=logits)
    finally:
        m.close()
    assert np.array_equal(a, a2)
    assert np.array_equal(a[perm], b)


def _deltanet_inputs(seed, B, S=128, groups=16, rank=32, d_conv=4):
    rng = np.random.default_rng(seed)
    d_inner = rank * S
    channels = 2 * S * groups + d_inner
    p = dict(d_conv=d_conv, d_state=S, n_group=groups, dt_rank=rank, d_inner=d_inner, channels=channels, rms_eps=1e-6,
             conv_kernel=rng.normal(0, 0.5, size=(channels, d_conv)).astype(np.float32), dt_bias=np.zeros(rank, np.float32),
             ssm_a=-np.ones(rank, np.float32), ssm_norm=(1 + rng.normal(0, 0.1, S)).astype(np.float32))
    qkv = rng.normal(0, 1, size=(B, channels)).astype(np.float32)
    z = rng.normal(0, 1, size=(B, d_inner)).astype(np.float32)
    ba = rng.normal(0, 1, size=(B, 2 * rank)).astype(np.float32)
    conv = rng.normal(0, 1, size=(B, channels, d_conv - 1)).astype(np.float32)
    rec = rng.normal(0, 0.05, size=(B, rank, S, S)).astype(np.float32)
    return p, qkv, z, ba, conv, rec


@pytest.mark.parametrize("B", [1, 8])
@pytest.mark.parametrize("shape", [(128, 16, 32), (64, 2, 4)])
def test_deltanet_step(B, shape):
    S, groups, rank = shape
    p, qkv, z, ba, conv, rec = _deltanet_inputs(40 + B, B, S, groups, rank)
    conv_g, rec_g = conv.copy(), rec.copy()
    out = None
    for step in range(3):          # three steps: the conv window and the state carry over
        qs = np.roll(qkv, step, axis=1)
        out = rc.deltanet_step(p, qs, z, ba, conv_g, rec_g)
        for b in range(B):
            ref = ol.deltanet_mid(p, qs[b], z[b], ba[b], conv[b], rec[b])
            # tolerances of the reference's stage tools (native/redlite_native_deltanet_state_cli.c:267-269)
            assert np.all(np.abs(rec_g[b] - rec[b]) <= 3e-6 + 3e-5 * np.abs(rec[b])), (step, b)
            assert np.array_equal(conv_g[b], conv[b])
            assert np.max(np.abs(out[b] - ref)) <= REL_OUT * np.max(np.abs(ref)), (step, b)


def test_ep_pieces_single_rank_match_fused_forward(full_layer):
    """route / experts / shared / combine device entry points (the expert-parallel halves) chained on one GPU with the
    dispatch plan of ep.py must equal the fused forward (same kernels; the shared part is rounded once more on its way
    through its own buffer, hence a few ulp)."""
    import torch
    from dwarfstar_red_lite_b200 import ep
    rng = np.random.default_rng(12)
    T = 24
    x = rng.normal(0, 1, size=(T, 2048)).astype(np.float32)
    logits = synth.zipf_routing_logits(79, T)
    m = rc.MoeLayer(full_layer, max_tokens=T)
    try:
        want = m.forward(x, logits_in=logits)
        dev = torch.device("cuda", 0)
        xd, ld = torch.from_numpy(x).to(dev), torch.from_numpy(logits).to(dev)
        out = torch.empty(T, 2048, device=dev)
        layer = ep.EpMoeLayer(m, 0, 1, T)
        layer.forward(xd, out, logits=ld)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
    finally:
        m.close()
    assert np.max(np.abs(got - want)) <= 2e-6 * np.max(np.abs(want))


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_ep_gather_form_shards_sum_to_fused_forward(full_layer, world):
    """The all-gather form of expert parallelism, its ranks emulated one after the other on one GPU: `world` shards with
    interleaved experts (expert e on shard e % world) each compute the partial sums of their own experts over every
    token; the partial sums plus the shared expert equal the fused single-GPU forward."""
    import torch
    rng = np.random.default_rng(31 + world)
    T = 40
    x = rng.normal(0, 1, size=(T, 2048)).astype(np.float32)
    logits = synth.zipf_routing_logits(91, T)
    full = rc.MoeLayer(full_layer, max_tokens=T)
    try:
        want, ids, w, _ = full.forward(x, logits_in=logits, want_routing=True)
    finally:
        full.close()
    dev = torch.device("cuda", 0)
    d = full_layer.dims
    width = d.hidden + 2 * d.top_k
    packed = torch.zeros(T, width, device=dev)
    packed[:, :d.hidden] = torch.from_numpy(x).to(dev)
    packed[:, d.hidden:d.hidden + d.top_k] = torch.from_numpy(ids.view(np.float32)).to(dev)
    packed[:, d.hidden + d.top_k:] = torch.from_numpy(w).to(dev)
    total = torch.zeros(T, d.hidden, device=dev)
    part = torch.empty(T, d.hidden, device=dev)
    shared = torch.empty(T, d.hidden, device=dev)
    for r in range(world):
        m = rc.MoeLayer(full_layer, max_tokens=T, expert_begin=r, expert_stride=world)
        try:
            base = packed.data_ptr()
            m.partial_device(T, base, width, base + 4 * d.hidden, base + 4 * (d.hidden + d.top_k), width, part.data_ptr(), 0)
            if r == 0:
                xd = packed[:, :d.hidden].contiguous()
                m.shared_device(T, xd.data_ptr(), shared.data_ptr(), 0)
            torch.cuda.synchronize()
            total += part
        finally:
            m.close()
    got = (total + shared).cpu().numpy()
    assert np.max(np.abs(got - want)) <= 4e-6 * np.max(np.abs(want))


def test_ep_gather_layer_single_rank_matches_fused_forward(full_layer):
    """EpGatherMoeLayer.forward with one rank (no collectives): routing, packing, partial sums, the shared expert on its
    side stream and the final add must reproduce the fused forward."""
    import torch
    from dwarfstar_red_lite_b200 import ep
    rng = np.random.default_rng(17)
    T = 24
    x = rng.normal(0, 1, size=(T, 2048)).astype(np.float32)
    logits = synth.zipf_routing_logits(83, T)
    m = rc.MoeLayer(full_layer, max_tokens=T)
    try:
        want = m.forward(x, logits_in=logits)
        dev = torch.device("cuda", 0)
        layer = ep.EpGatherMoeLayer(m, 0, 1, T)
        for _ in range(2):       # twice: buffers and the side stream are reused
            got = layer.forward(torch.from_numpy(x).to(dev), logits=torch.from_numpy(logits).to(dev))
            torch.cuda.synchronize()
            assert np.max(np.abs(got.cpu().numpy() - want)) <= 4e-6 * np.max(np.abs(want))
    finally:
        m.close()


def test_ep_step_call_single_rank_matches_fused_forward(full_layer):
    """redcuda_ep_step with one rank (no NCCL): the library's own step call over two layer objects reproduces the fused
    forward of each layer on its own input."""
    import torch
    from dwarfstar_red_lite_b200 import ep
    rng = np.random.default_rng(18)
    T = 24
    x = rng.normal(0, 1, size=(2, T, 2048)).astype(np.float32)
    logits = np.stack([synth.zipf_routing_logits(84 + l, T) for l in range(2)])
    shards = [rc.MoeLayer(full_layer, max_tokens=T) for _ in range(2)]
    ctx = None
    try:
        want = [shards[l].forward(x[l], logits_in=logits[l]) for l in range(2)]
        dev = torch.device("cuda", 0)
        ctx = ep.EpStep(shards, 0, 1, T)
        ctx.bind(torch.from_numpy(x).to(dev), torch.from_numpy(logits).to(dev))
        for _ in range(2):
            got = ctx.step()
            torch.cuda.synchronize()
            for l in range(2):
                assert np.max(np.abs(got[l].cpu().numpy() - want[l])) <= 4e-6 * np.max(np.abs(want[l]))
    finally:
        if ctx:
            ctx.close()
        for m in shards:
            m.close()
