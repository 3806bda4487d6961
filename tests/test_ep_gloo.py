"""Expert-parallel host logic on CPU: two gloo ranks, experts sharded 8 + 8, tokens stay with their rank. The dispatch
plan, both all-to-all exchanges and the per-token combine of dwarfstar_red_lite_b200/ep.py must reproduce the
single-process MoE layer; the expert arithmetic on either side of the exchange is played by the CPU oracle here."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _layer_and_inputs():
    from dwarfstar_red_lite_b200 import synth
    dims = synth.MoeDims(hidden=256, n_expert=16, top_k=4, ffn=256, ffn_sh=256)
    layer = synth.moe_layer(5, dims, expert_scale=0.5)
    rng = np.random.default_rng(6)
    x = rng.normal(0, 1, size=(2, 5, dims.hidden)).astype(np.float32)        # [rank][token][hidden]
    return dims, layer, x


def _worker(rank, world, port, q):
    for p in (ROOT, HERE):
        if p not in sys.path:
            sys.path.insert(0, p)
    import oracle_lib as ol
    from dwarfstar_red_lite_b200 import ep
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dims, layer, x_all = _layer_and_inputs()
        x = torch.from_numpy(x_all[rank])
        T, k = x.shape[0], dims.top_k
        ids = np.empty((T, k), np.int64)
        w = np.empty((T, k), np.float32)
        shared = np.empty((T, dims.hidden), np.float32)
        full = np.empty((T, dims.hidden), np.float32)
        for t in range(T):
            full[t], i_, w_, _ = ol.moe_ffn(layer, x_all[rank][t])
            ids[t], w[t] = i_, w_
            routed = ol.routed_experts(layer, i_, w_, x_all[rank][t])
            shared[t] = (full[t].astype(np.float64) - routed).astype(np.float32)
        lo, hi = rank * dims.n_expert // world, (rank + 1) * dims.n_expert // world
        seen = []

        def experts_fn(px, pe):
            out = np.empty((px.shape[0], dims.hidden), np.float32)
            for i in range(px.shape[0]):
                e = int(pe[i])
                assert lo <= e < hi, "a pair reached the wrong shard"
                seen.append(e)
                out[i] = ol.routed_experts(layer, np.array([e], np.uint32), np.array([1.0], np.float32), px[i].numpy()).astype(np.float32)
            return torch.from_numpy(out)

        def combine_fn(back, pair_row, weights, add):
            out = add.clone()
            for t in range(T):
                for kk in range(k):
                    out[t] += weights[t, kk] * back[int(pair_row[t * k + kk])]
            return out

        out, plan = ep.ep_moe_forward(x, torch.from_numpy(ids), torch.from_numpy(w), dims.n_expert, world, experts_fn,
                                      lambda xx: torch.from_numpy(shared), combine_fn)
        err = float(np.max(np.abs(out.numpy() - full)) / np.max(np.abs(full)))
        q.put((rank, err, sum(plan.send_counts), sum(plan.recv_counts), len(seen)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_ep_two_ranks_gloo_matches_single_process():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    sent = sum(r[2] for r in res)
    recv = sum(r[3] for r in res)
    assert sent == recv == 2 * 5 * 4                       # every pair crossed the exchange exactly once
    for rank, err, s, r, n in res:
        assert err <= 1e-5, (rank, err)
        assert n == r


def _gather_worker(rank, world, port, q):
    for p in (ROOT, HERE):
        if p not in sys.path:
            sys.path.insert(0, p)
    import oracle_lib as ol
    from dwarfstar_red_lite_b200 import ep
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dims, layer, x_all = _layer_and_inputs()
        T, k, H = x_all.shape[1], dims.top_k, dims.hidden
        packed = np.zeros((T, H + 2 * k), np.float32)
        full = np.empty((T, H), np.float32)
        shared = np.empty((T, H), np.float32)
        for t in range(T):
            full[t], i_, w_, _ = ol.moe_ffn(layer, x_all[rank][t])
            routed = ol.routed_experts(layer, i_, w_, x_all[rank][t])
            shared[t] = (full[t].astype(np.float64) - routed).astype(np.float32)
            packed[t, :H] = x_all[rank][t]
            packed[t, H:H + k] = np.asarray(i_, np.uint32).view(np.float32)
            packed[t, H + k:] = w_
        ran = []

        def partial_fn(allp):
            a = allp.numpy()
            out = np.zeros((a.shape[0], H), np.float32)
            for t in range(a.shape[0]):
                ids, w = a[t, H:H + k].view(np.uint32), a[t, H + k:]
                for kk in range(k):
                    if int(ids[kk]) % world == rank:             # interleaved placement: expert e on rank e % world
                        ran.append(int(ids[kk]))
                        out[t] += (w[kk] * ol.routed_experts(layer, ids[kk:kk + 1].copy(), np.array([1.0], np.float32), a[t, :H].copy())).astype(np.float32)
            return torch.from_numpy(out)

        out = ep.gather_moe_forward(torch.from_numpy(packed), H, k, world, partial_fn, lambda pk: torch.from_numpy(shared.copy()))
        err = float(np.max(np.abs(out.numpy() - full)) / np.max(np.abs(full)))
        q.put((rank, err, len(ran)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_ep_gather_form_two_ranks_gloo_matches_single_process():
    """all-gather of the token rows, per-rank partial sums over the rank's interleaved experts, reduce-scatter back"""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_gather_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sum(r[2] for r in res) == 2 * 5 * 4             # every pair ran on exactly one rank
    for rank, err, n in res:
        assert err <= 1e-5, (rank, err)


def test_plan_dispatch_single_rank_is_identity_permutation():
    from dwarfstar_red_lite_b200 import ep
    ids = torch.tensor([[3, 1], [0, 2], [1, 3]])
    plan = ep.plan_dispatch(ids, 4, 1)
    assert plan.send_counts == [6] and plan.recv_counts == [6]
    assert torch.equal(plan.order, torch.arange(6)) and torch.equal(plan.inverse, torch.arange(6))
